"""Example programs: harness, Llama and Qwen drivers, schedule builders, base schedules."""
