"""End-to-end Qwen3 MoE driver for the JSON-driven training-DAG runtime (run through ``examples/test_harness.py``)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples.common import add_common_args, derive_num_stages, run_driver  # noqa: E402
from piper_b200.models.qwen3 import QWEN3_CONFIGS, PiperQwen3Model  # noqa: E402
from piper_b200.nn import cross_entropy_loss  # noqa: E402


def main(args, pg=None):
    cfg = QWEN3_CONFIGS[args.model]
    num_stages = int(getattr(args, "num_stages", 0) or derive_num_stages(args.schedule_directives_file))
    return run_driver(args, PiperQwen3Model, (cfg, num_stages, args.seq_len), cfg, cross_entropy_loss,
                      PiperQwen3Model.const_attrs(cfg, args.seq_len))


_derive_num_stages = derive_num_stages


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Test JSON-driven Qwen TrainingDAG execution")
    p.add_argument("--model", choices=sorted(QWEN3_CONFIGS), default="9M")
    add_common_args(p, "examples/base-schedules/pp2_dp2_ep2.json")
    return p.parse_args(argv)
