"""Import-compatibility package: ``from src.piper import annotate`` keeps working for programs written for the reference."""
