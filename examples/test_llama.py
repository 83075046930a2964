"""End-to-end Llama driver for the JSON-driven training-DAG runtime (run through ``examples/test_harness.py``)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples.common import add_common_args, derive_num_stages, run_driver  # noqa: E402
from piper_b200.models.llama3 import LLAMA_CONFIGS, Transformer  # noqa: E402
from piper_b200.nn import cross_entropy_loss  # noqa: E402


def main(args, pg=None):
    cfg = LLAMA_CONFIGS[args.model]
    num_stages = int(getattr(args, "num_stages", 0) or derive_num_stages(args.schedule_directives_file))
    return run_driver(args, Transformer, (cfg, args.seq_len, num_stages), cfg, cross_entropy_loss,
                      Transformer.const_attrs(cfg, args.seq_len))


_derive_num_stages = derive_num_stages


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Test JSON-driven Llama TrainingDAG execution")
    p.add_argument("--model", choices=sorted(LLAMA_CONFIGS), default="debug")
    p.add_argument("--num-checkpoints", type=int, default=1)
    add_common_args(p, "examples/base-schedules/dp2.json")
    return p.parse_args(argv)
