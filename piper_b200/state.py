"""Process-wide state and logging.

``piper_metadata`` is the singleton the compile driver and the step driver
share (schedule, per-device DAGs, the local actor); ``create_logger`` gives
every module the same stdout format as the reference (``src/state.py``).
"""
from __future__ import annotations

import logging
import os
import sys
from typing import Any, Optional

LOG_LEVEL = os.environ.get("PIPER_LOG_LEVEL", "INFO")


def create_logger(name: str, log_level: str = LOG_LEVEL) -> logging.Logger:
    level = getattr(logging, str(log_level).upper(), logging.INFO)
    logger = logging.getLogger(name)
    logger.setLevel(level)
    if not logger.handlers:
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(logging.Formatter("%(asctime)s - %(name)s - %(levelname)s - %(message)s"))
        logger.addHandler(h)
        logger.propagate = False
    return logger


class PiperMetadata:
    """What one process knows about the compiled program."""

    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        self.actors: dict = {}                 # pp_rank -> PiperActor (this process holds exactly one)
        self.visualize_dag: bool = False
        self.artifact_dir: str = "out"
        self.training_dag = None               # global DAG after directive rewrites
        self.per_pp_training_dags = None       # one DAG per device set, sorted by device tuple
        self.schedule_directives: list = []
        self.schedule_directives_file: Optional[str] = None
        self.schedule_info: dict[str, Any] = {}
        self.tokens_per_step: Optional[int] = None
        self.segments = None


piper_metadata = PiperMetadata()
