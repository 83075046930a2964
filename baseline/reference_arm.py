"""``bench.py --impl reference``.

The reference is installed with ``pip install --no-deps --target baseline/_ref`` (its packages are ``src`` and
``examples``).  Its public entry points (``src.compile.piper_setup``, ``src.piper.piper_exec_dag``,
``examples/test_harness.py``) import ``ray`` at module scope and create Ray actors, placement groups and named
actors to run; ``ray`` is not installed in this image and cannot be installed offline, so the stock code path
cannot start.  In that case this arm prints the ``unavailable`` line and exits 0.
"""
from __future__ import annotations

import importlib.util
import os


def run(args) -> dict:
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if not os.path.isdir(os.path.join(ref, "src")):
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed on this box"}
    if importlib.util.find_spec("ray") is None:
        return {"impl": "reference",
                "unavailable": "reference installs with --no-deps but its public API imports ray "
                               "(src/piper.py:5, src/compile.py:1, src/actor.py:1) and ray is not in this image"}
    return {"impl": "reference", "unavailable": "reference arm launcher for a Ray-enabled image is not implemented"}
