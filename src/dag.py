"""``src.dag`` of the reference, provided by ``piper_b200.compiler.dag``."""
from piper_b200.compiler.dag import *  # noqa: F401,F403
from piper_b200.compiler.dag import (TrainingDAG, TrainingDAGEdge, TrainingDAGNode, _has_path,  # noqa: F401
                                     _topological_levels, _topological_order, build_training_dag)
