"""``src.visualization`` of the reference, provided by ``piper_b200.compiler.viz``."""
from piper_b200.compiler.viz import (log_training_dag_dependencies, print_training_dag_order,  # noqa: F401
                                     render_training_dag, visualize_order_directives)
