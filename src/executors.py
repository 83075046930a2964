"""``src.executors`` of the reference: one ``DagExecutor`` covers the compute and communication executors."""
from piper_b200.runtime.actor import DagExecutor  # noqa: F401
from piper_b200.runtime.faults import FaultInjector, InjectedFault, parse_fault_spec  # noqa: F401
