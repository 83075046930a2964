"""``src.bucket`` of the reference, provided by ``piper_b200.compiler.bucket``."""
from piper_b200.compiler.bucket import bucket_stage, plan_buckets  # noqa: F401
