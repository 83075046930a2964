"""``src.fx`` of the reference, provided by ``piper_b200.compiler.fxsplit``."""
from piper_b200.compiler.fxsplit import (PIPER_ANNOTATIONS_META_KEY, AnnotationSegment,  # noqa: F401
                                         split_gm_by_annotations)
