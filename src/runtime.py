"""``src.runtime`` of the reference: flat parameter storage and rank layout of this runtime."""
from piper_b200.runtime.layout import ProcessGroups, RankLayout, make_layout  # noqa: F401
from piper_b200.runtime.storage import AdamConfig, ParamSlot, ParamStorage  # noqa: F401
