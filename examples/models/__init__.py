"""Model definitions used by the example drivers (the implementations live in ``piper_b200.models``)."""
