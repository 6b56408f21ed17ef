"""B200-native (sm_100a) implementation of the SonicMoE MoE layer forward and
backward behind the reference's `sonicmoe` module / functional API."""
from . import _lib  # noqa: F401  (raises if libsmoe_b200.so is missing)
from . import ops  # noqa: F401
