"""B200-native (sm_100a) implementation of the SonicMoE MoE layer forward and
backward behind the reference's `sonicmoe` module / functional API
(sonicmoe/__init__.py:68-101).  Importing this package loads libsmoe_b200.so and
raises if it is missing - there is no fallback path."""
__version__ = "0.1.0"

from . import _lib  # noqa: F401
from . import ops  # noqa: F401
from .config import SonicMoEConfig, get_active_config, set_active_config  # noqa: F401
from .count_cumsum import count_cumsum  # noqa: F401
from .enums import ActivationType, KernelBackendMoE  # noqa: F401
from .ernie_compat.deepep_metadata import deepep_topk_to_sonic_metadata  # noqa: F401
from .functional import (  # noqa: F401
    _DownProjection,
    _UpProjection,
    clear_weight_cache,
    drop_weight_fp8,
    enable_fp8,
    enable_quack_gemm,
    general_routing_router_metadata,
    moe_general_routing_inputs,
    moe_TC_softmax_topk_layer,
    precompute_weight_fp8,
)
from .interface import run_sonic_moe  # noqa: F401
from .moe import MoE  # noqa: F401
from .quack_utils import pack_blockscaled_1x32_scales  # noqa: F401
from .routing import token_rounding_routing  # noqa: F401
