"""Enums of the reference API (sonicmoe/enums.py:12-50)."""
from enum import Enum

LIBRARY_NAME = "sonicmoe"


class KernelBackendMoE(Enum):
    scattermoe = "scattermoe"
    torch = "torch"
    sonicmoe = "sonicmoe"


class ActivationType(Enum):
    SWIGLU = "swiglu"
    SWIGLU_PRECISE = "swiglu_precise"
    GEGLU = "geglu"
    REGLU = "reglu"
    SITU_GLU = "situ_glu"
    RELU_SQ = "relu_sq"
    RELU = "relu"
    GELU = "gelu"
    SILU = "silu"


def is_glu(activation_type) -> bool:
    return activation_type in (ActivationType.SWIGLU, ActivationType.REGLU, ActivationType.GEGLU,
                               ActivationType.SWIGLU_PRECISE, ActivationType.SITU_GLU)


def require_swiglu(activation_type):
    """The sm_100a kernels implement SwiGLU (the precise sigmoid form) only."""
    if isinstance(activation_type, str):
        activation_type = ActivationType(activation_type)
    if activation_type not in (ActivationType.SWIGLU, ActivationType.SWIGLU_PRECISE):
        raise NotImplementedError(f"activation {activation_type} is outside the MXFP8 SwiGLU hot path of this build")
    return activation_type
