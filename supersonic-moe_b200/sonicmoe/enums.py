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


# codes the kernels take: the GEMM epilogues carry 0 (SwiGLU, the precise sigmoid form); 1 and 2 run through plain
# GEMMs + the stand-alone activation kernels
ACTIVATION_CODES = {ActivationType.SWIGLU: 0, ActivationType.SWIGLU_PRECISE: 0, ActivationType.REGLU: 1,
                    ActivationType.GEGLU: 2}


def activation_code(activation_type) -> int:
    """0 swiglu, 1 reglu, 2 geglu; everything else (SiTU-GLU, the non-gated activations) is not built."""
    if isinstance(activation_type, str):
        activation_type = ActivationType(activation_type.split(":", 1)[0])
    if activation_type not in ACTIVATION_CODES:
        raise NotImplementedError(f"activation {activation_type} is outside the MXFP8 gated-activation path of this "
                                  "build (SwiGLU, ReGLU, GEGLU)")
    return ACTIVATION_CODES[activation_type]


def require_swiglu(activation_type):
    """Kept for callers that need the fused path specifically."""
    if activation_code(activation_type) != 0:
        raise NotImplementedError(f"activation {activation_type}: only SwiGLU has fused GEMM epilogues")
    return activation_type
