"""`SonicMoEConfig`: thread-local configuration object of the reference API
(sonicmoe/config.py:149-300).  This build has one compute path - the MXFP8
frontier path - so the flags that selected other backends are accepted and
recorded but do not switch code paths."""
from __future__ import annotations

import os
import threading
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Optional

_tls = threading.local()


def _env_bool(name: str) -> bool:
    return os.getenv(name, "").strip().lower() in ("1", "true", "yes", "on")


def get_active_config() -> Optional["SonicMoEConfig"]:
    return getattr(_tls, "config", None)


def set_active_config(cfg: Optional["SonicMoEConfig"]) -> None:
    _tls.config = cfg


@dataclass
class SonicMoEConfig:
    use_fp8: Optional[bool] = None
    use_quack_gemm: Optional[bool] = None
    fp8_wgrad: Optional[bool] = None
    save_z_fp8: Optional[bool] = None
    recompute_z: Optional[bool] = None
    epilogue_quant: Optional[bool] = None
    fused_zy1_quant: Optional[bool] = None
    fuse_y1_quant: Optional[bool] = None
    fuse_y1_bf16_trunc: Optional[bool] = None
    fused_weight_layout: Optional[bool] = None
    assume_aligned: Optional[bool] = None
    stagewise_memory: Optional[bool] = None
    iso32_weight: Optional[bool] = None
    swiglu_clamp_value: Optional[float] = None

    def __post_init__(self) -> None:
        if self.use_fp8 is True and self.use_quack_gemm is None:
            self.use_quack_gemm = True
        if self.swiglu_clamp_value:
            raise NotImplementedError("swiglu_clamp_value is not built")

    def resolve_use_fp8(self) -> bool:
        return bool(self.use_fp8)

    def resolve_recompute_z(self) -> bool:
        """Drop z after the forward and regenerate it in the backward by re-running the up-projection GEMM
        (sonicmoe/config.py:154-170, functional/__init__.py:884-903,2047-2053 of the reference): trades one extra
        up-projection per step for TKp x 2I bytes (+ scales) of saved activations per layer."""
        return bool(self.recompute_z)

    def resolve_iso32_weight(self) -> bool:
        """One FP8 buffer per weight, quantised with one scale per 32x32 block and read in both orientations,
        instead of two 1x32 copies (sonicmoe/config.py:208-211; env SONIC_MOE_FP8_ISO32_WEIGHT, default off)."""
        if self.iso32_weight is not None:
            return bool(self.iso32_weight)
        return _env_bool("SONIC_MOE_FP8_ISO32_WEIGHT")

    def resolve_stagewise_memory(self) -> bool:
        """Memory-lean ordering of the backward (every operand is produced right before its one consumer and freed
        right after) plus a per-stage record of allocated / peak bytes (sonicmoe/config.py:203-206; env
        SONIC_MOE_STAGEWISE_MEMORY, default off)."""
        if self.stagewise_memory is not None:
            return bool(self.stagewise_memory)
        return _env_bool("SONIC_MOE_STAGEWISE_MEMORY")

    @contextmanager
    def activate(self):
        prev = get_active_config()
        set_active_config(self)
        try:
            yield self
        finally:
            set_active_config(prev)
