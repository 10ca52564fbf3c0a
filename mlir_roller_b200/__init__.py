"""roller_b200: the Roller rTile search driving GEMM kernels written for NVIDIA B200 (fp32
operands through TF32 / 3xTF32, and bf16 / fp16 operands for 16-bit problem descriptors).

Modules mirror the reference project's layout: `arch` (device models), `utils`, `analyze`
(the search), `roller` (compile / launch / time), `benchmark` (the sweep), plus `mgpu` (output
sharding across the GPUs of one node) and `_lib` (ctypes binding of libroller_b200.so).
"""
from .analyze import (MODE_1XTF32, MODE_3XTF32, MODE_BF16, MODE_F16, MatmulConfig,  # noqa: F401
                      TileDict, get_roller_hints)
from .arch import B200, CUDA, TileDevice  # noqa: F401

__all__ = ["MatmulConfig", "TileDict", "get_roller_hints", "B200", "CUDA", "TileDevice",
           "MODE_1XTF32", "MODE_3XTF32", "MODE_BF16", "MODE_F16"]
