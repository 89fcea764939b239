"""B200 (sm_100a) implementation of the Elleci BitNet INT2 linear hot path.

Host side: PyTorch modules with the reference's BitLinear / Int2LinearTC / int2_tc_ops interface.
Compute: hand-written CUDA behind a C ABI (include/elleci_int2.h, csrc/), loaded with ctypes.
"""
from . import _lib, checkpoint, int2_tc_ops, sharded, token_parallel
from ._lib import LIB_PATH, ElleciError
from .bitnet_int2_optimized import (BitLinearInt2, SwiGLUFFNInt2, convert_all_linear_to_int2, disable_hysteresis, enable_hysteresis,
                                    get_int2_layers, get_non_int2_params, set_all_int2_lr)
from .int2_linear_tc import (Int2LinearTC, Int2LinearTCFunction, Int2LinearTCOffload, Int2LinearTCOffloadWithGradHook,
                             Int2LinearTCWithGradHook)

__all__ = [
    "int2_tc_ops", "sharded", "token_parallel", "checkpoint", "LIB_PATH", "ElleciError", "BitLinearInt2", "SwiGLUFFNInt2", "convert_all_linear_to_int2", "enable_hysteresis",
    "disable_hysteresis", "get_int2_layers", "get_non_int2_params", "set_all_int2_lr", "Int2LinearTC",
    "Int2LinearTCFunction", "Int2LinearTCWithGradHook", "Int2LinearTCOffload", "Int2LinearTCOffloadWithGradHook",
]
