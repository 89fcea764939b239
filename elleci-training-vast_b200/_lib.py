"""ctypes binding of libelleci_int2.so, the C-ABI CUDA library (include/elleci_int2.h).

The library is the only compute path: there is no CPU or eager fallback.  Importing this module on a
machine where the library has not been built raises at first use (`lib()`), with the build command.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# ELLECI_INT2_LIB points at another build of the same library (a debug or experimental build)
LIB_PATH = os.environ.get("ELLECI_INT2_LIB") or os.path.join(_HERE, "lib", "libelleci_int2.so")

EL_OK = 0
EL_ERR_INVALID_ARG, EL_ERR_NULL_PTR, EL_ERR_ALIGNMENT, EL_ERR_UNSUPPORTED_SHAPE = -1, -2, -3, -4
EL_ERR_CUDA, EL_ERR_DEVICE, EL_ERR_DRIVER, EL_ERR_TOO_LARGE = -5, -6, -7, -8
EL_F16, EL_BF16, EL_F32, EL_I32 = 0, 1, 2, 3
EL_PATH_AUTO, EL_PATH_SIMPLE, EL_PATH_TC, EL_PATH_TC_SINGLE = 0, 1, 2, 3
EL_FLAG_LEAN = 0x100
EL_QUANT_FULL, EL_QUANT_ABSMAX_ONLY, EL_QUANT_WITH_ABSMAX = 0, 1, 2

_vp, _i, _f, _ll, _u32 = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_uint32

#: name -> argtypes, exactly the declarations of include/elleci_int2.h
SIGNATURES = {
    "el_version": [],
    "el_status_string": [_i],
    "el_last_cuda_error": [],
    "el_pack_ternary": [_vp, _vp, _i, _i, _i, _vp],
    "el_ternarize_pack": [_vp, _f, _vp, _i, _i, _vp],
    "el_unpack_ternary": [_vp, _vp, _i, _i, _i, _vp],
    "el_quantize_rows": [_vp, _i, _ll, _vp, _vp, _i, _i, _f, _i, _vp, _vp, _vp],
    "el_quantize_tensor": [_vp, _i, _vp, _vp, _ll, _vp],
    "el_dequantize_tensor": [_vp, _vp, _vp, _i, _ll, _vp],
    "el_quantize_grad": [_vp, _i, _ll, _vp, _vp, _vp, _i, _i, _vp],
    "el_scale_rows": [_vp, _vp, _i, _vp, _i, _f, _i, _i, _vp],
    "el_gemm_fwd": [_vp, _vp, _vp, _i, _vp, _i, _f, _i, _i, _i, _i, _vp, _vp],
    "el_gemm_workspace_bytes": [_i, _i, _i, _i],
    "el_gemm_fwd_ws": [_vp, _vp, _vp, _i, _vp, _i, _f, _i, _i, _i, _i, _vp, C.c_size_t, _vp, _vp],
    "el_gemm_dx_ws": [_vp, _vp, _vp, _i, _vp, _i, _f, _i, _i, _i, _i, _vp, C.c_size_t, _vp, _vp],
    "el_gemm_fwd_gather": [_vp, _vp, _vp, _i, _ll, _ll, _i, _vp, _i, _f, _i, _i, _i, _vp, _vp],
    "el_gemm_dx_scatter": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "el_reduce_scale_gather": [_vp, _vp, _i, _i, _i, _vp, _f, _i, _i, _vp],
    "el_gemm_dx": [_vp, _vp, _vp, _i, _vp, _i, _f, _i, _i, _i, _i, _vp, _vp],
    "el_gemm_dw": [_vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _vp],
    "el_decode_workspace_bytes": [_i],
    "el_rmsnorm_quantize_rows": [_vp, _i, C.c_longlong, _vp, _f, _vp, _vp, _vp, _i, _i, _f, _vp],
    "el_rmsnorm_backward_workspace_bytes": [_i],
    "el_swiglu_quantize_rows": [_vp, _vp, _i, C.c_longlong, _vp, _f, _vp, _vp, _vp, _i, _i, _f, _vp],
    "el_swiglu_backward_workspace_bytes": [_i],
    "el_sigmoid_fixed": [_vp, _vp, C.c_longlong, _vp],
    "el_prelinear_rows": [_vp, _vp, _i, C.c_longlong, _vp, _f, _vp, _i, _i, _vp],
    "el_swiglu_backward": [_vp, _vp, _vp, _i, C.c_longlong, _vp, _vp, _vp, _vp, C.c_longlong, _vp, _vp, C.c_size_t, _i, _i, _vp],
    "el_rmsnorm_backward": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _i, _i, _vp],
    "el_set_decode_gemv_max_tokens": [_i],
    "el_set_decode_overlap": [_i],
    "el_peer_barrier": [_vp, _i, _i, _u32, _vp, _vp],
    "el_peer_barrier_put": [_vp, _i, _i, _u32, _vp, _vp, _vp, C.c_size_t, _vp],
    "el_set_decode_mma_max_tokens": [_i],
    "el_set_peer_barrier_limit_us": [_ll],
    "el_peer_put": [_vp, _vp, _i, C.c_size_t, C.c_size_t, _i, _vp],
    "el_quantize_grad_scatter": [_vp, _i, _ll, _vp, _vp, _i, _vp, _vp, _i, _ll, _i, _i, _vp],
    "el_linear_decode": [_vp, _i, _vp, _vp, _i, _f, _vp, _vp, _vp, C.c_size_t, _i, _i, _i, _vp, _vp],
    "el_linear_decode_static": [_vp, _i, _vp, _vp, _i, _f, _i, _i, _i, _vp, _vp],
    "el_hysteresis_from_dw": [_vp, _vp, _vp, _f, _f, _i, _f, _i, _i, _i, _u32, _i, _vp],
    "el_dw_hysteresis": [_vp, _vp, _vp, _vp, _vp, _f, _f, _i, _f, _i, _u32, _i, _i, _i, _vp, _vp],
    "el_dw_hysteresis_step_ptr": [_vp, _vp, _vp, _vp, _vp, _f, _f, _i, _f, _vp, _u32, _i, _i, _i, _vp, _vp],
    "el_peer_barrier_next": [_vp, _i, _i, _vp, _vp, _vp, C.c_size_t, _vp],
    "el_counter_add": [_vp, _i, _vp],
    "el_peer_put_dma": [_vp, _vp, _i, C.c_size_t, C.c_size_t, _vp],
}


class ElleciError(RuntimeError):
    """A library call returned a non-zero status (the reference's wrappers raise RuntimeError too)."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: {detail} (status {status})")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ElleciError("load", EL_ERR_DEVICE,
                              f"{LIB_PATH} is missing: build it with `python elleci-training-vast_b200/build.py` "
                              "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = (C.c_char_p if name == "el_status_string" else
                          C.c_size_t if name in ("el_decode_workspace_bytes", "el_rmsnorm_backward_workspace_bytes", "el_swiglu_backward_workspace_bytes",
                                                "el_gemm_workspace_bytes") else C.c_int)
        _lib = handle
    return _lib


def check(fn: str, status: int) -> None:
    if status != EL_OK:
        handle = lib()
        detail = handle.el_status_string(status).decode()
        if status == EL_ERR_CUDA:
            detail += f" (cudaError {handle.el_last_cuda_error()})"
        raise ElleciError(fn, status, detail)


def call(name: str, *args) -> None:
    check(name, getattr(lib(), name)(*args))
