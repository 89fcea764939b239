"""ctypes loaders for the oracle's native checkers (TEST INFRASTRUCTURE ONLY).

* `oracle_lib()`  -> oracle/_build/liboracle.so, the C restatement (oracle/int2_oracle.c)
* `ref_cpu_lib()` -> oracle/_ref/libref_cpu.so, the reference's own kernel sources compiled for the
                     host by oracle/build_ref.sh (None when it has not been built)
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")


def build_oracle_lib() -> str:
    """Compile oracle/int2_oracle.c (make) and return the library path."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True, env={**os.environ, "GCC": os.environ.get("ORACLE_GCC", "/usr/bin/gcc")})
    return os.path.join(_HERE, "_build", "liboracle.so")


_oracle = None
_ref = None


def oracle_lib():
    global _oracle
    if _oracle is None:
        path = os.path.join(_HERE, "_build", "liboracle.so")
        if not os.path.exists(path):
            path = build_oracle_lib()
        lib = C.CDLL(path)
        lib.oracle_num_threads.restype = C.c_int
        lib.oracle_hysteresis_step.argtypes = [_f32p, _u8p, _u8p, C.c_float, C.c_float, C.c_int, C.c_float,
                                               C.c_uint32, C.c_int, C.c_int, C.c_uint32, C.c_int]
        lib.oracle_quantize_rows.argtypes = [_f32p, _i8p, _f32p, C.c_int, C.c_int, C.c_float]
        lib.oracle_unpack_ternary.argtypes = [_u8p, _i8p, C.c_int, C.c_int]
        lib.oracle_gemm_nt_i8.argtypes = [_i8p, _i8p, _i32p, C.c_int, C.c_int, C.c_int]
        lib.oracle_gemm_tn_i8.argtypes = [_i8p, _i8p, _i32p, C.c_int, C.c_int, C.c_int]
        _oracle = lib
    return _oracle


def ref_cpu_lib():
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref_cpu.so")
        if not os.path.exists(path):
            return None
        lib = C.CDLL(path)
        lib.ref_hysteresis_v2_cpu.argtypes = [_f32p, _u8p, _u8p, C.c_float, C.c_float, C.c_int, C.c_float,
                                              C.c_int, C.c_int, C.c_int, C.c_int]
        lib.ref_quantize_tensor_cpu.argtypes = [_u16p, _i8p, _f32p, C.c_int, C.c_int]
        lib.ref_dequantize_tensor_cpu.argtypes = [_i8p, _u16p, _f32p, C.c_int]
        _ref = lib
    return _ref


def c_hysteresis_step(dW, W_packed, H_packed, lr, lr_scale, threshold, decay, step, K, idx_base=0, ftz=True):
    """C restatement; returns new (W_packed, H_packed) copies."""
    W = np.ascontiguousarray(W_packed, dtype=np.uint8).copy()
    H = np.ascontiguousarray(H_packed, dtype=np.uint8).copy()
    dW = np.ascontiguousarray(dW, dtype=np.float32)
    oracle_lib().oracle_hysteresis_step(dW, W, H, lr, lr_scale, int(threshold), decay, int(step) & 0xFFFFFFFF,
                                        dW.shape[0], K, int(idx_base) & 0xFFFFFFFF, int(bool(ftz)))
    return W, H


def ref_hysteresis_step(dW, W_packed, H_packed, lr, lr_scale, threshold, decay, step, K, ftz=True):
    """The reference kernel source run on the host; returns new (W_packed, H_packed) copies.
    The buffers are padded to a multiple of 4 bytes because the kernel's 32-bit read-modify-writes
    touch the whole word that holds a field."""
    lib = ref_cpu_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libref_cpu.so not built (run oracle/build_ref.sh)")
    dW = np.ascontiguousarray(dW, dtype=np.float32)
    N = dW.shape[0]

    def padded(a):
        flat = np.ascontiguousarray(a, dtype=np.uint8).reshape(-1)
        buf = np.zeros((flat.size + 7) // 4 * 4, dtype=np.uint8)
        buf[: flat.size] = flat
        return buf

    W, H = padded(W_packed), padded(H_packed)
    lib.ref_hysteresis_v2_cpu(dW, W, H, lr, lr_scale, int(threshold), decay, int(step), N, K, int(bool(ftz)))
    return (W[: W_packed.size].reshape(W_packed.shape).copy(), H[: H_packed.size].reshape(H_packed.shape).copy())


def c_sigmoid_fixed(g):
    """sigmoid(g) in float32 with the fixed polynomial exponential (oracle/int2_oracle.c: exp_fixed)."""
    g = np.ascontiguousarray(g, dtype=np.float32)
    out = np.empty_like(g)
    lib = oracle_lib()
    lib.oracle_sigmoid_fixed.argtypes = [_f32p, _f32p, C.c_longlong]
    lib.oracle_sigmoid_fixed(g.reshape(-1), out.reshape(-1), g.size)
    return out
