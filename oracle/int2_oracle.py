"""CPU oracle for the BitNet INT2 linear hot path (TEST INFRASTRUCTURE ONLY).

This module restates, in plain NumPy, the arithmetic of the reference's INT2 linear layer.
It is the checker the CUDA kernels are compared with; it is never on a product code path.
Only the tests, the smoke check and the benchmark's CPU-baseline leg may import it.

Every function names the reference file:line it follows (paths are relative to the
reference project root):

* 2-bit weight code and int4 counter code ........ kernels/int2/int2_packed.cuh:9-86
* host packers ................................... core/bitnet/int2_linear_tc.py:414-436,
                                                   kernels/tests/kernel_build.py:69-90
* absmean ternarisation .......................... core/bitnet/int2_linear_tc.py:391-412,
                                                   model/common/bitnet_legacy.py:89-118
* per-token absmax int8 quantisation ............. model/common/bitnet_legacy.py:58-87
* per-tensor absmax int8 quantisation ............ kernels/int2/int2_activation_quant.cu:88-167
* forward / dX integer GEMMs and their epilogue .. kernels/int2/int2_matmul_int8_tc_v2.cu:118-121,261
                                                   kernels/int2/int2_backward_int8_tc_v2.cu:88-92,233
* hysteresis update .............................. kernels/int2/int2_hysteresis_v2.cu:54-152
* SwiGLU gate (silu(w1 x) * w2 x) ................ model/model.py:86-108
* pre-linear RMSNorm ............................. core/bitnet/bitnet_int2_optimized.py:72-86,
                                                   model/common/bitnet_legacy.py:10-25

Parity status: packing, ternarisation and per-token quantisation are pinned against the
reference's own Python code (imported from the reference tree by tests/golden/make_golden.py);
the hysteresis update is pinned against the reference kernel source compiled for the host
(oracle/build_ref.sh).  The pre-linear RMSNorm is pinned against the reference's module within floating-point
tolerance (its row sums follow torch's summation order, which this restatement replaces by an exact one).  The weight-gradient GEMM has no reproducible definition in the reference
(it is a library fp16 GEMM whose values no reference test pins): the integer definition used
here (`grad_quantize` + `gemm_dw`) is this project's own and is "parity unpinned" against the
reference.
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------------------
# 2-bit weight code / 4-bit counter code   (kernels/int2/int2_packed.cuh:9-86)
# ----------------------------------------------------------------------------------------------

#: decode table of the 2-bit code: 00 -> -1, 01 -> 0, 10 -> +1, 11 -> 0 (int2_packed.cuh:13-18)
DECODE_LUT = np.array([-1, 0, 1, 0], dtype=np.int8)


def packed_k(K: int) -> int:
    """Bytes per packed weight row: ceil(K/4) (int2_packed.cuh:112-114)."""
    return (K + 3) // 4


def packed_h(K: int) -> int:
    """Bytes per packed counter row: ceil(K/2) (int2_packed.cuh:116-118)."""
    return (K + 1) // 2


def pack_ternary(w: np.ndarray, pad_code: int = 1) -> np.ndarray:
    """[N,K] values in {-1,0,+1} -> [N, ceil(K/4)] uint8.

    Weight k of a row sits in byte k//4 at bit offset 2*(k%4); -1 -> 0, 0 -> 1, +1 -> 2
    (int2_packed.cuh:29-40).  `pad_code` fills the unused fields of the last byte: the module
    packer pads with code 0 (core/bitnet/int2_linear_tc.py:424-427), the test packer with code 1
    (kernels/tests/kernel_build.py:74-76).  Kernels never read a field with k >= K.
    """
    w = np.asarray(w)
    N, K = w.shape
    pk = packed_k(K)
    enc = (np.clip(w, -1, 1).astype(np.int16) + 1).astype(np.uint8)
    pad = pk * 4 - K
    if pad:
        enc = np.concatenate([enc, np.full((N, pad), pad_code, dtype=np.uint8)], axis=1)
    enc = enc.reshape(N, pk, 4)
    return (enc[:, :, 0] | (enc[:, :, 1] << 2) | (enc[:, :, 2] << 4) | (enc[:, :, 3] << 6)).astype(np.uint8)


def unpack_ternary(W_packed: np.ndarray, K: int) -> np.ndarray:
    """[N, ceil(K/4)] uint8 -> [N,K] int8 in {-1,0,+1}; code 3 decodes to 0 (int2_packed.cuh:13-26)."""
    W_packed = np.asarray(W_packed, dtype=np.uint8)
    N, pk = W_packed.shape
    shifts = np.array([0, 2, 4, 6], dtype=np.uint8)
    fields = (W_packed[:, :, None] >> shifts) & 3
    return DECODE_LUT[fields].reshape(N, pk * 4)[:, :K]


def pack_counters(h: np.ndarray) -> np.ndarray:
    """[N,K] int counters -> [N, ceil(K/2)] uint8; even k in the low nibble, 4-bit two's
    complement, clamped to [-8,7] on write (int2_packed.cuh:66-86)."""
    h = np.asarray(h)
    N, K = h.shape
    ph = packed_h(K)
    bits = (np.clip(h, -8, 7).astype(np.int16) & 0xF).astype(np.uint8)
    if K % 2:
        bits = np.concatenate([bits, np.zeros((N, 1), dtype=np.uint8)], axis=1)
    bits = bits.reshape(N, ph, 2)
    return (bits[:, :, 0] | (bits[:, :, 1] << 4)).astype(np.uint8)


def unpack_counters(H_packed: np.ndarray, K: int) -> np.ndarray:
    """[N, ceil(K/2)] uint8 -> [N,K] int8 counters, sign-extended from 4 bits (int2_packed.cuh:56-64)."""
    H_packed = np.asarray(H_packed, dtype=np.uint8)
    N, ph = H_packed.shape
    lo = (H_packed & 0x0F).astype(np.int16)
    hi = (H_packed >> 4).astype(np.int16)
    nib = np.stack([lo, hi], axis=2).reshape(N, ph * 2)[:, :K]
    return np.where(nib & 8, nib - 16, nib).astype(np.int8)


# ----------------------------------------------------------------------------------------------
# Ternarisation   (core/bitnet/int2_linear_tc.py:391-412; model/common/bitnet_legacy.py:104-113)
# ----------------------------------------------------------------------------------------------

def absmean_scale(W: np.ndarray) -> float:
    """gamma = max(mean(|W|), 1e-5) (int2_linear_tc.py:395-397).  The reference takes the mean
    with torch; its summation order is not specified, so callers that need the reference's exact
    gamma pass it in explicitly."""
    return max(float(np.mean(np.abs(W.astype(np.float32)), dtype=np.float64)), 1e-5)


def ternarize(W: np.ndarray, gamma: float) -> np.ndarray:
    """q = clamp(round_half_even(W / gamma), -1, 1) in float32 (int2_linear_tc.py:399-400)."""
    q = np.rint(W.astype(np.float32) / np.float32(gamma))
    return np.clip(q, -1, 1).astype(np.int8)


# ----------------------------------------------------------------------------------------------
# Activation quantisation
# ----------------------------------------------------------------------------------------------

def quantize_rows(x: np.ndarray, eps: float = 1e-5):
    """Per-token absmax int8 quantisation (model/common/bitnet_legacy.py:71-78).

    In float32: a[m] = max(max_k |x[m,k]|, eps); s[m] = 127 / a[m];
    q = clamp(round_half_even(x * s), -128, 127).  Non-finite inputs count as 0 (the reference's
    CUDA quantiser does the same, int2_activation_quant.cu:104-105,138-141; the torch code leaves
    them undefined).  Returns (q int8 [M,K], a float32 [M]); consumers dequantise with a/127.
    """
    x = np.asarray(x, dtype=np.float32)
    x = np.where(np.isfinite(x), x, np.float32(0))
    if x.shape[1] == 0:
        a = np.full((x.shape[0],), np.float32(eps), dtype=np.float32)
    else:
        a = np.maximum(np.max(np.abs(x), axis=1), np.float32(eps)).astype(np.float32)
    s = (np.float32(127.0) / a).astype(np.float32)
    q = np.clip(np.rint(x * s[:, None]), -128, 127).astype(np.int8)
    return q, a


def quantize_tensor(x: np.ndarray):
    """Per-tensor absmax int8 quantisation (kernels/int2/int2_activation_quant.cu:88-167).

    absmax over the finite |x|; inv = absmax > 1e-8 ? 127/absmax : 0;
    q = clamp(roundf(x*inv), -127, 127) with roundf = half away from zero; non-finite -> 0.
    The reference builds with fast-math, whose approximate division can move `inv` by an ulp;
    this restatement divides in IEEE float32.  Returns (q int8, absmax float32 scalar).
    """
    x = np.asarray(x, dtype=np.float32)
    x = np.where(np.isfinite(x), x, np.float32(0))
    absmax = np.float32(np.max(np.abs(x))) if x.size else np.float32(0)
    inv = np.float32(127.0) / absmax if absmax > np.float32(1e-8) else np.float32(0)
    y = (x * inv).astype(np.float32)
    r = np.sign(y) * np.floor(np.abs(y) + np.float32(0.5))  # half away from zero, as roundf
    q = np.clip(r, -127, 127).astype(np.int8)
    return q, absmax


def dequantize_tensor(q: np.ndarray, absmax) -> np.ndarray:
    """float32(q) * (absmax / 127) (int2_activation_quant.cu:172-202), before the fp16 store."""
    return q.astype(np.float32) * (np.float32(absmax) / np.float32(127.0))


# ----------------------------------------------------------------------------------------------
# Integer GEMMs and their epilogue
# ----------------------------------------------------------------------------------------------

def _imatmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Exact integer matrix product through float64 BLAS (|sum| < 2**53 for every shape here)."""
    return np.rint(a.astype(np.float64) @ b.astype(np.float64)).astype(np.int64)


def gemm_fwd_acc(Xq: np.ndarray, W_packed: np.ndarray, K: int) -> np.ndarray:
    """acc[m,n] = sum_k Xq[m,k] * Wq[n,k], exact (int2_matmul_int8_tc_v2.cu:142-233,466-470)."""
    Wq = unpack_ternary(W_packed, K)
    return _imatmul(Xq, Wq.T).astype(np.int32)


def gemm_dx_acc(dYq: np.ndarray, W_packed: np.ndarray, K: int) -> np.ndarray:
    """acc[m,k] = sum_n dYq[m,n] * Wq[n,k], exact (int2_backward_int8_tc_v2.cu:112-205,436-440)."""
    Wq = unpack_ternary(W_packed, K)
    return _imatmul(dYq, Wq).astype(np.int32)


def gemm_dw_acc(Gq: np.ndarray, Xq: np.ndarray) -> np.ndarray:
    """acc[n,k] = sum_m Gq[m,n] * Xq[m,k], exact integer weight-gradient accumulators."""
    return _imatmul(Gq.T, Xq).astype(np.int32)


def scale_rows(acc: np.ndarray, absmax, gamma: float) -> np.ndarray:
    """float32 epilogue: out = float(acc) * ((absmax/127) * gamma), each step rounded to float32
    (int2_matmul_int8_tc_v2.cu:118-121,261: `(*d_scale_x / 127.0f) * gamma`, then
    `(float)acc * out_scale`).  `absmax` is a scalar (per-tensor) or one value per row (per-token)."""
    a = np.asarray(absmax, dtype=np.float32)
    sc = ((a / np.float32(127.0)).astype(np.float32) * np.float32(gamma)).astype(np.float32)
    if sc.ndim == 1:
        sc = sc[:, None]
    return (acc.astype(np.float32) * sc).astype(np.float32)


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round float32 to bfloat16 (nearest even) and return it as float32 values."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = np.isnan(x)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    out = r.astype(np.uint32).view(np.float32)
    return np.where(nan, np.float32(np.nan), out).astype(np.float32)


def to_f16(x: np.ndarray) -> np.ndarray:
    """Round float32 to float16 (nearest even) and return it as float32 values."""
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Weight gradient (this project's integer definition; no reproducible counterpart in the
# reference, which calls a library fp16 GEMM: core/bitnet/int2_linear_tc.py:525-537)
# ----------------------------------------------------------------------------------------------

GRAD_ABSMAX_FLOOR = np.float32(1e-30)


def grad_fold(dY: np.ndarray, x_absmax: np.ndarray) -> np.ndarray:
    """G[m,n] = dY[m,n] * (x_absmax[m] / 127) in float32: the per-token activation scale folded
    into the output gradient so that dW = sum_m G[m,n] * Xq[m,k] needs no per-row scale."""
    sx = (np.asarray(x_absmax, dtype=np.float32) / np.float32(127.0)).astype(np.float32)
    dY = np.asarray(dY, dtype=np.float32)
    dY = np.where(np.isfinite(dY), dY, np.float32(0))
    return (dY * sx[:, None]).astype(np.float32)


def grad_quantize(dY: np.ndarray, x_absmax: np.ndarray, g_absmax=None):
    """Per-tensor int8 quantisation of G = grad_fold(dY, x_absmax).

    g = max |G|; inv = g >= 1e-30 ? 127/g : 0; Gq = clamp(round_half_even(G*inv), -127, 127).
    `g_absmax` may be supplied (a shard of a larger tensor uses the global maximum).
    Returns (Gq int8 [M,N], g float32)."""
    G = grad_fold(dY, x_absmax)
    g = np.float32(np.max(np.abs(G))) if g_absmax is None else np.float32(g_absmax)
    inv = np.float32(127.0) / g if g >= GRAD_ABSMAX_FLOOR else np.float32(0)
    Gq = np.clip(np.rint((G * inv).astype(np.float32)), -127, 127).astype(np.int8)
    return Gq, g


def dw_from_acc(acc: np.ndarray, g_absmax) -> np.ndarray:
    """dW[n,k] = float32(acc[n,k]) * (g_absmax / 127), each step rounded to float32."""
    sc = np.float32(g_absmax) / np.float32(127.0)
    return (acc.astype(np.float32) * sc).astype(np.float32)


# ----------------------------------------------------------------------------------------------
# Hysteresis update   (kernels/int2/int2_hysteresis_v2.cu:54-152)
# ----------------------------------------------------------------------------------------------

_FLT_MIN = np.float32(1.17549435e-38)


def _ftz(x: np.ndarray) -> np.ndarray:
    """Flush float32 denormals to zero: the reference kernels are built with fast-math
    (core/bitnet/int2_linear_tc.py:46), which flushes denormal inputs and results."""
    x = np.asarray(x, dtype=np.float32)
    return np.where(np.abs(x) < _FLT_MIN, np.float32(0), x).astype(np.float32)


def _hash24(idx: np.ndarray, step: int, mult: int) -> np.ndarray:
    """Two mixing rounds of ((h>>16)^h)*0x45d9f3b on idx ^ (step*mult), uint32 wrap-around; the
    low 24 bits divided by 2**24 (int2_hysteresis_v2.cu:88-96)."""
    s = np.uint32((int(step) & 0xFFFFFFFF) * mult & 0xFFFFFFFF)
    h = idx ^ s
    for _ in range(2):
        h = (((h >> np.uint32(16)) ^ h).astype(np.uint64) * np.uint64(0x45D9F3B) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    return (h & np.uint32(0xFFFFFF)).astype(np.float32) / np.float32(16777216.0)


def hysteresis_step(dW, W_packed, H_packed, lr, lr_scale, threshold, decay_rate, step, K,
                    idx_base: int = 0, ftz: bool = True):
    """One hysteresis update of every weight; returns new (W_packed, H_packed).

    Follows int2_hysteresis_v2.cu:66-151 per weight with idx = n*K + k (+ idx_base for a row
    shard of a larger matrix, so that a sharded run draws the same random numbers):
      thr = clamp(threshold, 1, 7)
      r1, r2 = hash24(idx, step, 2654435761), hash24(idx, step, 2246822519)
      d_raw = -dW * ((lr*lr_scale)*thr);  delta = sign*(floor|d_raw| + [r1 < frac]) clamped +-31
      h' = h + delta;  if q != 0 and r2 < decay: h' -= sign(q)
      h' >= thr: -1 -> 0, 0 -> +1 (counter reset) or saturate at +1;  symmetric for <= -thr
      h' clamped to +-thr;  both fields rewritten (code 3 is re-encoded as 1).
    `ftz=True` models the reference build (fast-math flush-to-zero)."""
    dW = np.asarray(dW, dtype=np.float32)
    N = dW.shape[0]
    assert dW.shape == (N, K)
    thr = min(max(int(threshold), 1), 7)
    q = unpack_ternary(W_packed, K).astype(np.int32)
    h = unpack_counters(H_packed, K).astype(np.int32)

    idx = ((np.arange(N * K, dtype=np.int64) + int(idx_base)) & 0xFFFFFFFF).astype(np.uint32).reshape(N, K)
    r1 = _hash24(idx, step, 2654435761)
    r2 = _hash24(idx, step, 2246822519)

    lr32, ls32, dc32 = np.float32(lr), np.float32(lr_scale), np.float32(decay_rate)
    prod = np.float32(lr32 * ls32)
    if ftz:
        lr32, ls32, dc32 = _ftz(lr32), _ftz(ls32), _ftz(dc32)
        prod = _ftz(np.float32(lr32 * ls32))
    lr_scaled = np.float32(prod * np.float32(thr))
    grad = _ftz(dW) if ftz else dW
    if ftz:
        lr_scaled = _ftz(lr_scaled)
    with np.errstate(invalid="ignore", over="ignore"):
        d_raw = (-grad * lr_scaled).astype(np.float32)
        if ftz:
            d_raw = _ftz(d_raw)
        sign = np.where(d_raw >= 0, np.float32(1), np.float32(-1))
        a = np.abs(d_raw)
        fl = np.floor(a)
        frac = (a - fl).astype(np.float32)
        inc = np.where(r1 < frac, np.float32(1), np.float32(0))
        val = (sign * (fl + inc)).astype(np.float32)
    # float -> int32 as the GPU converts: NaN -> 0, saturating
    val = np.where(np.isnan(val), np.float32(0), val)
    delta = np.clip(val, -2147483648.0, 2147483520.0).astype(np.int64)
    delta = np.clip(delta, -31, 31).astype(np.int32)

    hn = h + delta
    decay = (q != 0) & (r2 < dc32)
    hn = np.where(decay, hn - np.sign(q), hn)

    qn = q.copy()
    up = hn >= thr
    dn = (~up) & (hn <= -thr)
    # upward crossing
    qn = np.where(up & (q == -1), 0, qn)
    qn = np.where(up & (q == 0), 1, qn)
    hn = np.where(up & (q != 1), 0, hn)
    hn = np.where(up & (q == 1), thr, hn)
    # downward crossing
    qn = np.where(dn & (q == 1), 0, qn)
    qn = np.where(dn & (q == 0), -1, qn)
    hn = np.where(dn & (q != -1), 0, hn)
    hn = np.where(dn & (q == -1), -thr, hn)
    hn = np.clip(hn, -thr, thr)

    # rewrite the fields with k < K only; padding fields keep their bits
    W_new = _repack_fields(np.asarray(W_packed, dtype=np.uint8), qn + 1, K, bits=2)
    H_new = _repack_fields(np.asarray(H_packed, dtype=np.uint8), hn & 0xF, K, bits=4)
    return W_new, H_new


def _repack_fields(old: np.ndarray, fields: np.ndarray, K: int, bits: int) -> np.ndarray:
    per = 8 // bits
    N, pb = old.shape
    mask = (1 << bits) - 1
    full = np.zeros((N, pb * per), dtype=np.uint8)
    shifts = (np.arange(per, dtype=np.uint8) * bits).astype(np.uint8)
    full[:, :] = ((old[:, :, None] >> shifts) & mask).reshape(N, pb * per)
    full[:, :K] = fields.astype(np.uint8)
    full = full.reshape(N, pb, per)
    out = np.zeros((N, pb), dtype=np.uint8)
    for j in range(per):
        out |= (full[:, :, j] << np.uint8(j * bits)).astype(np.uint8)
    return out


# ----------------------------------------------------------------------------------------------
# pre-linear RMSNorm   (core/bitnet/bitnet_int2_optimized.py:72-86; model/common/bitnet_legacy.py:10-25)
# ----------------------------------------------------------------------------------------------

def _round_io(x: np.ndarray, io: str) -> np.ndarray:
    """float32 values rounded to the layer's I/O type ("bf16", "f16" or "f32") and held as float32."""
    if io == "bf16":
        return to_bf16(x)
    if io == "f16":
        return to_f16(x)
    return np.asarray(x, dtype=np.float32)


def rmsnorm_rstd(x: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """rstd[m] = 1 / sqrt(mean_k x[m,k]^2 + eps) as the reference computes it in float32
    (`x_f32 * torch.rsqrt(x_f32.pow(2).mean(-1) + eps)`): squares rounded to float32, their sum taken
    exactly (float64 accumulation, then rounded to float32 - torch's own float32 summation order is not
    reproducible, this is the order-free definition), divided by K, plus eps, sqrt, reciprocal - each
    a float32 operation."""
    x = np.asarray(x, dtype=np.float32)
    K = x.shape[1]
    sq = (x * x).astype(np.float32)
    ssum = sq.astype(np.float64).sum(axis=1).astype(np.float32)
    ms = (ssum / np.float32(K)).astype(np.float32)
    v = (ms + np.float32(eps)).astype(np.float32)
    return (np.float32(1.0) / np.sqrt(v).astype(np.float32)).astype(np.float32)


def rmsnorm_forward(x: np.ndarray, weight: np.ndarray, eps: float = 1e-6, io: str = "bf16"):
    """The reference's pre-linear RMSNorm: `norm.type_as(x) * weight.type_as(x)`: the normalised value is
    rounded to the I/O type, the weight is rounded to the I/O type, and so is their product.
    Returns (y float32 holding I/O-type values [M,K], rstd float32 [M])."""
    x = _round_io(x, io)
    rstd = rmsnorm_rstd(x, eps)
    norm = _round_io((x * rstd[:, None]).astype(np.float32), io)
    w = _round_io(np.asarray(weight, dtype=np.float32), io)
    return _round_io((norm * w[None, :]).astype(np.float32), io), rstd


def rmsnorm_quantize_rows(x, weight, norm_eps: float = 1e-6, quant_eps: float = 1e-5, io: str = "bf16"):
    """RMSNorm followed by the per-token quantiser: what the fused kernel returns.
    (q int8 [M,K], absmax float32 [M], rstd float32 [M])."""
    y, rstd = rmsnorm_forward(x, weight, norm_eps, io)
    q, a = quantize_rows(y, quant_eps)
    return q, a, rstd


def rmsnorm_backward(g: np.ndarray, x: np.ndarray, weight: np.ndarray, rstd: np.ndarray, io: str = "bf16"):
    """Gradient of rmsnorm_forward for an upstream gradient g (I/O type), the quantiser being a
    straight-through estimator (model/common/bitnet_legacy.py:83-87).  Follows autograd through the
    reference's expression, each step in float32:
      gn = io(g * io(w))                       gradient of `norm.type_as(x)`
      c[m] = sum_k gn[m,k] * x[m,k]            exact sum of float32 products, rounded to float32
      coef[m] = ((rstd*rstd)*rstd) * c / K
      dx = io(gn * rstd - x * coef)
      dweight[k] = sum_m g[m,k] * io(x*rstd)[m,k]   exact sum of float32 products, rounded to float32
    Returns (dx float32 holding I/O-type values, dweight float32 [K])."""
    g = _round_io(g, io)
    x = _round_io(x, io)
    rstd = np.asarray(rstd, dtype=np.float32)
    K = x.shape[1]
    w = _round_io(np.asarray(weight, dtype=np.float32), io)
    gn = _round_io((g * w[None, :]).astype(np.float32), io)
    c = (gn * x).astype(np.float32).astype(np.float64).sum(axis=1).astype(np.float32)
    r3 = ((rstd * rstd).astype(np.float32) * rstd).astype(np.float32)
    coef = ((r3 * c).astype(np.float32) / np.float32(K)).astype(np.float32)
    t1 = (gn * rstd[:, None]).astype(np.float32)
    t2 = (x * coef[:, None]).astype(np.float32)
    dx = _round_io((t1 - t2).astype(np.float32), io)
    norm = _round_io((x * rstd[:, None]).astype(np.float32), io)
    dweight = (g * norm).astype(np.float32).astype(np.float64).sum(axis=0).astype(np.float32)
    return dx, dweight


# ----------------------------------------------------------------------------------------------
# SwiGLU gate in front of the down projection   (model/model.py:86-108: w3(silu(w1 x) * w2 x))
# ----------------------------------------------------------------------------------------------

def sigmoid_fixed(g: np.ndarray) -> np.ndarray:
    """1/(1 + e^-g) in float32 with the fixed polynomial exponential of oracle/int2_oracle.c (the one
    piece of this file that needs the C library: NumPy has no fused multiply-add)."""
    from . import native
    return native.c_sigmoid_fixed(np.asarray(g, dtype=np.float32))


def swiglu_hidden(gate: np.ndarray, up: np.ndarray, io: str = "bf16"):
    """`F.silu(gate) * up` as two tensor operations of the I/O type (model/model.py:107-108):
    s = io(gate * sigmoid(gate)), h = io(s * up).  Returns (h, s, sig) as float32 arrays."""
    g = _round_io(gate, io)
    u = _round_io(up, io)
    sig = sigmoid_fixed(g)
    s = _round_io((g * sig).astype(np.float32), io)
    h = _round_io((s * u).astype(np.float32), io)
    return h, s, sig


def swiglu_quantize_rows(gate, up, norm_weight=None, norm_eps: float = 1e-6, quant_eps: float = 1e-5, io: str = "bf16"):
    """What the down projection's GEMM reads: the gated product, normalised by the layer's pre-linear
    RMSNorm when `norm_weight` is given (core/bitnet/bitnet_int2_optimized.py:201-204), quantised per
    token.  Returns (q int8 [M,H], absmax float32 [M], rstd float32 [M] or None)."""
    h, _, _ = swiglu_hidden(gate, up, io)
    if norm_weight is None:
        q, a = quantize_rows(h, quant_eps)
        return q, a, None
    return rmsnorm_quantize_rows(h, norm_weight, norm_eps, quant_eps, io)


def swiglu_backward(gy, gate, up, norm_weight=None, rstd=None, io: str = "bf16"):
    """Gradients of swiglu_quantize_rows' input for the upstream gradient gy with respect to the quantised
    row (straight-through quantiser), following autograd through the tensor operations:
      dh = rmsnorm_backward(gy, h) (or gy);  ds = io(dh*up);  d_up = io(dh*s);
      d_gate = io((ds*sig) * (1 + gate*(1 - sig)))     (torch's silu backward, float32)
    Returns (d_gate, d_up, d_norm_weight or None)."""
    g = _round_io(gate, io)
    u = _round_io(up, io)
    h, s, sig = swiglu_hidden(g, u, io)
    if norm_weight is None:
        dh, dweight = _round_io(gy, io), None
    else:
        dh, dweight = rmsnorm_backward(gy, h, norm_weight, rstd, io)
    ds = _round_io((dh * u).astype(np.float32), io)
    d_up = _round_io((dh * s).astype(np.float32), io)
    one = np.float32(1.0)
    t = (one + (g * (one - sig).astype(np.float32)).astype(np.float32)).astype(np.float32)
    d_gate = _round_io(((ds * sig).astype(np.float32) * t).astype(np.float32), io)
    return d_gate, d_up, dweight


# ----------------------------------------------------------------------------------------------
# Composite layer step (per-token mode): forward, dX, dW + hysteresis
# ----------------------------------------------------------------------------------------------

def bitlinear_forward(x, W_packed, gamma, K, out="bf16"):
    """x [M,K] float -> (Y, Xq, x_absmax).  Y = round_out(float(acc) * ((a/127)*gamma))."""
    Xq, a = quantize_rows(x)
    y = scale_rows(gemm_fwd_acc(Xq, W_packed, K), a, gamma)
    y = {"bf16": to_bf16, "f16": to_f16, "f32": lambda v: v}[out](y)
    return y, Xq, a


def bitlinear_backward_dx(dY, W_packed, gamma, K, out="bf16"):
    """dY [M,N] float -> dX [M,K] = round_out(float(sum_n dYq*Wq) * ((a_dy/127)*gamma))."""
    dYq, a = quantize_rows(dY, eps=GRAD_ABSMAX_FLOOR)
    dx = scale_rows(gemm_dx_acc(dYq, W_packed, K), a, gamma)
    return {"bf16": to_bf16, "f16": to_f16, "f32": lambda v: v}[out](dx)


def bitlinear_dw(dY, Xq, x_absmax, g_absmax=None):
    """Integer weight gradient: returns (dW float32 [N,K], acc int32 [N,K], g_absmax)."""
    Gq, g = grad_quantize(dY, x_absmax, g_absmax)
    acc = gemm_dw_acc(Gq, Xq)
    return dw_from_acc(acc, g), acc, g
