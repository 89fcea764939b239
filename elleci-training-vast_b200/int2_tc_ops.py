"""The operator surface of the INT2 linear path, on torch tensors.

The first group of functions keeps the names, argument meaning and error behaviour of the reference's
extension module `int2_tc_ops` (kernels/int2/int2_tc_ops.cpp:502-538): CUDA tensors in, outputs
allocated here, work queued on the current CUDA stream, `W_packed` / `H_packed` updated in place,
`RuntimeError` on bad arguments.  The second group is the per-token (bf16) path and the fused
weight-gradient + hysteresis step, which the reference does not have.

Every function ends in one call of the C-ABI library (include/elleci_int2.h); none computes in torch.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import EL_BF16, EL_F16, EL_F32, EL_FLAG_LEAN, EL_I32, EL_PATH_AUTO, EL_PATH_SIMPLE, EL_PATH_TC, ElleciError, call

_DT = {torch.float16: EL_F16, torch.bfloat16: EL_BF16, torch.float32: EL_F32, torch.int32: EL_I32}
GRAD_EPS = 1e-30          # floor of a gradient row's absmax (an all-zero row quantises to zeros)
ACT_EPS = 1e-5            # floor of an activation row's absmax (model/common/bitnet_legacy.py:45,75)

_status_bufs: dict = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _cuda(t: torch.Tensor, name: str) -> None:
    _require(isinstance(t, torch.Tensor) and t.is_cuda, f"{name} must be a CUDA tensor")


def device_status(device: torch.device) -> torch.Tensor:
    """The int32 word the tensor-core kernels write when a bounded wait gives up (0 = healthy)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    buf = _status_bufs.get(key)
    if buf is None:
        buf = torch.zeros(1, dtype=torch.int32, device=device)
        _status_bufs[key] = buf
    return buf


def check_device_status(device: torch.device) -> None:
    """Synchronises and raises if a tensor-core kernel reported a failed wait.  A kernel that gave up may have left
    partial sums in a decode workspace, which every call expects to find zeroed: the cached workspaces of the device are
    dropped, so the next decode call starts from a fresh zeroed one."""
    code = int(device_status(device).item())
    if code != 0:
        device_status(device).zero_()
        index = device.index if device.index is not None else torch.cuda.current_device()
        for key in [k for k in _decode_ws if k[0] == index]:
            del _decode_ws[key]
        raise ElleciError("tensor-core kernel", code, f"a bounded barrier wait gave up (code {code})")


def _maybe_check(device: torch.device) -> None:
    if os.environ.get("ELLECI_CHECK_STATUS") == "1":
        check_device_status(device)


# ==============================================================================================
# Group 1: the reference extension's surface (per-tensor scales, fp16 I/O)
# ==============================================================================================

def quantize_activation_async(input: torch.Tensor, d_global_max: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(int8 tensor, absmax[1]) of a float tensor, per-tensor rule; no host sync
    (tc_quantize_activation_async, kernels/int2/int2_tc_ops.cpp:343-371).  `d_global_max` is accepted for
    signature compatibility; the absmax is accumulated in the returned scale tensor, so concurrent
    streams do not share scratch."""
    _cuda(input, "Input")
    _cuda(d_global_max, "d_global_max")
    _require(input.dtype in (torch.float16, torch.bfloat16, torch.float32), "Input must be float16")
    x = input.contiguous()
    out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    call("el_quantize_tensor", x.data_ptr(), _DT[x.dtype], out.data_ptr(), scale.data_ptr(), x.numel(), _stream())
    return out, scale


def quantize_activation(input: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """tc_quantize_activation (kernels/int2/int2_tc_ops.cpp:279-305)."""
    _cuda(input, "Input")
    return quantize_activation_async(input, input)


def dequantize_activation(input_int8: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """int8 * (absmax/127) -> fp16 (tc_dequantize_activation, kernels/int2/int2_tc_ops.cpp:310-337)."""
    _cuda(input_int8, "Input")
    _cuda(scale, "scale")
    _require(input_int8.dtype == torch.int8, "Input must be int8")
    _require(scale.dtype == torch.float32, "scale must be float32")
    q = input_int8.contiguous()
    out = torch.empty(q.shape, dtype=dtype, device=q.device)
    call("el_dequantize_tensor", q.data_ptr(), scale.data_ptr(), out.data_ptr(), _DT[dtype], q.numel(), _stream())
    return out


_gemm_ws: dict = {}


def _gemm_workspace(device: torch.device, mode: int, M: int, N: int, K: int):
    """(pointer, bytes) of the scratch a GEMM with few output tiles uses to split its reduction over idle CTA pairs, or
    (None, 0) when the shape is not split.  One buffer per device and stream, grown on demand; calls on one stream are
    ordered, so they can share it."""
    need = _lib.lib().el_gemm_workspace_bytes(mode, M, N, K)
    if need == 0:
        return None, 0
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    buf = _gemm_ws.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.uint8, device=device)
        _gemm_ws[key] = buf
    return buf.data_ptr(), buf.numel()


def _gemm_fwd(Xq, W_packed, absmax, stride, gamma, out_dtype, path=EL_PATH_AUTO):
    _cuda(Xq, "X_int8"); _cuda(W_packed, "W_packed"); _cuda(absmax, "d_scale_x")
    _require(Xq.dtype == torch.int8, "X_int8 must be int8")
    _require(W_packed.dtype == torch.uint8, "W_packed must be uint8")
    _require(absmax.dtype == torch.float32, "d_scale_x must be float32")
    _require(W_packed.dim() == 2, "W_packed must be 2-D [N, ceil(K/4)]")
    N, pK = W_packed.shape
    K = Xq.shape[-1]
    _require((K + 3) // 4 == pK, f"Dimension mismatch: X has {K} features but W_packed has packed_K={pK} "
                                 f"(expected ceil(K/4)={(K + 3) // 4})")
    Xf = Xq.contiguous().view(-1, K)
    M = Xf.shape[0]
    _require(stride == 0 or absmax.numel() == M, "one absmax per token expected")
    Wc = W_packed.contiguous()
    Y = torch.empty(M, N, dtype=out_dtype, device=Xq.device)
    st = device_status(Xq.device)
    ws, ws_bytes = _gemm_workspace(Xq.device, 0, M, N, K) if (path & ~EL_FLAG_LEAN) in (EL_PATH_AUTO, EL_PATH_TC) else (None, 0)
    call("el_gemm_fwd_ws", Xf.data_ptr(), Wc.data_ptr(), Y.data_ptr(), _DT[out_dtype], absmax.data_ptr(), stride,
         float(gamma), M, N, K, path, ws, ws_bytes, st.data_ptr(), _stream())
    _maybe_check(Xq.device)
    return Y.view(*Xq.shape[:-1], N)


def _gemm_dx(dYq, W_packed, absmax, stride, gamma, K, out_dtype, path=EL_PATH_AUTO):
    _cuda(dYq, "dY_int8"); _cuda(W_packed, "W_packed"); _cuda(absmax, "d_scale_dy")
    _require(dYq.dtype == torch.int8, "dY_int8 must be int8")
    _require(W_packed.dtype == torch.uint8, "W_packed must be uint8")
    _require(absmax.dtype == torch.float32, "d_scale_dy must be float32")
    N, pK = W_packed.shape
    _require(dYq.shape[-1] == N, f"dY has {dYq.shape[-1]} features but W_packed has {N} rows")
    _require((K + 3) // 4 == pK, f"K={K} does not match W_packed's packed_K={pK}")
    Yf = dYq.contiguous().view(-1, N)
    M = Yf.shape[0]
    _require(stride == 0 or absmax.numel() == M, "one absmax per token expected")
    Wc = W_packed.contiguous()
    dX = torch.empty(M, K, dtype=out_dtype, device=dYq.device)
    st = device_status(dYq.device)
    ws, ws_bytes = _gemm_workspace(dYq.device, 1, M, N, int(K)) if (path & ~EL_FLAG_LEAN) in (EL_PATH_AUTO, EL_PATH_TC) else (None, 0)
    call("el_gemm_dx_ws", Yf.data_ptr(), Wc.data_ptr(), dX.data_ptr(), _DT[out_dtype], absmax.data_ptr(), stride,
         float(gamma), M, N, int(K), path, ws, ws_bytes, st.data_ptr(), _stream())
    _maybe_check(dYq.device)
    return dX.view(*dYq.shape[:-1], K)


def matmul_int8(X_int8: torch.Tensor, W_packed: torch.Tensor, d_scale_x: torch.Tensor, gamma: float,
                out_dtype: torch.dtype = torch.float16, path: int = EL_PATH_AUTO) -> torch.Tensor:
    """Y = X_int8 @ W^T * (scale_x/127) * gamma, fp16 out (tc_matmul_int8, kernels/int2/int2_tc_ops.cpp:381-425)."""
    return _gemm_fwd(X_int8, W_packed, d_scale_x, 0, gamma, out_dtype, path)


def backward_input_int8(dY_int8: torch.Tensor, W_packed: torch.Tensor, d_scale_dy: torch.Tensor, gamma: float, K: int,
                        out_dtype: torch.dtype = torch.float16, path: int = EL_PATH_AUTO) -> torch.Tensor:
    """dX = dY_int8 @ W * (scale_dy/127) * gamma (tc_backward_input_int8, kernels/int2/int2_tc_ops.cpp:435-470)."""
    return _gemm_dx(dY_int8, W_packed, d_scale_dy, 0, gamma, K, out_dtype, path)


def hysteresis_step_v2(dW: torch.Tensor, W_packed: torch.Tensor, H_packed: torch.Tensor, lr: float, lr_scale: float,
                       threshold: int, decay: float, step: int, idx_base: int = 0, ftz: bool = True) -> None:
    """In-place hysteresis update from a float32 gradient (tc_hysteresis_step_v2,
    kernels/int2/int2_tc_ops.cpp:214-257); same checks, same integer results."""
    _cuda(dW, "dW")
    _require(W_packed.is_cuda and H_packed.is_cuda, "State must be on CUDA")
    _require(dW.dtype == torch.float32, "dW must be float32")
    _require(dW.dim() == 2, "dW must be 2-D [N, K]")
    dW = dW.contiguous()
    N, K = dW.shape
    pK, pH = (K + 3) // 4, (K + 1) // 2
    _require(W_packed.dim() == 2 and tuple(W_packed.shape) == (N, pK), f"W_packed expected [{N}, {pK}] = [N, ceil(K/4)]")
    _require(H_packed.dim() == 2 and tuple(H_packed.shape) == (N, pH), f"H_packed expected [{N}, {pH}] = [N, ceil(K/2)]")
    _require(W_packed.dtype == torch.uint8 and H_packed.dtype == torch.uint8, "W_packed/H_packed must be uint8")
    _require(W_packed.is_contiguous() and H_packed.is_contiguous(), "W_packed/H_packed must be contiguous")
    step32 = int(step) & 0xFFFFFFFF
    step_i = step32 - (1 << 32) if step32 >= (1 << 31) else step32
    call("el_hysteresis_from_dw", dW.data_ptr(), W_packed.data_ptr(), H_packed.data_ptr(), float(lr), float(lr_scale),
         int(threshold), float(decay), step_i, N, K, int(idx_base) & 0xFFFFFFFF, int(bool(ftz)), _stream())


def unpack_int2(W_packed: torch.Tensor, W_out: torch.Tensor, K: int) -> None:
    """W_packed -> dense {-1,0,+1} matrix in W_out's dtype (tc_unpack_int2, kernels/int2/int2_tc_ops.cpp:476-499)."""
    _cuda(W_packed, "W_packed"); _cuda(W_out, "W_fp16")
    _require(W_packed.dtype == torch.uint8, "W_packed must be uint8")
    N = W_packed.shape[0]
    _require(W_out.shape[0] == N, "W_fp16 row count must match W_packed")
    _require(W_out.shape[1] == K, "W_fp16 col count must equal K")
    _require(W_out.is_contiguous() and W_packed.is_contiguous(), "tensors must be contiguous")
    dt = EL_I32 if W_out.dtype == torch.int8 else _DT[W_out.dtype]
    call("el_unpack_ternary", W_packed.data_ptr(), W_out.data_ptr(), dt, N, int(K), _stream())


def memory_stats() -> dict:
    """GPU memory statistics (tc_memory_stats, kernels/int2/int2_tc_ops.cpp:264-273)."""
    free, total = torch.cuda.mem_get_info()
    return {"free_bytes": free, "total_bytes": total, "used_bytes": total - free}


# ==============================================================================================
# Group 2: per-token path, packing, integer weight gradient, fused dW + hysteresis
# ==============================================================================================

def pack_int2(w_ternary: torch.Tensor, pad_code: int = 0) -> torch.Tensor:
    """[N,K] in {-1,0,1} (any dtype) -> packed uint8 [N, ceil(K/4)] on the device."""
    _cuda(w_ternary, "w_ternary")
    w = w_ternary.to(torch.int8).contiguous()
    N, K = w.shape
    out = torch.empty(N, (K + 3) // 4, dtype=torch.uint8, device=w.device)
    call("el_pack_ternary", w.data_ptr(), out.data_ptr(), N, K, int(pad_code), _stream())
    return out


def ternarize_pack(weight: torch.Tensor, gamma: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """clamp(round(W/gamma), -1, 1) packed in one pass (the arithmetic of Int2LinearTC.init_from_float,
    core/bitnet/int2_linear_tc.py:399-400, then _pack_int2_cpu)."""
    _cuda(weight, "weight")
    w = weight.float().contiguous()
    N, K = w.shape
    if out is None:
        out = torch.empty(N, (K + 3) // 4, dtype=torch.uint8, device=w.device)
    _require(out.is_contiguous() and tuple(out.shape) == (N, (K + 3) // 4), "bad W_packed buffer")
    call("el_ternarize_pack", w.data_ptr(), float(gamma), out.data_ptr(), N, K, _stream())
    return out


def _rows_view(t: torch.Tensor):
    """(tensor, M, cols, row pitch) of a 2-D view whose rows are contiguous (a column window of a wider
    matrix qualifies), or of any tensor after flattening its leading dimensions."""
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) >= t.shape[1]:
        return t, t.shape[0], t.shape[1], t.stride(0)
    tc = t.contiguous()
    cols = tc.shape[-1]
    return tc, math.prod(tc.shape[:-1]), cols, cols


def quantize_rows(x: torch.Tensor, eps: float = ACT_EPS, fold_absmax: Optional[torch.Tensor] = None,
                  raw_absmax: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    """Per-token absmax int8 quantisation.  Returns (q int8, absmax float32 [M]) and, when `fold_absmax` [M] is
    given, also max_m(rawmax[m]*fold_absmax[m]/127) as a float32 [1] tensor.  `raw_absmax` [M] supplies row
    maxima found elsewhere (reduced over the ranks of a column-sharded tensor); it is floored at eps in place
    and returned as the absmax.  A 2-D column window `x[:, a:b]` is read in place.  `out` (contiguous int8, M*K
    elements: a row block of a larger buffer, say) receives the quantised rows instead of a new tensor."""
    _cuda(x, "x")
    _require(x.dtype in _DT and x.dtype != torch.int32, "x must be float16, bfloat16 or float32")
    xv, M, K, ld = _rows_view(x)
    if out is None:
        q = torch.empty(*x.shape[:-1], K, dtype=torch.int8, device=x.device)
    else:
        _require(out.is_cuda and out.dtype == torch.int8 and out.is_contiguous() and out.numel() == M * K,
                 "out must be a contiguous int8 CUDA tensor of M*K elements")
        q = out
    if raw_absmax is None:
        a = torch.empty(M, dtype=torch.float32, device=x.device)
        mode = _lib.EL_QUANT_FULL
    else:
        _require(raw_absmax.dtype == torch.float32 and raw_absmax.numel() == M and raw_absmax.is_contiguous(),
                 "raw_absmax must be a contiguous float32 [M]")
        a = raw_absmax
        mode = _lib.EL_QUANT_WITH_ABSMAX
    fold_max = None
    if fold_absmax is not None:
        _require(fold_absmax.dtype == torch.float32 and fold_absmax.numel() == M, "fold_absmax must be float32 [M]")
        fold_max = torch.zeros(1, dtype=torch.float32, device=x.device)
    call("el_quantize_rows", xv.data_ptr(), _DT[xv.dtype], ld, q.data_ptr(), a.data_ptr(), M, K, float(eps), mode,
         _ptr(fold_absmax), _ptr(fold_max), _stream())
    return (q, a) if fold_absmax is None else (q, a, fold_max)


NORM_EPS = 1e-6            # default eps of the reference's pre-linear RMSNorm (core/bitnet/bitnet_int2_optimized.py:78)
_norm_ws: dict = {}


def rmsnorm_supported(x: torch.Tensor) -> bool:
    """Shapes the fused RMSNorm kernels take: a float CUDA tensor whose feature count is a multiple of 8 (at most
    25600) and whose rows are 16-byte aligned."""
    K = x.shape[-1] if x.dim() else 0
    return (x.is_cuda and x.dtype in (torch.float16, torch.bfloat16, torch.float32) and K > 0 and K % 8 == 0
            and K <= 25600 and x.is_contiguous() and x.data_ptr() % 16 == 0)


def rmsnorm_quantize_rows(x: torch.Tensor, weight: torch.Tensor, norm_eps: float = NORM_EPS, quant_eps: float = ACT_EPS):
    """The reference's pre-linear RMSNorm (`_ExtraRMSNorm`, core/bitnet/bitnet_int2_optimized.py:72-86) followed by
    the per-token quantiser, in one pass over x.  `weight` is the float32 norm weight [K].  Returns
    (q int8 like x, absmax float32 [M], rstd float32 [M]); q and absmax equal quantize_rows(norm(x))."""
    _cuda(x, "x"); _cuda(weight, "weight")
    _require(x.dtype in (torch.float16, torch.bfloat16, torch.float32), "x must be float16, bfloat16 or float32")
    xv, M, K, ld = _rows_view(x)
    _require(weight.dtype == torch.float32 and weight.numel() == K and weight.is_contiguous(), "weight must be a contiguous float32 [K]")
    q = torch.empty(*x.shape[:-1], K, dtype=torch.int8, device=x.device)
    a = torch.empty(M, dtype=torch.float32, device=x.device)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    call("el_rmsnorm_quantize_rows", xv.data_ptr(), _DT[xv.dtype], ld, weight.data_ptr(), float(norm_eps), q.data_ptr(),
         a.data_ptr(), rstd.data_ptr(), M, K, float(quant_eps), _stream())
    return q, a, rstd


def rmsnorm_backward(g: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rstd: torch.Tensor):
    """Backward of the pre-linear RMSNorm for the gradient g with respect to its output (same shape and dtype as x).
    Returns (dx like x, dweight float32 [K])."""
    _cuda(g, "g"); _cuda(x, "x")
    _require(g.dtype == x.dtype and g.shape == x.shape, "g and x must have the same shape and dtype")
    K = x.shape[-1]
    gc, xc = g.contiguous(), x.contiguous()
    M = xc.numel() // K if K else 0
    _require(weight.dtype == torch.float32 and weight.numel() == K, "weight must be float32 [K]")
    _require(rstd.dtype == torch.float32 and rstd.numel() == M, "rstd must be float32 [M]")
    need = _lib.lib().el_rmsnorm_backward_workspace_bytes(K)
    key = (x.device.index, _stream(), K)       # one scratch buffer per stream: calls on different streams may overlap
    ws = _norm_ws.get(key)
    if ws is None:
        ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        _norm_ws[key] = ws
    dx = torch.empty_like(xc)
    dw = torch.empty(K, dtype=torch.float32, device=x.device)
    call("el_rmsnorm_backward", gc.data_ptr(), xc.data_ptr(), _DT[xc.dtype], weight.contiguous().data_ptr(), rstd.data_ptr(),
         dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), need, M, K, _stream())
    return dx.view_as(x), dw


def _gate_up_views(gate: torch.Tensor, up: torch.Tensor):
    """2-D views of gate and up with one common row pitch (the two halves of a [M, 2H] matrix qualify)."""
    _require(gate.dtype == up.dtype and gate.shape == up.shape, "gate and up must have the same shape and dtype")
    _require(gate.dtype in (torch.float16, torch.bfloat16, torch.float32), "gate and up must be float16, bfloat16 or float32")
    gv, M, H, ld = _rows_view(gate)
    uv, _, _, ld_u = _rows_view(up)
    if ld_u != ld:
        gv, uv, ld = gv.contiguous(), uv.contiguous(), H
    return gv, uv, M, H, ld


def swiglu_supported(gate: torch.Tensor) -> bool:
    """Shapes the fused SwiGLU kernels take: a float CUDA tensor whose hidden size is a multiple of 8 (at most 25600)
    and whose rows are 16-byte aligned."""
    return rmsnorm_supported(gate)


def sigmoid_fixed(g: torch.Tensor) -> torch.Tensor:
    """sigmoid(g) for a float32 CUDA tensor, exactly as the fused SwiGLU kernels compute it."""
    _cuda(g, "g")
    _require(g.dtype == torch.float32, "g must be float32")
    gc = g.contiguous()
    out = torch.empty_like(gc)
    call("el_sigmoid_fixed", gc.data_ptr(), out.data_ptr(), gc.numel(), _stream())
    return out


def prelinear_rows(x: torch.Tensor, up: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                   norm_eps: float = NORM_EPS) -> torch.Tensor:
    """The input of an INT2 layer as the fused training kernels form it (`silu(x) * up` when `up` is given, then the
    pre-linear RMSNorm when `norm_weight` is given), written out in x's dtype: what `linear_decode` is fed at inference."""
    _cuda(x, "x")
    if up is not None:
        _cuda(up, "up")
        xv, uv, M, K, ld = _gate_up_views(x, up)
    else:
        _require(x.dtype in (torch.float16, torch.bfloat16, torch.float32), "x must be float16, bfloat16 or float32")
        xv, M, K, ld = _rows_view(x)
        uv = None
    if norm_weight is not None:
        _require(norm_weight.dtype == torch.float32 and norm_weight.numel() == K and norm_weight.is_contiguous(),
                 "norm_weight must be a contiguous float32 [K]")
    y = torch.empty(*x.shape[:-1], K, dtype=xv.dtype, device=x.device)
    call("el_prelinear_rows", xv.data_ptr(), _ptr(uv), _DT[xv.dtype], ld, _ptr(norm_weight), float(norm_eps), y.data_ptr(), M, K,
         _stream())
    return y


def swiglu_quantize_rows(gate: torch.Tensor, up: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
                         norm_eps: float = NORM_EPS, quant_eps: float = ACT_EPS):
    """`F.silu(gate) * up` of the reference's feed-forward block (model/model.py:107-108), the pre-linear RMSNorm of the
    INT2 layer that consumes it (core/bitnet/bitnet_int2_optimized.py:201-204; skipped when `norm_weight` is None) and
    the per-token quantiser, in one pass.  Returns (q int8 like gate, absmax float32 [M], rstd float32 [M] or None)."""
    _cuda(gate, "gate"); _cuda(up, "up")
    gv, uv, M, H, ld = _gate_up_views(gate, up)
    if norm_weight is not None:
        _require(norm_weight.dtype == torch.float32 and norm_weight.numel() == H and norm_weight.is_contiguous(),
                 "norm_weight must be a contiguous float32 [H]")
    q = torch.empty(*gate.shape[:-1], H, dtype=torch.int8, device=gate.device)
    a = torch.empty(M, dtype=torch.float32, device=gate.device)
    rstd = torch.empty(M, dtype=torch.float32, device=gate.device) if norm_weight is not None else None
    call("el_swiglu_quantize_rows", gv.data_ptr(), uv.data_ptr(), _DT[gv.dtype], ld, _ptr(norm_weight), float(norm_eps),
         q.data_ptr(), a.data_ptr(), _ptr(rstd), M, H, float(quant_eps), _stream())
    return q, a, rstd


def swiglu_backward(gy: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
                    rstd: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    """Backward of swiglu_quantize_rows for the gradient gy with respect to the row that was quantised.  Returns
    (d_gate, d_up, d_norm_weight or None); with `out` (a [M, 2H] tensor of the I/O type) the two gradients are written
    into its halves (the gradient of a fused gate|up projection) and returned as views."""
    _cuda(gy, "gy"); _cuda(gate, "gate"); _cuda(up, "up")
    gv, uv, M, H, ld = _gate_up_views(gate, up)
    _require(gy.dtype == gv.dtype and gy.numel() == M * H, "gy must have the shape and dtype of gate")
    gyc = gy.contiguous()
    if out is None:
        d_gate, d_up, ld_d = torch.empty(M, H, dtype=gv.dtype, device=gv.device), torch.empty(M, H, dtype=gv.dtype, device=gv.device), H
    else:
        _require(out.dtype == gv.dtype and out.shape == (M, 2 * H) and out.is_contiguous(), "out must be a contiguous [M, 2H] tensor")
        d_gate, d_up, ld_d = out[:, :H], out[:, H:], 2 * H
    dw, ws, need = None, None, 0
    if norm_weight is not None:
        _require(norm_weight.dtype == torch.float32 and norm_weight.numel() == H, "norm_weight must be float32 [H]")
        _require(rstd is not None and rstd.dtype == torch.float32 and rstd.numel() == M, "rstd must be float32 [M]")
        need = _lib.lib().el_swiglu_backward_workspace_bytes(H)
        key = (gv.device.index, _stream(), H)
        ws = _norm_ws.get(key)
        if ws is None:
            ws = torch.empty(need, dtype=torch.uint8, device=gv.device)
            _norm_ws[key] = ws
        dw = torch.empty(H, dtype=torch.float32, device=gv.device)
        norm_weight = norm_weight.contiguous()
    call("el_swiglu_backward", gyc.data_ptr(), gv.data_ptr(), uv.data_ptr(), _DT[gv.dtype], ld, _ptr(norm_weight), _ptr(rstd),
         d_gate.data_ptr(), d_up.data_ptr(), ld_d, _ptr(dw), _ptr(ws), need, M, H, _stream())
    if out is None:
        return d_gate.view_as(gate), d_up.view_as(up), dw
    return d_gate, d_up, dw


def absmax_rows(x: torch.Tensor) -> torch.Tensor:
    """Raw max |x[m,:]| per row (float32 [M]), without the eps floor: the first half of quantize_rows for a
    column shard, to be max-reduced over ranks and passed back as `raw_absmax`."""
    _cuda(x, "x")
    _require(x.dtype in _DT and x.dtype != torch.int32, "x must be float16, bfloat16 or float32")
    xv, M, K, ld = _rows_view(x)
    a = torch.empty(M, dtype=torch.float32, device=x.device)
    call("el_quantize_rows", xv.data_ptr(), _DT[xv.dtype], ld, None, a.data_ptr(), M, K, 1.0, _lib.EL_QUANT_ABSMAX_ONLY,
         None, None, _stream())
    return a


def scale_rows(acc: torch.Tensor, row_absmax: torch.Tensor, gamma: float, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """out = acc * (row_absmax[m]/127) * gamma for int32 sums [M,C] (the GEMM epilogue as its own pass)."""
    _cuda(acc, "acc")
    _require(acc.dtype == torch.int32 and acc.dim() == 2 and acc.is_contiguous(), "acc must be a contiguous int32 [M,C]")
    M, C = acc.shape
    stride = 0 if row_absmax.numel() == 1 else 1
    _require(stride == 0 or row_absmax.numel() == M, "one absmax per row expected")
    out = torch.empty(M, C, dtype=out_dtype, device=acc.device)
    call("el_scale_rows", acc.data_ptr(), out.data_ptr(), _DT[out_dtype], row_absmax.data_ptr(), stride, float(gamma), M, C,
         _stream())
    return out


def matmul_rows(Xq: torch.Tensor, W_packed: torch.Tensor, row_absmax: torch.Tensor, gamma: float,
                out_dtype: torch.dtype = torch.bfloat16, path: int = EL_PATH_AUTO) -> torch.Tensor:
    """Y[m,:] = (Xq[m,:] @ W^T) * (row_absmax[m]/127) * gamma: the forward GEMM with per-token scales."""
    return _gemm_fwd(Xq, W_packed, row_absmax, 1, gamma, out_dtype, path)


def matmul_rows_gather(Xq: torch.Tensor, W_packed: torch.Tensor, row_absmax: torch.Tensor, gamma: float,
                       out_ptrs, ld_total: int, col_offset: int, out_dtype: torch.dtype = torch.bfloat16) -> None:
    """Forward GEMM of an N-shard whose epilogue writes the result into column window `col_offset` of every rank's
    [M, ld_total] output buffer (`out_ptrs`: device addresses, own buffer and peer mappings): a fused all-gather."""
    _cuda(Xq, "X_int8"); _cuda(W_packed, "W_packed"); _cuda(row_absmax, "row_absmax")
    _require(Xq.dtype == torch.int8 and W_packed.dtype == torch.uint8, "Xq must be int8 and W_packed uint8")
    N, pK = W_packed.shape
    K = Xq.shape[-1]
    _require((K + 3) // 4 == pK, f"X has {K} features but W_packed has packed_K={pK}")
    Xf = Xq.contiguous().view(-1, K)
    M = Xf.shape[0]
    _require(row_absmax.numel() == M, "one absmax per token expected")
    keep, arr = _ptr_array(out_ptrs)
    st = device_status(Xq.device)
    call("el_gemm_fwd_gather", Xf.data_ptr(), W_packed.contiguous().data_ptr(), arr, len(out_ptrs),
         int(ld_total), int(col_offset), _DT[out_dtype], row_absmax.data_ptr(), 1, float(gamma), M, N, K, st.data_ptr(), _stream())
    _maybe_check(Xq.device)


def _ptr_array(ptrs):
    import ctypes
    arr = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr, ctypes.cast(arr, ctypes.c_void_p)


def backward_input_scatter(dYq: torch.Tensor, W_packed: torch.Tensor, K: int, parts_ptrs, rank: int) -> None:
    """dX GEMM of an N-shard whose epilogue scatters the int32 partial sums: token rows owned by rank d go to slot
    `rank` of rank d's staging buffer [n_ranks, M/n_ranks, K] (`parts_ptrs`: device addresses, own and peer mappings)."""
    _cuda(dYq, "dY_int8"); _cuda(W_packed, "W_packed")
    _require(dYq.dtype == torch.int8 and W_packed.dtype == torch.uint8, "dYq must be int8 and W_packed uint8")
    N = W_packed.shape[0]
    Yf = dYq.contiguous().view(-1, N)
    M = Yf.shape[0]
    keep, arr = _ptr_array(parts_ptrs)
    st = device_status(dYq.device)
    call("el_gemm_dx_scatter", Yf.data_ptr(), W_packed.contiguous().data_ptr(), arr, len(parts_ptrs), int(rank), M, N, int(K),
         st.data_ptr(), _stream())
    _maybe_check(dYq.device)


def reduce_scale_gather(parts: torch.Tensor, out_ptrs, rank: int, row_absmax: torch.Tensor, gamma: float, M: int, K: int,
                        out_dtype: torch.dtype = torch.bfloat16) -> None:
    """Owner side of the dX reduction: sums this rank's [n_ranks, M/n_ranks, K] int32 partials, scales them and writes
    the rows into every rank's dX [M, K] (`out_ptrs`).  `row_absmax` holds the absmax of all M tokens."""
    _cuda(parts, "parts")
    _require(parts.dtype == torch.int32 and parts.is_contiguous(), "parts must be a contiguous int32 tensor")
    _require(row_absmax.dtype == torch.float32 and row_absmax.numel() == M, "row_absmax must be float32 [M]")
    keep, arr = _ptr_array(out_ptrs)
    call("el_reduce_scale_gather", parts.data_ptr(), arr, len(out_ptrs), int(rank), _DT[out_dtype], row_absmax.data_ptr(),
         float(gamma), int(M), int(K), _stream())


def peer_barrier(flag_ptrs, rank: int, epoch: int, device: torch.device) -> None:
    """Barrier number `epoch` (1, 2, ... in the same order on every rank) between the ranks whose flag arrays
    (uint32 [n_ranks] each, peer-mapped, zeroed before the first barrier) are `flag_ptrs`: one small kernel on the
    current stream; a rank that does not arrive within seconds shows up in check_device_status."""
    keep, arr = _ptr_array(flag_ptrs)
    st = device_status(device)
    call("el_peer_barrier", arr, len(flag_ptrs), int(rank), int(epoch) & 0xFFFFFFFF, st.data_ptr(), _stream())


def peer_barrier_put(flag_ptrs, rank: int, epoch: int, device: torch.device, word: torch.Tensor, dst_ptrs, dst_offset_bytes: int) -> None:
    """peer_barrier that first delivers the 4-byte tensor `word` to byte offset `dst_offset_bytes` of every rank's buffer in
    `dst_ptrs`: after it, every rank holds every rank's word."""
    _cuda(word, "word")
    _require(word.numel() * word.element_size() == 4, "word must hold exactly four bytes")
    keep, arr = _ptr_array(flag_ptrs)
    keep2, arr2 = _ptr_array(dst_ptrs)
    st = device_status(device)
    call("el_peer_barrier_put", arr, len(flag_ptrs), int(rank), int(epoch) & 0xFFFFFFFF, st.data_ptr(), word.data_ptr(), arr2,
         int(dst_offset_bytes), _stream())


def peer_barrier_next(flag_ptrs, rank: int, device: torch.device, word: Optional[torch.Tensor] = None, dst_ptrs=None,
                      dst_offset_bytes: int = 0) -> None:
    """peer_barrier / peer_barrier_put whose epoch is one more than the epoch this rank published last (read by the kernel
    from the rank's own flag array): a launch that can be recorded in a CUDA graph and replayed."""
    keep, arr = _ptr_array(flag_ptrs)
    st = device_status(device)
    if word is None:
        call("el_peer_barrier_next", arr, len(flag_ptrs), int(rank), st.data_ptr(), None, None, 0, _stream())
        return
    _cuda(word, "word")
    _require(word.numel() * word.element_size() == 4, "word must hold exactly four bytes")
    keep2, arr2 = _ptr_array(dst_ptrs)
    call("el_peer_barrier_next", arr, len(flag_ptrs), int(rank), st.data_ptr(), word.data_ptr(), arr2, int(dst_offset_bytes),
         _stream())


def counter_add(counter: torch.Tensor, delta: int = 1) -> None:
    """counter[0] += delta on the device, in stream order (int32 [1])."""
    _cuda(counter, "counter")
    _require(counter.dtype == torch.int32 and counter.numel() == 1, "counter must be int32 [1]")
    call("el_counter_add", counter.data_ptr(), int(delta), _stream())


def backward_input_rows(dYq: torch.Tensor, W_packed: torch.Tensor, row_absmax: torch.Tensor, gamma: float, K: int,
                        out_dtype: torch.dtype = torch.bfloat16, path: int = EL_PATH_AUTO) -> torch.Tensor:
    """dX[m,:] = (dYq[m,:] @ W) * (row_absmax[m]/127) * gamma: the dX GEMM with per-token scales."""
    return _gemm_dx(dYq, W_packed, row_absmax, 1, gamma, K, out_dtype, path)


def quantize_grad(dY: torch.Tensor, x_absmax: torch.Tensor, g_absmax: torch.Tensor) -> torch.Tensor:
    """Gq = int8 of (dY * x_absmax[m]/127) under the per-tensor maximum g_absmax[1]; a 2-D column window of a
    wider dY is read in place."""
    _cuda(dY, "dY")
    yv, M, N, ld = _rows_view(dY)
    _require(x_absmax.dtype == torch.float32 and x_absmax.numel() == M, "x_absmax must be float32 [M]")
    _require(g_absmax.dtype == torch.float32 and g_absmax.numel() == 1, "g_absmax must be float32 [1]")
    Gq = torch.empty(*dY.shape[:-1], N, dtype=torch.int8, device=dY.device)
    call("el_quantize_grad", yv.data_ptr(), _DT[yv.dtype], ld, x_absmax.data_ptr(), g_absmax.data_ptr(), Gq.data_ptr(), M, N,
         _stream())
    return Gq


def quantize_grad_scatter(dY: torch.Tensor, x_absmax: torch.Tensor, g_slots: torch.Tensor, recv_ptrs, row_offset: int,
                          g_out: Optional[torch.Tensor] = None) -> None:
    """quantize_grad of this rank's gradient rows whose output is the all-to-all: column window d of every row goes to row
    `row_offset + m` of rank d's receive buffer [M_total, N/g] (`recv_ptrs`: device addresses, own buffer and peer
    mappings).  `g_slots` holds the ranks' partial maxima; their maximum is the scale and lands in `g_out` [1]."""
    _cuda(dY, "dY")
    yv, M, N, ld = _rows_view(dY)
    _require(x_absmax.dtype == torch.float32 and x_absmax.numel() == M, "x_absmax must be float32 [M]")
    _require(g_slots.dtype == torch.float32 and g_slots.is_contiguous(), "g_slots must be a contiguous float32 tensor")
    keep, arr = _ptr_array(recv_ptrs)
    call("el_quantize_grad_scatter", yv.data_ptr(), _DT[yv.dtype], ld, x_absmax.data_ptr(), g_slots.data_ptr(), g_slots.numel(),
         _ptr(g_out), arr, len(recv_ptrs), int(row_offset), M, N, _stream())


def peer_put(src: torch.Tensor, dst_ptrs, dst_offset_bytes: int, max_ctas: int = 0) -> None:
    """Copies the contiguous tensor `src` to byte offset `dst_offset_bytes` of every buffer in `dst_ptrs` (device
    addresses of peer mappings): one rank's push of an all-gather, as plain stores over NVLink from one kernel
    (`max_ctas` >= 0: its grid limit, 0 = as many as saturate the links) or, with `max_ctas` < 0, as one copy-engine
    copy per destination in the order given."""
    _cuda(src, "src")
    _require(src.is_contiguous(), "src must be contiguous")
    if len(dst_ptrs) == 0 or src.numel() == 0:
        return
    keep, arr = _ptr_array(dst_ptrs)
    if max_ctas < 0:
        call("el_peer_put_dma", src.data_ptr(), arr, len(dst_ptrs), int(dst_offset_bytes), src.numel() * src.element_size(),
             _stream())
        return
    call("el_peer_put", src.data_ptr(), arr, len(dst_ptrs), int(dst_offset_bytes), src.numel() * src.element_size(),
         int(max_ctas), _stream())


def weight_grad(Gq: torch.Tensor, Xq: torch.Tensor, g_absmax: torch.Tensor, raw: bool = False,
                path: int = EL_PATH_AUTO) -> torch.Tensor:
    """dW[n,k] = (sum_m Gq[m,n]*Xq[m,k]) * (g_absmax/127) as float32 [N,K] (int32 sums when raw=True)."""
    _cuda(Gq, "Gq"); _cuda(Xq, "Xq")
    _require(Gq.dtype == torch.int8 and Xq.dtype == torch.int8, "Gq and Xq must be int8")
    N, K = Gq.shape[-1], Xq.shape[-1]
    G2, X2 = Gq.contiguous().view(-1, N), Xq.contiguous().view(-1, K)
    M = G2.shape[0]
    _require(X2.shape[0] == M, "Gq and Xq must have the same number of tokens")
    dt = torch.int32 if raw else torch.float32
    dW = torch.empty(N, K, dtype=dt, device=Gq.device)
    st = device_status(Gq.device)
    call("el_gemm_dw", G2.data_ptr(), X2.data_ptr(), dW.data_ptr(), _DT[dt], g_absmax.data_ptr(), M, N, K, path,
         st.data_ptr(), _stream())
    _maybe_check(Gq.device)
    return dW


def dw_hysteresis_supported(N: int, K: int) -> bool:
    """Shapes the fused weight-gradient + hysteresis kernel takes (others use weight_grad + hysteresis_step_v2)."""
    return N % 16 == 0 and K % 32 == 0


def dw_hysteresis(Gq: torch.Tensor, Xq: torch.Tensor, g_absmax: torch.Tensor, W_packed: torch.Tensor,
                  H_packed: torch.Tensor, lr: float, lr_scale: float, threshold: int, decay: float, step,
                  idx_base: int = 0) -> None:
    """Fused weight-gradient GEMM + hysteresis update, in place on W_packed / H_packed.  `step`: the step number, or an
    int32 [1] CUDA tensor that holds it (for launches recorded in a CUDA graph; see counter_add)."""
    _cuda(Gq, "Gq"); _cuda(Xq, "Xq")
    _require(Gq.dtype == torch.int8 and Xq.dtype == torch.int8, "Gq and Xq must be int8")
    N, K = Gq.shape[-1], Xq.shape[-1]
    G2, X2 = Gq.contiguous().view(-1, N), Xq.contiguous().view(-1, K)
    M = G2.shape[0]
    _require(X2.shape[0] == M, "Gq and Xq must have the same number of tokens")
    _require(tuple(W_packed.shape) == (N, (K + 3) // 4) and tuple(H_packed.shape) == (N, (K + 1) // 2),
             "W_packed / H_packed shape mismatch")
    _require(W_packed.is_contiguous() and H_packed.is_contiguous(), "W_packed/H_packed must be contiguous")
    st = device_status(Gq.device)
    if isinstance(step, torch.Tensor):          # the step number is read from device memory when the kernel runs
        _cuda(step, "step")
        _require(step.dtype == torch.int32 and step.numel() == 1, "a step tensor must be int32 [1]")
        call("el_dw_hysteresis_step_ptr", G2.data_ptr(), X2.data_ptr(), g_absmax.data_ptr(), W_packed.data_ptr(),
             H_packed.data_ptr(), float(lr), float(lr_scale), int(threshold), float(decay), step.data_ptr(),
             int(idx_base) & 0xFFFFFFFF, M, N, K, st.data_ptr(), _stream())
        return
    step32 = int(step) & 0xFFFFFFFF
    step_i = step32 - (1 << 32) if step32 >= (1 << 31) else step32
    call("el_dw_hysteresis", G2.data_ptr(), X2.data_ptr(), g_absmax.data_ptr(), W_packed.data_ptr(), H_packed.data_ptr(),
         float(lr), float(lr_scale), int(threshold), float(decay), step_i, int(idx_base) & 0xFFFFFFFF, M, N, K,
         st.data_ptr(), _stream())
    _maybe_check(Gq.device)


_decode_ws: dict = {}


def linear_decode(x: torch.Tensor, W_packed: torch.Tensor, gamma: float, out_dtype: Optional[torch.dtype] = None,
                  workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Small-M layer call (1 <= M <= 64 tokens): per-token quantisation + the weight-streaming tensor-core kernel.
    Same integers and rounding as quantize_rows + matmul_rows.  `workspace` (uint8, zero before first use, left
    zero) defaults to a cached buffer per device, stream and N, so calls on different streams never share one."""
    _cuda(x, "x"); _cuda(W_packed, "W_packed")
    _require(x.dtype in (torch.float16, torch.bfloat16, torch.float32), "x must be float16, bfloat16 or float32")
    _require(W_packed.dtype == torch.uint8 and W_packed.dim() == 2, "W_packed must be uint8 [N, ceil(K/4)]")
    N, pK = W_packed.shape
    K = x.shape[-1]
    _require((K + 3) // 4 == pK, f"x has {K} features but W_packed has packed_K={pK}")
    xc = x.contiguous().view(-1, K)
    M = xc.shape[0]
    _require(1 <= M <= 64, "linear_decode takes 1..64 tokens; use quantize_rows + matmul_rows beyond that")
    out_dtype = out_dtype or x.dtype
    need = _lib.lib().el_decode_workspace_bytes(N)
    if workspace is None:
        key = (x.device.index, _stream(), N)       # per stream: calls that share a workspace must be stream-ordered
        workspace = _decode_ws.get(key)
        if workspace is None:
            workspace = torch.zeros(need, dtype=torch.uint8, device=x.device)
            _decode_ws[key] = workspace
    _require(workspace.is_cuda and workspace.numel() * workspace.element_size() >= need, "workspace too small")
    xq = torch.empty(M, K, dtype=torch.int8, device=x.device)
    a = torch.empty(M, dtype=torch.float32, device=x.device)
    Y = torch.empty(M, N, dtype=out_dtype, device=x.device)
    st = device_status(x.device)
    call("el_linear_decode", xc.data_ptr(), _DT[xc.dtype], W_packed.contiguous().data_ptr(), Y.data_ptr(), _DT[out_dtype],
         float(gamma), xq.data_ptr(), a.data_ptr(), workspace.data_ptr(), workspace.numel() * workspace.element_size(),
         M, N, K, st.data_ptr(), _stream())
    _maybe_check(x.device)
    return Y.view(*x.shape[:-1], N)


def set_decode_overlap(enable: bool) -> None:
    """Lets consecutive small-M decode calls (up to the GEMV token limit) overlap: the call is issued as a programmatic
    dependent launch that loads its packed weights while earlier work of the stream finishes, and reads x / writes Y
    only afterwards.  Only valid while nothing queued on the stream writes W_packed (inference).  Process-wide."""
    call("el_set_decode_overlap", 1 if enable else 0)


def linear_decode_static(x: torch.Tensor, W_packed: torch.Tensor, gamma: float, out: torch.Tensor) -> torch.Tensor:
    """linear_decode for hosts that cannot allocate device memory: the library call behind it keeps its scratch in
    a static device array (M <= 64, N <= 16384, K <= 16384) and writes into the caller's `out` [M, N].  Calls on one
    device share that array: keep them stream-ordered.  Make the first call on a device outside stream capture."""
    _cuda(x, "x"); _cuda(W_packed, "W_packed"); _cuda(out, "out")
    _require(x.dtype in (torch.float16, torch.bfloat16, torch.float32) and x.is_contiguous(), "x must be a contiguous float tensor")
    _require(W_packed.dtype == torch.uint8 and W_packed.dim() == 2 and W_packed.is_contiguous(), "W_packed must be contiguous uint8 [N, ceil(K/4)]")
    N, pK = W_packed.shape
    K = x.shape[-1]
    M = math.prod(x.shape[:-1])
    _require((K + 3) // 4 == pK, f"x has {K} features but W_packed has packed_K={pK}")
    _require(out.is_contiguous() and out.numel() == M * N and out.dtype in (torch.float16, torch.bfloat16, torch.float32),
             "out must be a contiguous float tensor of M*N elements")
    st = device_status(x.device)
    call("el_linear_decode_static", x.data_ptr(), _DT[x.dtype], W_packed.data_ptr(), out.data_ptr(), _DT[out.dtype],
         float(gamma), M, N, K, st.data_ptr(), _stream())
    _maybe_check(x.device)
    return out
