"""A stand-in for the package's operator module that computes with the CPU oracle on CPU tensors, so that the
host-side logic built on top of the operators (the N-sharded layer and its collectives) can be tested without
a GPU.  Test infrastructure only."""
import numpy as np
import torch

from oracle import int2_oracle as O
from oracle import native

_RND = {torch.bfloat16: O.to_bf16, torch.float16: O.to_f16, torch.float32: lambda v: v}


def _n(t):
    t = t.detach()
    return (t.float() if t.dtype in (torch.bfloat16, torch.float16) else t).contiguous().numpy()


def ternarize_pack(weight, gamma):
    return torch.from_numpy(O.pack_ternary(O.ternarize(_n(weight), gamma), pad_code=0))


def quantize_rows(x, eps=1e-5, fold_absmax=None, raw_absmax=None, out=None):
    xn = _n(x)
    xn = np.where(np.isfinite(xn), xn, np.float32(0))
    raw = np.abs(xn).max(axis=1).astype(np.float32) if raw_absmax is None else _n(raw_absmax).copy()
    a = np.maximum(raw, np.float32(eps)).astype(np.float32)
    s = (np.float32(127.0) / a).astype(np.float32)
    q = np.clip(np.rint(xn * s[:, None]), -128, 127).astype(np.int8)
    if out is not None:
        out.copy_(torch.from_numpy(q))
    if raw_absmax is not None:
        raw_absmax.copy_(torch.from_numpy(a))
    at = raw_absmax if raw_absmax is not None else torch.from_numpy(a)
    qt = out if out is not None else torch.from_numpy(q)
    if fold_absmax is None:
        return qt, at
    sx = (_n(fold_absmax) / np.float32(127.0)).astype(np.float32)
    g = np.float32((raw * sx).astype(np.float32).max())
    return qt, at, torch.tensor([g], dtype=torch.float32)


def absmax_rows(x):
    xn = _n(x)
    xn = np.where(np.isfinite(xn), xn, np.float32(0))
    return torch.from_numpy(np.abs(xn).max(axis=1).astype(np.float32))


def matmul_rows(Xq, W_packed, row_absmax, gamma, out_dtype=torch.bfloat16, path=0):
    K = Xq.shape[-1]
    acc = O.gemm_fwd_acc(_n(Xq), _n(W_packed), K)
    if out_dtype == torch.int32:
        return torch.from_numpy(acc)
    return torch.from_numpy(_RND[out_dtype](O.scale_rows(acc, _n(row_absmax), gamma))).to(out_dtype)


def backward_input_rows(dYq, W_packed, row_absmax, gamma, K, out_dtype=torch.bfloat16, path=0):
    acc = O.gemm_dx_acc(_n(dYq), _n(W_packed), K)
    if out_dtype == torch.int32:
        return torch.from_numpy(acc)
    return torch.from_numpy(_RND[out_dtype](O.scale_rows(acc, _n(row_absmax), gamma))).to(out_dtype)


def scale_rows(acc, row_absmax, gamma, out_dtype=torch.bfloat16):
    return torch.from_numpy(_RND[out_dtype](O.scale_rows(_n(acc), _n(row_absmax), gamma))).to(out_dtype)


def quantize_grad(dY, x_absmax, g_absmax):
    Gq, _ = O.grad_quantize(_n(dY), _n(x_absmax), g_absmax=_n(g_absmax)[0])
    return torch.from_numpy(Gq)


def weight_grad(Gq, Xq, g_absmax, raw=False, path=0):
    acc = O.gemm_dw_acc(_n(Gq), _n(Xq))
    return torch.from_numpy(acc if raw else O.dw_from_acc(acc, _n(g_absmax)[0]))


def hysteresis_step_v2(dW, W_packed, H_packed, lr, lr_scale, threshold, decay, step, idx_base=0, ftz=True):
    K = dW.shape[1]
    W, H = native.c_hysteresis_step(_n(dW), _n(W_packed), _n(H_packed), lr, lr_scale, threshold, decay, step, K,
                                    idx_base=idx_base, ftz=ftz)
    W_packed.copy_(torch.from_numpy(W))
    H_packed.copy_(torch.from_numpy(H))


def dw_hysteresis_supported(N, K):
    return False
