"""The timed CPU baseline of the layer step (TEST / BENCHMARK INFRASTRUCTURE ONLY).

A port of the reference's CPU-runnable layer, model/common/bitnet_legacy.py:58-141 (BitLinear: per-token
absmax fake-quantisation of the activations, absmean ternary fake-quantisation of the weights, F.linear,
straight-through backward giving dX and dW), followed by the C restatement of the hysteresis kernel
(oracle/int2_oracle.c, after kernels/int2/int2_hysteresis_v2.cu:54-152), which the reference only has in CUDA.
The layer's RMSNorm is left out on both sides of the comparison: the GPU step starts at the quantiser too.
Runs on all host threads torch and OpenMP give it.
"""
from __future__ import annotations

import time

import numpy as np
import torch
import torch.nn.functional as F

from . import int2_oracle as O
from . import native


def _activation_quant(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    x32 = x.float()
    scale = 127.0 / x32.abs().max(dim=-1, keepdim=True).values.clamp_(min=eps)
    xq = (x32 * scale).round().clamp_(-128, 127) / scale
    return x + (xq.to(x.dtype) - x).detach()


def _weight_quant(w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    w32 = w.float()
    gamma = torch.clamp(w32.abs().mean(), min=eps)
    wq = torch.clamp(torch.round(w32 / gamma), -1, 1) * gamma
    return w + (wq.to(w.dtype) - w).detach()


class CpuLayer:
    """One [N,K] layer: latent float weights for the torch part, packed state for the hysteresis part."""

    def __init__(self, K: int, N: int, dtype: torch.dtype, seed: int, counters: int = 3):
        g = torch.Generator().manual_seed(seed)
        self.K, self.N, self.dtype = K, N, dtype
        self.weight = (torch.randn(N, K, generator=g) * 0.02).to(dtype).requires_grad_(True)
        w32 = self.weight.detach().float().numpy()
        gamma = O.absmean_scale(w32)
        self.W_packed = O.pack_ternary(O.ternarize(w32, gamma))
        rng = np.random.default_rng(seed)
        self.H_packed = O.pack_counters(rng.integers(-counters, counters + 1, (N, K)).astype(np.int8))
        self.step = 0

    def gemm_part(self, x: torch.Tensor, dY: torch.Tensor):
        """forward + backward (dX, dW) on the given tokens; returns dW float32 [N,K]."""
        self.weight.grad = None
        xin = x.detach().requires_grad_(True)
        y = F.linear(_activation_quant(xin), _weight_quant(self.weight))
        y.backward(dY)
        return self.weight.grad.float().numpy()

    def hysteresis_part(self, dW: np.ndarray, lr: float, threshold: int):
        self.step += 1
        lib = native.oracle_lib()
        lib.oracle_hysteresis_step(np.ascontiguousarray(dW, dtype=np.float32), self.W_packed, self.H_packed, lr, 5.0,
                                   int(threshold), 0.001, self.step, self.N, self.K, 0, 1)


def time_step(layers, M_full: int, M_sample: int, dtype: torch.dtype, lr: float = 1e-2, threshold: int = 3, seed: int = 0):
    """Times one layer step on a bounded sample: the torch part (forward, dX, dW) on M_sample tokens, scaled to
    M_full tokens, plus the hysteresis update of the whole weight matrix (its cost does not depend on M).
    Returns (seconds per full step, seconds of CPU time actually spent)."""
    g = torch.Generator().manual_seed(seed)
    t_gemm = 0.0
    t_hyst = 0.0
    for layer in layers:
        x = torch.randn(M_sample, layer.K, generator=g).to(dtype)
        dY = (torch.randn(M_sample, layer.N, generator=g) * 1e-3).to(dtype)
        t0 = time.perf_counter()
        dW = layer.gemm_part(x, dY)
        t1 = time.perf_counter()
        layer.hysteresis_part(dW, lr, threshold)
        t2 = time.perf_counter()
        t_gemm += t1 - t0
        t_hyst += t2 - t1
    return t_gemm * (M_full / M_sample) + t_hyst, t_gemm + t_hyst


def cores_used() -> int:
    return max(torch.get_num_threads(), native.oracle_lib().oracle_num_threads())
