"""The timed CPU baseline of the layer step (TEST / BENCHMARK INFRASTRUCTURE ONLY).

A port of the reference's CPU-runnable layer, model/common/bitnet_legacy.py:58-141 (BitLinear: per-token
absmax fake-quantisation of the activations, absmean ternary fake-quantisation of the weights, F.linear,
straight-through backward giving dX and dW), followed by the C restatement of the hysteresis kernel
(oracle/int2_oracle.c, after kernels/int2/int2_hysteresis_v2.cu:54-152), which the reference only has in CUDA.
The layer's RMSNorm is left out on both sides of the comparison: the GPU step starts at the quantiser too.
Every step is timed on ALL tokens of the workload (nothing is extrapolated), in bfloat16 and in float32 (the
reference's layer is not tied to a dtype, and host cores without bfloat16 units run float32 faster); the caller
reports the faster one.  The thread count is set explicitly, because launchers such as torch.distributed.run export
OMP_NUM_THREADS=1.
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch
import torch.nn.functional as F

from . import int2_oracle as O
from . import native


def use_all_cores() -> int:
    """All host cores for torch's and the C library's loops; returns the count in use."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(n)
    native.oracle_lib().oracle_set_num_threads(n)
    return n


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

    def __init__(self, K: int, N: int, seed: int, counters: int = 3):
        g = torch.Generator().manual_seed(seed)
        self.K, self.N = K, N
        self.master = torch.randn(N, K, generator=g) * 0.02
        self.weights = {}
        w32 = self.master.numpy()
        gamma = O.absmean_scale(w32)
        self.W_packed = O.pack_ternary(O.ternarize(w32, gamma))
        rng = np.random.default_rng(seed)
        self.H_packed = O.pack_counters(rng.integers(-counters, counters + 1, (N, K)).astype(np.int8))
        self.step = 0

    def weight(self, dtype: torch.dtype) -> torch.Tensor:
        if dtype not in self.weights:
            self.weights[dtype] = self.master.to(dtype).requires_grad_(True)
        return self.weights[dtype]

    def gemm_part(self, x: torch.Tensor, dY: torch.Tensor):
        """forward + backward (dX, dW) on the given tokens; returns dW float32 [N,K]."""
        w = self.weight(x.dtype)
        w.grad = None
        xin = x.detach().requires_grad_(True)
        y = F.linear(_activation_quant(xin), _weight_quant(w))
        y.backward(dY)
        return w.grad.float().numpy()

    def hysteresis_part(self, dW: np.ndarray, lr: float, threshold: int):
        self.step += 1
        lib = native.oracle_lib()
        lib.oracle_hysteresis_step(np.ascontiguousarray(dW, dtype=np.float32), self.W_packed, self.H_packed, lr, 5.0,
                                   int(threshold), 0.001, self.step, self.N, self.K, 0, 1)


def time_step(layers, M: int, dtype: torch.dtype, lr: float = 1e-2, threshold: int = 3, seed: int = 0, dy_std: float = 1e-3):
    """One full layer step on all M tokens in `dtype`: forward, dX, dW (torch) and the hysteresis update of every weight
    (C).  Returns the wall-clock seconds of the step (input generation excluded)."""
    g = torch.Generator().manual_seed(seed)
    total = 0.0
    for layer in layers:
        x = torch.randn(M, layer.K, generator=g).to(dtype)
        dY = (torch.randn(M, layer.N, generator=g) * dy_std).to(dtype)
        t0 = time.perf_counter()
        dW = layer.gemm_part(x, dY)
        layer.hysteresis_part(dW, lr, threshold)
        total += time.perf_counter() - t0
    return total


def cores_used() -> int:
    return max(torch.get_num_threads(), native.oracle_lib().oracle_num_threads())
