"""INT2 linear layer and its autograd function, with the reference's names and state layout.

Mirrors core/bitnet/int2_linear_tc.py (Int2LinearTCFunction :239-305, Int2LinearTC :308-649,
Int2LinearTCWithGradHook :652-676) and the grad-hook / accumulation gate of
core/bitnet/int2_linear_tc_offload.py (:289-371).  Buffers and parameters keep the reference's names and
shapes (`W_packed` uint8 [N, ceil(K/4)], `H_packed` uint8 [N, ceil(K/2)], `gamma` [1], `bias`, `_step`),
so a reference checkpoint loads unchanged.

Two quantisation modes:
  * "per_token" (default): activations and output gradients get one absmax scale per token, any of
    bf16 / fp16 / fp32 in and out; the weight gradient is an exact int8 GEMM fused with the hysteresis update.
  * "per_tensor": the reference CUDA path's rule (one absmax per tensor, fp16 in and out).

The 2:4-sparsity and Hadamard-INT4 options of the reference layer are outside this path and raise.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
from torch.autograd import Function

from . import int2_tc_ops
from .int2_tc_ops import ACT_EPS, GRAD_EPS

HAS_TC_OPS = True
HAS_INT2_OPS = True

_FLOAT_IO = (torch.float16, torch.bfloat16, torch.float32)


class Int2LinearTCFunction(Function):
    """Y = Q(X) . W^T scaled by gamma; backward gives dX = Q(dY) . W scaled by gamma; gamma gets no gradient
    (core/bitnet/int2_linear_tc.py:255-305).  `layer`, when given, selects the quantisation mode, receives the
    quantised activation for the later weight update and orders that update against dX."""

    _absmax_bufs: dict = {}

    @staticmethod
    def _get_absmax_buf(device: torch.device) -> torch.Tensor:
        key = str(device)
        if key not in Int2LinearTCFunction._absmax_bufs:
            Int2LinearTCFunction._absmax_bufs[key] = torch.zeros(1, dtype=torch.float32, device=device)
        return Int2LinearTCFunction._absmax_bufs[key]

    @staticmethod
    def forward(ctx, X: torch.Tensor, W_packed: torch.Tensor, gamma: torch.Tensor, K: int,
                gamma_cached: Optional[float] = None, layer: Optional["Int2LinearTC"] = None,
                norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 1e-6,
                up: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`norm_weight` (per-token mode): the weight of the reference's pre-linear RMSNorm
        (core/bitnet/bitnet_int2_optimized.py:72-86,203-204); normalisation and quantisation then run as one kernel
        over X and the backward pass returns the gradients of X and of the norm weight.
        `up` (per-token mode): X is the gate projection's output and the layer's input is `silu(X) * up`, the
        reference's feed-forward expression (model/model.py:107-108); the product, the norm and the quantiser run as
        one kernel, and the backward pass returns the gradients of X and of `up`."""
        ctx.has_norm = False
        ctx.has_gate = False
        ctx.K = K
        ctx.gamma_cached = gamma_cached
        ctx.layer = layer
        mode = layer.quant_mode if layer is not None else "per_tensor"
        ctx.mode = mode
        gamma_val = gamma_cached if gamma_cached is not None else gamma.item()
        if mode == "per_token":
            out_dtype = X.dtype if X.dtype in _FLOAT_IO else torch.bfloat16
            ctx.io_dtype = out_dtype
            Xin = X if X.dtype in _FLOAT_IO else X.to(out_dtype)
            if up is not None:
                if up.dtype != Xin.dtype or up.shape != Xin.shape:
                    raise RuntimeError("gate and up must have the same shape and dtype")
                Xq, ax, rstd = int2_tc_ops.swiglu_quantize_rows(Xin, up, norm_weight, norm_eps, ACT_EPS)
                ctx.has_gate = True
                ctx.has_norm = norm_weight is not None
                if ctx.has_norm:
                    ctx.save_for_backward(W_packed, gamma, Xin, up, norm_weight, rstd)
                else:
                    ctx.save_for_backward(W_packed, gamma, Xin, up)
            elif norm_weight is not None:
                Xin = Xin.contiguous()
                Xq, ax, rstd = int2_tc_ops.rmsnorm_quantize_rows(Xin, norm_weight, norm_eps, ACT_EPS)
                ctx.has_norm = True
                ctx.save_for_backward(W_packed, gamma, Xin, norm_weight, rstd)
            else:
                Xq, ax = int2_tc_ops.quantize_rows(Xin, ACT_EPS)
                ctx.save_for_backward(W_packed, gamma)
            if layer is not None and layer.training:
                layer._saved_input = (Xq, ax)
                layer._saved_input_shape = X.shape
            return int2_tc_ops.matmul_rows(Xq, W_packed, ax, gamma_val, out_dtype)
        if norm_weight is not None or up is not None:
            raise RuntimeError("the fused pre-linear RMSNorm and SwiGLU gate need quant_mode='per_token'")
        ctx.save_for_backward(W_packed, gamma)
        X_half = X.half() if X.dtype != torch.float16 else X
        ctx.io_dtype = torch.float16
        X_int8, d_scale_x = int2_tc_ops.quantize_activation_async(X_half.contiguous(),
                                                                  Int2LinearTCFunction._get_absmax_buf(X.device))
        if layer is not None and layer.training:
            layer._saved_input = (X_int8, d_scale_x)
            layer._saved_input_shape = X_half.shape
        return int2_tc_ops.matmul_int8(X_int8, W_packed, d_scale_x, gamma_val)

    @staticmethod
    def backward(ctx, dY: torch.Tensor) -> Tuple[Optional[torch.Tensor], ...]:
        saved = ctx.saved_tensors        # read once: under activation checkpointing a second read is an error
        W_packed, gamma = saved[:2]
        layer = ctx.layer
        dX = None
        d_norm_weight = None
        d_up = None
        if ctx.needs_input_grad[0] or (ctx.has_norm and ctx.needs_input_grad[6]) or (ctx.has_gate and ctx.needs_input_grad[8]):
            gamma_val = ctx.gamma_cached if ctx.gamma_cached is not None else gamma.item()
            if ctx.mode == "per_token":
                cached = layer._take_dy_cache(dY) if layer is not None else None
                if cached is None:
                    dYc = dY if dY.dtype in _FLOAT_IO else dY.to(ctx.io_dtype)
                    dYq, ady = int2_tc_ops.quantize_rows(dYc, GRAD_EPS)
                else:
                    dYq, ady = cached
                dX = int2_tc_ops.backward_input_rows(dYq, W_packed, ady, gamma_val, ctx.K, ctx.io_dtype)
            else:
                dY_half = dY.half() if dY.dtype != torch.float16 else dY
                dY_int8, d_scale_dy = int2_tc_ops.quantize_activation_async(
                    dY_half.contiguous(), Int2LinearTCFunction._get_absmax_buf(dY.device))
                dX = int2_tc_ops.backward_input_int8(dY_int8, W_packed, d_scale_dy, gamma_val, ctx.K)
            if ctx.has_gate:
                gate, up = saved[2:4]
                norm_weight, rstd = saved[4:6] if ctx.has_norm else (None, None)
                dX, d_up, d_norm_weight = int2_tc_ops.swiglu_backward(dX.view_as(gate), gate, up, norm_weight, rstd)
            elif ctx.has_norm:
                Xin, norm_weight, rstd = saved[2:]
                dX, d_norm_weight = int2_tc_ops.rmsnorm_backward(dX.view_as(Xin), Xin, norm_weight, rstd)
        if layer is not None:
            layer._run_pending_update()
        return dX, None, None, None, None, None, d_norm_weight, None, d_up


class Int2LinearTC(nn.Module):
    """Linear layer over 2-bit packed ternary weights with int4 hysteresis counters
    (core/bitnet/int2_linear_tc.py:308-649): 0.25 + 0.5 bytes per weight."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, threshold: int = 7,
                 lr_scale: float = 5.0, decay_rate: float = 0.001, compress_activations: bool = True,
                 use_24_sparsity: bool = False, use_hadamard_int4: bool = False, quant_mode: str = "per_token",
                 hysteresis_order: str = "reference"):
        super().__init__()
        if use_24_sparsity or use_hadamard_int4:
            raise NotImplementedError("2:4 sparsity and Hadamard-INT4 activations are outside the INT2 linear hot path")
        if quant_mode not in ("per_token", "per_tensor"):
            raise ValueError("quant_mode must be 'per_token' or 'per_tensor'")
        if hysteresis_order not in ("reference", "after_dx"):
            raise ValueError("hysteresis_order must be 'reference' or 'after_dx'")
        self.in_features = in_features
        self.out_features = out_features
        self.threshold = threshold
        self.lr_scale = lr_scale
        self.decay_rate = decay_rate
        self.compress_activations = compress_activations
        self.use_24_sparsity = False
        self.use_hadamard_int4 = False
        self.quant_mode = quant_mode
        # "reference": the update fires in the output's gradient hook, i.e. before dX, which therefore sees the
        # updated weights (core/bitnet/int2_linear_tc_offload.py:338-367).  "after_dx": forward, dX, then update.
        self.hysteresis_order = hysteresis_order

        self.register_buffer("W_packed", torch.zeros(out_features, (in_features + 3) // 4, dtype=torch.uint8))
        self.register_buffer("H_packed", torch.zeros(out_features, (in_features + 1) // 2, dtype=torch.uint8))
        self.gamma = nn.Parameter(torch.ones(1))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features))
        else:
            self.register_parameter("bias", None)
        self.register_buffer("_step", torch.tensor(0, dtype=torch.int64))
        self._step_py = 0
        self._saved_input = None
        self._saved_input_shape = None
        self._initialized = False
        self._gamma_cached: Optional[float] = None
        self._dy_cache = None
        self._pending_update = None
        # row offset of this layer's rows inside a larger (sharded) weight matrix: keeps the per-weight random
        # numbers of a shard equal to those of the unsharded layer
        self.row_offset = 0

    # ---- initialisation ------------------------------------------------------------------------------------
    def init_from_float(self, weight: torch.Tensor, scale: Optional[float] = None):
        """gamma = max(mean|W|, 1e-5); W_packed = pack(clamp(round(W/gamma), -1, 1)); counters zeroed
        (core/bitnet/int2_linear_tc.py:391-412)."""
        assert weight.shape == (self.out_features, self.in_features)
        if scale is None:
            scale = max(weight.abs().mean().item(), 1e-5)
        dev = self.W_packed.device if self.W_packed.is_cuda else torch.device("cuda")
        packed = int2_tc_ops.ternarize_pack(weight.to(dev), scale)
        self.W_packed.copy_(packed)
        self.gamma.data.fill_(scale)
        self._gamma_cached = scale
        self.H_packed.zero_()
        self._initialized = True

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        if prefix + "W_packed" in state_dict:
            self._initialized = True
            self._gamma_cached = None
            self._step_py = int(self._step.item())

    def sync_step_buffer(self):
        """Writes the Python step counter into the `_step` buffer before a checkpoint (train.py:797-798)."""
        self._step.fill_(self._step_py)

    # ---- forward ---------------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, pre_norm: Optional[nn.Module] = None, up: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`pre_norm`: an RMSNorm module (`weight` float32 [K], `eps`) to apply to x first, fused with the quantiser.
        `up`: x is a gate and the layer's input is `silu(x) * up` (the reference's SwiGLU block), fused as well."""
        if not self._initialized:
            w_init = torch.randn(self.out_features, self.in_features, device=x.device, dtype=torch.float32) * (
                1.0 / math.sqrt(self.in_features))
            self.init_from_float(w_init)
        if self._gamma_cached is None:
            self._gamma_cached = self.gamma.detach().item()
        out = self._decode_forward(x, pre_norm, up)
        if out is None:
            args = (x, self.W_packed, self.gamma, self.in_features, self._gamma_cached, self)
            if up is not None:
                out = Int2LinearTCFunction.apply(*args, None if pre_norm is None else pre_norm.weight,
                                                 1e-6 if pre_norm is None else pre_norm.eps, up)
            elif pre_norm is not None:
                out = Int2LinearTCFunction.apply(*args, pre_norm.weight, pre_norm.eps)
            else:
                out = Int2LinearTCFunction.apply(*args)
        if self.bias is not None:
            out = out + self.bias.to(out.dtype)
        return out

    def _decode_forward(self, x: torch.Tensor, pre_norm: Optional[nn.Module], up: Optional[torch.Tensor]):
        """Inference with a few tokens (no gradient recorded, 1..64 tokens, per-token mode): the layer input is formed by
        one small kernel when a norm or a gate comes first, and the weight-streaming decode call does the rest - the
        path of the reference's `generate` (model/model.py:505-623), where its own kernels fall back to a scalar loop
        (kernels/int2/int2_matmul_int8_tc_v2.cu:452-473).  Same output as the training-time forward, bit for bit.
        Returns None when the call does not qualify."""
        K = self.in_features
        if (torch.is_grad_enabled() or self.quant_mode != "per_token" or not x.is_cuda or x.dtype not in _FLOAT_IO or K % 64 != 0
                or x.shape[-1] != K):
            return None
        M = x.numel() // K
        if not 1 <= M <= 64:
            return None
        if pre_norm is not None and (pre_norm.weight.dtype != torch.float32 or not pre_norm.weight.is_contiguous()):
            return None
        if up is not None and (up.dtype != x.dtype or up.shape != x.shape):
            return None
        y = x
        if pre_norm is not None or up is not None:
            y = int2_tc_ops.prelinear_rows(x, up, None if pre_norm is None else pre_norm.weight,
                                           1e-6 if pre_norm is None else pre_norm.eps)
        return int2_tc_ops.linear_decode(y, self.W_packed, self._gamma_cached, x.dtype)

    # ---- weight update -----------------------------------------------------------------------------------------
    def _take_dy_cache(self, dY: torch.Tensor):
        c, self._dy_cache = self._dy_cache, None
        if c is not None and c[0] == dY.data_ptr() and c[1] == tuple(dY.shape):
            return c[2], c[3]
        return None

    def _run_pending_update(self):
        p, self._pending_update = self._pending_update, None
        if p is not None:
            self.hysteresis_update(*p)

    def hysteresis_update(self, dY: torch.Tensor, lr: float):
        """dW = dY^T . X-hat as an exact int8 GEMM, then the hysteresis update of W_packed / H_packed
        (core/bitnet/int2_linear_tc.py:483-548).  The layer's own counter, pre-incremented, is the random step."""
        if self._saved_input is None:
            raise RuntimeError("No saved input. Call forward() first in training mode.")
        self._step_py += 1
        Xq, ax = self._saved_input
        N, K = self.out_features, self.in_features
        dY2 = dY.reshape(-1, N)
        if dY2.dtype not in _FLOAT_IO:
            dY2 = dY2.float()
        if self.quant_mode == "per_tensor":
            dY2 = dY2.half() if dY2.dtype != torch.float16 else dY2
        dY2 = dY2.contiguous()
        M = dY2.shape[0]
        ax_rows = ax if ax.numel() == M else ax.expand(M).contiguous()
        dYq, ady, gmax = int2_tc_ops.quantize_rows(dY2, GRAD_EPS, fold_absmax=ax_rows)
        if self.quant_mode == "per_token":
            self._dy_cache = (dY.data_ptr(), tuple(dY.shape), dYq.view(*dY.shape[:-1], N), ady)
        Gq = int2_tc_ops.quantize_grad(dY2, ax_rows, gmax)
        Xq2 = Xq.reshape(-1, K)
        idx_base = self.row_offset * K
        if int2_tc_ops.dw_hysteresis_supported(N, K):
            int2_tc_ops.dw_hysteresis(Gq, Xq2, gmax, self.W_packed, self.H_packed, lr, self.lr_scale, self.threshold,
                                      self.decay_rate, self._step_py, idx_base)
        else:
            dW = int2_tc_ops.weight_grad(Gq, Xq2, gmax)
            int2_tc_ops.hysteresis_step_v2(dW, self.W_packed, self.H_packed, lr, self.lr_scale, self.threshold,
                                           self.decay_rate, self._step_py, idx_base)
        self._saved_input = None
        self._saved_input_shape = None

    def memory_footprint(self) -> Dict[str, Any]:
        total_weights = self.out_features * self.in_features
        w_bytes, h_bytes = self.W_packed.numel(), self.H_packed.numel()
        bias_bytes = self.bias.numel() * 4 if self.bias is not None else 0
        return {
            "total_weights": total_weights,
            "total_bytes": w_bytes + h_bytes + 4 + bias_bytes,
            "w_bytes": w_bytes,
            "h_bytes": h_bytes,
            "bytes_per_weight": (w_bytes + h_bytes) / total_weights,
            "compression_vs_fp32": total_weights * 4 / (w_bytes + h_bytes),
            "fp32_equivalent_bytes": total_weights * 4,
            "compress_activations": self.compress_activations,
            "activation_compression_ratio": 0.5 if self.compress_activations else 1.0,
        }

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"threshold={self.threshold}, quant={self.quant_mode}, TC=True")


class Int2LinearTCWithGradHook(Int2LinearTC):
    """Int2LinearTC whose weight update fires from a gradient hook on the layer output, gated by a class-level
    switch for gradient accumulation (core/bitnet/int2_linear_tc.py:652-676 and
    core/bitnet/int2_linear_tc_offload.py:289-371)."""

    _hysteresis_enabled: bool = True

    def __init__(self, *args, enable_offload: bool = False, **kwargs):
        super().__init__(*args, **kwargs)
        # CPU offload of saved activations is a PCIe side-car that the reference ships disabled; accepted, unused.
        self.enable_offload = False
        self._lr = 0.001

    def set_lr(self, lr: float):
        self._lr = lr

    @classmethod
    def enable_hysteresis(cls):
        Int2LinearTCWithGradHook._hysteresis_enabled = True

    @classmethod
    def disable_hysteresis(cls):
        Int2LinearTCWithGradHook._hysteresis_enabled = False

    def forward(self, x: torch.Tensor, pre_norm: Optional[nn.Module] = None, up: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = super().forward(x, pre_norm, up)
        if self.training and out.requires_grad:
            out.register_hook(self._grad_hook)
        return out

    def _grad_hook(self, grad: torch.Tensor):
        if not Int2LinearTCWithGradHook._hysteresis_enabled:
            # accumulation micro-batch: drop the saved activation, leave the weights alone
            self._saved_input = None
            self._saved_input_shape = None
            return
        if self._saved_input is None:
            return
        if self.hysteresis_order == "after_dx":
            self._pending_update = (grad, self._lr)     # runs at the end of Int2LinearTCFunction.backward
        else:
            self.hysteresis_update(grad, self._lr)


# Names under which the reference instantiates the layer (core/bitnet/int2_linear_tc_offload.py:31,289).
Int2LinearTCOffload = Int2LinearTC
Int2LinearTCOffloadWithGradHook = Int2LinearTCWithGradHook
