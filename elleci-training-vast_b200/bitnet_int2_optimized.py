"""The module API the model sees: BitLinearInt2 and the converters, as in
core/bitnet/bitnet_int2_optimized.py (:109-322 facade, :384-408 helpers, :411-689 conversion)."""
from __future__ import annotations

import copy
from typing import List, Optional

import torch
import torch.nn as nn

from . import int2_tc_ops
from .int2_linear_tc import Int2LinearTC, Int2LinearTCWithGradHook

USING_OPTIMIZED = True


class _ExtraRMSNorm(nn.Module):
    """RMSNorm in float32 applied before the linear layer (bitnet_int2_optimized.py:72-86)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x_f32 = x.float()
        norm = x_f32 * torch.rsqrt(x_f32.pow(2).mean(-1, keepdim=True) + self.eps)
        return norm.type_as(x) * self.weight.type_as(x)


class BitLinearInt2(nn.Module):
    """Facade over the INT2 layer with the reference's constructor and properties
    (bitnet_int2_optimized.py:120-322).  `io_dtype` None keeps the caller's dtype in per-token mode; the
    per-tensor mode casts to fp16 as the reference does (:207-208)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, threshold: int = 7,
                 lr_scale: float = 5.0, decay_rate: float = 0.001, use_grad_hook: bool = True, enable_offload: bool = True,
                 use_24_sparsity: bool = False, use_hadamard_int4: bool = False, use_extra_rmsnorm: bool = True,
                 rmsnorm_eps: float = 1e-6, use_hadamard_smooth: bool = False, quant_mode: str = "per_token",
                 hysteresis_order: str = "reference"):
        super().__init__()
        if use_hadamard_smooth:
            raise NotImplementedError("Hadamard smoothing is outside the INT2 linear hot path")
        self.in_features = in_features
        self.out_features = out_features
        self.use_extra_rmsnorm = use_extra_rmsnorm
        if use_extra_rmsnorm:
            self.extra_rmsnorm = _ExtraRMSNorm(in_features, eps=rmsnorm_eps)
        self.use_hadamard_smooth = False
        self.fuse_rmsnorm = True          # False: run the norm as separate tensor operations, as the reference does
        self.fuse_swiglu = True           # False: a gated input (forward's `up`) runs silu and the product as tensor operations
        cls = Int2LinearTCWithGradHook if use_grad_hook else Int2LinearTC
        self.int2_layer = cls(in_features=in_features, out_features=out_features, bias=bias, threshold=threshold,
                              lr_scale=lr_scale, decay_rate=decay_rate, use_24_sparsity=use_24_sparsity,
                              use_hadamard_int4=use_hadamard_int4, quant_mode=quant_mode,
                              hysteresis_order=hysteresis_order)
        self._use_grad_hook = use_grad_hook
        self._enable_offload = False

    @property
    def scale(self):
        return self.int2_layer.gamma.view(1, 1).expand(self.out_features, 1)

    @property
    def gamma(self):
        return self.int2_layer.gamma

    @property
    def weight_packed(self):
        return self.int2_layer.W_packed

    def forward(self, x: torch.Tensor, up: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`up`: x is the output of a gate projection and the layer's input is `silu(x) * up` (the reference's SwiGLU
        block, model/model.py:107-108); the product, the norm and the quantiser then run as one kernel."""
        fusable = (self.int2_layer.quant_mode == "per_token"
                   and (not self.use_extra_rmsnorm or self.extra_rmsnorm.weight.dtype == torch.float32))
        if up is not None:
            if self.fuse_swiglu and fusable and (self.fuse_rmsnorm or not self.use_extra_rmsnorm) and int2_tc_ops.swiglu_supported(x) \
                    and up.dtype == x.dtype and up.shape == x.shape:
                return self.int2_layer(x, pre_norm=self.extra_rmsnorm if self.use_extra_rmsnorm else None, up=up)
            x = torch.nn.functional.silu(x) * up
        if self.use_extra_rmsnorm:
            if self.fuse_rmsnorm and fusable and int2_tc_ops.rmsnorm_supported(x):
                # normalisation, quantisation (and their backward) as one kernel each instead of eight tensor passes
                return self.int2_layer(x, pre_norm=self.extra_rmsnorm)
            x = self.extra_rmsnorm(x)
        if self.int2_layer.quant_mode == "per_tensor" and x.dtype != torch.float16:
            x = x.half()
        return self.int2_layer(x)

    def set_lr(self, lr: float):
        if self._use_grad_hook and hasattr(self.int2_layer, "set_lr"):
            self.int2_layer.set_lr(lr)

    def hysteresis_update(self, dY: torch.Tensor, lr: float):
        self.int2_layer.hysteresis_update(dY, lr)

    def prefetch_activation(self):
        """No-op: saved activations stay on the device."""

    def reset_parameters(self):
        w_init = torch.empty(self.out_features, self.in_features, dtype=torch.float32)
        nn.init.kaiming_normal_(w_init, mode="fan_in", nonlinearity="linear")
        scale = max(w_init.abs().mean().item(), 1e-5)
        self.int2_layer.init_from_float(w_init.to(self.int2_layer.W_packed.device), scale=scale)

    @staticmethod
    def _source_weights(src: nn.Module, device: torch.device):
        """(latent float32 weight [N,K] on `device`, ternarisation scale) of the module being converted.  A module with a
        `master_weight` supplies it, and its `scale` tensor's mean when it has one (absmean of the weight otherwise); a
        module without latent weights is re-initialised (Kaiming-normal, scale 1/sqrt(K)), as the reference's converter
        does (core/bitnet/bitnet_int2_optimized.py:245-310).  The scale is floored at 1e-5."""
        N, K = src.out_features, src.in_features
        latent = getattr(src, "master_weight", None)
        if latent is None:
            weight = nn.init.kaiming_normal_(torch.empty(N, K, dtype=torch.float32, device=device), mode="fan_in",
                                             nonlinearity="linear")
            return weight, max(K ** -0.5, 1e-5)
        weight = latent.detach().to(device=device, dtype=torch.float32)
        stored = getattr(src, "scale", None)
        scale = float(stored.detach().float().mean()) if stored is not None else float(weight.abs().mean())
        return weight, max(scale, 1e-5)

    @classmethod
    def from_bitnetlinear(cls, bitlinear: nn.Module, use_24_sparsity: bool = False, **kwargs) -> "BitLinearInt2":
        """An INT2 layer on the GPU holding the ternarised weights (and the bias) of a BitNetLinear-style module."""
        device = torch.device("cuda")
        has_bias = bitlinear.bias is not None
        layer = cls(bitlinear.in_features, bitlinear.out_features, bias=has_bias, use_24_sparsity=use_24_sparsity, **kwargs).to(device)
        with torch.no_grad():
            layer.int2_layer.init_from_float(*cls._source_weights(bitlinear, device))
            if has_bias and layer.int2_layer.bias is not None:
                layer.int2_layer.bias.copy_(bitlinear.bias.detach().to(device))
        return layer

    def memory_footprint(self):
        return self.int2_layer.memory_footprint()

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, int2=tcgen05/{self.int2_layer.quant_mode}"


class SwiGLUFFNInt2(nn.Module):
    """The reference's feed-forward block over INT2 layers: `w3(silu(w1(x)) * w2(x))` with the hidden size rounded up
    to a multiple of 256 (SwiGLUFFN, model/model.py:86-108; same submodule names, so its state dict keys carry over).
    silu, the product, w3's pre-linear norm and w3's quantiser run as one kernel (and one in the backward pass);
    `fuse_swiglu = False` on w3 runs them as tensor operations instead."""

    def __init__(self, d_model: int, expansion_factor: float = 8 / 3, **layer_kwargs):
        super().__init__()
        hidden_dim = int(d_model * expansion_factor)
        hidden_dim = 256 * ((hidden_dim + 256 - 1) // 256)
        self.hidden_dim = hidden_dim
        self.w1 = BitLinearInt2(d_model, hidden_dim, **layer_kwargs)     # gate projection
        self.w2 = BitLinearInt2(d_model, hidden_dim, **layer_kwargs)     # up projection
        self.w3 = BitLinearInt2(hidden_dim, d_model, **layer_kwargs)     # down projection

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w3(self.w1(x), up=self.w2(x))


def get_int2_layers(module: nn.Module) -> List[BitLinearInt2]:
    return [m for m in module.modules() if isinstance(m, BitLinearInt2)]


def get_non_int2_params(module: nn.Module):
    int2_params = {id(p) for m in module.modules() if isinstance(m, BitLinearInt2) for p in m.parameters()}
    return [p for p in module.parameters() if id(p) not in int2_params]


def set_all_int2_lr(module: nn.Module, lr: float):
    for m in module.modules():
        if isinstance(m, BitLinearInt2):
            m.set_lr(lr)


def prefetch_all_activations(module: nn.Module):
    """No-op: saved activations stay on the device."""


def enable_hysteresis():
    Int2LinearTCWithGradHook.enable_hysteresis()


def disable_hysteresis():
    Int2LinearTCWithGradHook.disable_hysteresis()


_DEFAULT_EXCLUDE = ["lm_head", "embed_tokens", "token_emb", "wte", "wpe", "word_emb", "norm", "ln_", "layer_norm",
                    "rmsnorm", "bias"]


def _should_exclude_layer(name: str, module: nn.Module, min_size: int = 256, exclude_patterns: Optional[list] = None):
    """(exclude?, reason) with the reference's name patterns and size floor (bitnet_int2_optimized.py:445-476)."""
    patterns = _DEFAULT_EXCLUDE if exclude_patterns is None else exclude_patterns
    low = name.lower()
    for pat in patterns:
        if pat in low:
            return True, f"pattern '{pat}'"
    if not isinstance(module, nn.Linear):
        return True, "not nn.Linear"
    total = module.in_features * module.out_features
    if total < min_size * min_size:
        return True, f"too small ({total:,} < {min_size * min_size:,})"
    return False, ""


def convert_all_linear_to_int2(module: nn.Module, threshold: int = 7, lr_scale: float = 5.0, decay_rate: float = 0.001,
                               use_grad_hook: bool = True, enable_offload: bool = True, min_size: int = 256,
                               exclude_patterns: Optional[list] = None, inplace: bool = False, verbose: bool = True,
                               use_24_sparsity: bool = False, use_hadamard_int4: bool = False,
                               quant_mode: str = "per_token", hysteresis_order: str = "reference") -> nn.Module:
    """Replaces every eligible nn.Linear (and BitNetLinear) by BitLinearInt2 initialised from its weights
    (bitnet_int2_optimized.py:479-689).  Returns the converted module; `stats` are attached as
    `module._int2_conversion_stats`."""
    if not inplace:
        module = copy.deepcopy(module)
    device = torch.device("cuda")
    stats = {"converted": 0, "converted_params": 0, "excluded": {}, "errors": []}
    kw = dict(threshold=threshold, lr_scale=lr_scale, decay_rate=decay_rate, use_grad_hook=use_grad_hook,
              enable_offload=enable_offload, use_24_sparsity=use_24_sparsity, use_hadamard_int4=use_hadamard_int4,
              quant_mode=quant_mode, hysteresis_order=hysteresis_order)

    def convert_linear(linear: nn.Linear) -> BitLinearInt2:
        new_layer = BitLinearInt2(in_features=linear.in_features, out_features=linear.out_features,
                                  bias=linear.bias is not None, **kw).to(device)
        with torch.no_grad():
            weight = linear.weight.data.float().to(device)
            scale = max(weight.abs().mean().item(), 1e-5)
            new_layer.int2_layer.init_from_float(weight, scale=scale)
            if linear.bias is not None and new_layer.int2_layer.bias is not None:
                new_layer.int2_layer.bias.data.copy_(linear.bias.data.to(device))
        return new_layer

    def recurse(mod: nn.Module, prefix: str = ""):
        for name, child in list(mod.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if type(child).__name__ == "BitNetLinear":
                try:
                    setattr(mod, name, BitLinearInt2.from_bitnetlinear(child, **kw))
                    stats["converted"] += 1
                    stats["converted_params"] += child.in_features * child.out_features
                except Exception as e:  # noqa: BLE001 - the reference records and continues
                    stats["errors"].append(f"{full}: {e}")
            elif isinstance(child, nn.Linear):
                skip, reason = _should_exclude_layer(full, child, min_size, exclude_patterns)
                if skip:
                    ent = stats["excluded"].setdefault(reason, {"count": 0, "params": 0, "names": []})
                    ent["count"] += 1
                    ent["params"] += child.in_features * child.out_features
                    ent["names"].append(full)
                else:
                    try:
                        setattr(mod, name, convert_linear(child))
                        stats["converted"] += 1
                        stats["converted_params"] += child.in_features * child.out_features
                    except Exception as e:  # noqa: BLE001
                        stats["errors"].append(f"{full}: {e}")
            else:
                recurse(child, full)

    recurse(module)
    module._int2_conversion_stats = stats
    if verbose:
        excluded = sum(v["params"] for v in stats["excluded"].values())
        total = stats["converted_params"] + excluded
        pct = 100.0 * stats["converted_params"] / total if total else 0.0
        print(f"[INT2] converted {stats['converted']} layers, {stats['converted_params'] / 1e6:.1f}M params ({pct:.1f}%); "
              f"{len(stats['errors'])} errors")
    return module
