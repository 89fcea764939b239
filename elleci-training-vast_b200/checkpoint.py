"""Checkpoint compatibility for the INT2 layers.

The reference's trainer saves, next to the model's state dict, one entry per INT2 layer with the packed weights, the
packed hysteresis counters, gamma and the layer's step counter, in the layers' own buffer layout
(`save_checkpoint` / `load_checkpoint`, train.py:784-849).  The functions here write and read that structure for the
modules of this package, so a checkpoint moves between the two implementations unchanged, and convert the 2-bit code
of the reference's Triton inference layer (model/common/triton_kernels.py:33-34) into the code the INT2 layers use.
"""
from __future__ import annotations

from typing import Dict, Iterable, List

import torch
import torch.nn as nn


def _inner(layer: nn.Module) -> nn.Module:
    return layer.int2_layer if hasattr(layer, "int2_layer") else layer


def collect_int2_state(int2_layers: Iterable[nn.Module]) -> Dict[str, dict]:
    """`int2_state` of the reference's checkpoint (train.py:788-806): {"layer_<i>": {"W_packed", "H_packed", "gamma",
    "step"}} with CPU tensors, layers numbered in the order given (the trainer uses `get_int2_layers(model)`).  The
    Python-side step counter is written into the `_step` buffer first, as the reference does."""
    state = {}
    for i, layer in enumerate(int2_layers):
        int2 = _inner(layer)
        if hasattr(int2, "_step_py"):
            int2._step.fill_(int2._step_py)
        state[f"layer_{i}"] = {
            "W_packed": int2.W_packed.detach().cpu().clone(),
            "H_packed": int2.H_packed.detach().cpu().clone(),
            "gamma": int2.gamma.data.detach().cpu().clone(),
            "step": int2._step.detach().cpu().clone(),
        }
    return state


def load_int2_state(int2_layers: Iterable[nn.Module], int2_state: Dict[str, dict], strict: bool = True) -> List[str]:
    """Restores the layers from an `int2_state` dictionary.  Shapes must match; a missing entry raises when `strict`,
    otherwise its name is returned in the list of skipped layers.  Cached gamma and the Python step counter are
    re-synchronised, as the reference's `load_checkpoint` does (train.py:840-846)."""
    skipped = []
    for i, layer in enumerate(int2_layers):
        key = f"layer_{i}"
        int2 = _inner(layer)
        entry = int2_state.get(key)
        if entry is None:
            if strict:
                raise KeyError(f"int2_state has no entry '{key}'")
            skipped.append(key)
            continue
        for name in ("W_packed", "H_packed"):
            src, dst = entry[name], getattr(int2, name)
            if tuple(src.shape) != tuple(dst.shape) or src.dtype != torch.uint8:
                raise ValueError(f"{key}.{name}: expected uint8 {tuple(dst.shape)}, got {src.dtype} {tuple(src.shape)}")
            dst.copy_(src.to(dst.device))
        with torch.no_grad():
            int2.gamma.data.copy_(entry["gamma"].to(int2.gamma.device).reshape(int2.gamma.shape))
        step = entry["step"]
        int2._step.fill_(int(step.item() if hasattr(step, "item") else step))
        sync_after_load([layer])
    return skipped


def sync_after_load(int2_layers: Iterable[nn.Module]) -> None:
    """What the reference does after `model.load_state_dict` (train.py:840-846): the Python step counter follows the
    `_step` buffer and the cached gamma follows the parameter."""
    for layer in int2_layers:
        int2 = _inner(layer)
        if hasattr(int2, "_step_py"):
            int2._step_py = int(int2._step.item())
        if hasattr(int2, "_gamma_cached"):
            int2._gamma_cached = float(int2.gamma.detach().item())
        int2._initialized = True


# 2-bit code of the Triton inference layer: 00 -> 0, 01 -> +1, 10 -> -1, 11 -> 0 (model/common/triton_kernels.py:33-34,
# decode `(v & 1) - (v >> 1)`); code of the INT2 layers: 00 -> -1, 01 -> 0, 10 -> +1, 11 -> 0
# (kernels/int2/int2_packed.cuh:9-18).  Field positions agree (weight 4b+j at bits 2j..2j+1 of byte b).
_FIELD_MAP = (1, 2, 0, 1)


def _byte_table() -> torch.Tensor:
    table = torch.empty(256, dtype=torch.uint8)
    for b in range(256):
        out = 0
        for j in range(4):
            out |= _FIELD_MAP[(b >> (2 * j)) & 3] << (2 * j)
        table[b] = out
    return table


def convert_triton_packed(packed_weight: torch.Tensor) -> torch.Tensor:
    """Packed weights of the reference's Triton layer (int8 or uint8 [N, K/4]) re-coded for `W_packed` (uint8, same
    shape): the same ternary values, the INT2 layers' code."""
    if packed_weight.dtype not in (torch.int8, torch.uint8):
        raise ValueError("packed_weight must be int8 or uint8")
    idx = packed_weight.contiguous().view(torch.uint8).long()
    return _byte_table().to(packed_weight.device)[idx]
