"""Checkpoint layout of the INT2 layers against the reference trainer's (train.py:784-849), on CPU tensors."""
import io

import numpy as np
import torch

from oracle import int2_oracle as O


def _filled_layers(pkg, seed):
    g = torch.Generator().manual_seed(seed)
    layers = [pkg.BitLinearInt2(64, 48, threshold=3), pkg.BitLinearInt2(40, 16, use_extra_rmsnorm=False, use_grad_hook=False)]
    for i, l in enumerate(layers):
        il = l.int2_layer
        il.W_packed.copy_(torch.randint(0, 256, il.W_packed.shape, generator=g, dtype=torch.uint8))
        il.H_packed.copy_(torch.randint(0, 256, il.H_packed.shape, generator=g, dtype=torch.uint8))
        il.gamma.data.fill_(0.01 * (i + 1))
        il._step_py = 7 + i
    return layers


def test_state_dict_names_and_shapes_follow_the_reference(pkg):
    """Buffers and parameters carry the reference's names and shapes (core/bitnet/int2_linear_tc.py:362-381 under
    `int2_layer.` of the facade, bitnet_int2_optimized.py:164-176), so `model.load_state_dict` accepts a reference
    checkpoint."""
    l = pkg.BitLinearInt2(64, 48, bias=True)
    sd = l.state_dict()
    assert set(sd) == {"extra_rmsnorm.weight", "int2_layer.W_packed", "int2_layer.H_packed", "int2_layer.gamma",
                       "int2_layer.bias", "int2_layer._step"}
    assert sd["int2_layer.W_packed"].shape == (48, 16) and sd["int2_layer.W_packed"].dtype == torch.uint8
    assert sd["int2_layer.H_packed"].shape == (48, 32) and sd["int2_layer.H_packed"].dtype == torch.uint8
    assert sd["int2_layer.gamma"].shape == (1,) and sd["int2_layer._step"].dtype == torch.int64
    ffn = pkg.SwiGLUFFNInt2(64)
    assert ffn.hidden_dim == 256 and {k.split(".")[0] for k in ffn.state_dict()} == {"w1", "w2", "w3"}


def test_int2_state_round_trip_through_torch_save(pkg):
    ck = pkg.checkpoint
    src = _filled_layers(pkg, 1)
    state = ck.collect_int2_state(src)
    assert list(state) == ["layer_0", "layer_1"] and set(state["layer_0"]) == {"W_packed", "H_packed", "gamma", "step"}
    assert int(state["layer_1"]["step"]) == 8 and int(src[1].int2_layer._step) == 8      # buffer synchronised first
    buf = io.BytesIO()
    torch.save({"int2_state": state, "model_state_dict": {f"{i}.{k}": v for i, l in enumerate(src) for k, v in l.state_dict().items()}}, buf)
    buf.seek(0)
    loaded = torch.load(buf)
    dst = _filled_layers(pkg, 2)
    assert ck.load_int2_state(dst, loaded["int2_state"]) == []
    for a, b in zip(src, dst):
        assert torch.equal(a.int2_layer.W_packed, b.int2_layer.W_packed)
        assert torch.equal(a.int2_layer.H_packed, b.int2_layer.H_packed)
        assert b.int2_layer._step_py == a.int2_layer._step_py
        assert b.int2_layer._gamma_cached == float(a.int2_layer.gamma.item())
    # the model state dict route: load_state_dict, then the reference's re-synchronisation
    dst2 = _filled_layers(pkg, 3)
    for i, l in enumerate(dst2):
        l.load_state_dict({k[len(f"{i}."):]: v for k, v in loaded["model_state_dict"].items() if k.startswith(f"{i}.")})
    ck.sync_after_load(dst2)
    assert dst2[0].int2_layer._step_py == 7 and torch.equal(dst2[1].int2_layer.H_packed, src[1].int2_layer.H_packed)


def test_int2_state_rejects_wrong_shapes_and_missing_layers(pkg):
    import pytest
    ck = pkg.checkpoint
    src = _filled_layers(pkg, 1)
    state = ck.collect_int2_state(src)
    with pytest.raises(KeyError):
        ck.load_int2_state(src + [pkg.BitLinearInt2(8, 8)], state)
    assert ck.load_int2_state(src + [pkg.BitLinearInt2(8, 8)], state, strict=False) == ["layer_2"]
    state["layer_0"]["W_packed"] = state["layer_0"]["W_packed"][:, :-1]
    with pytest.raises(ValueError):
        ck.load_int2_state(src, state)


def test_triton_code_conversion_keeps_the_ternary_values(pkg):
    """Every byte value: decoding the Triton layer's code `(v & 1) - (v >> 1)` (model/common/triton_kernels.py:33-34,
    52-56) gives the same four weights as decoding the converted byte with the INT2 code."""
    b = torch.arange(256, dtype=torch.uint8).view(16, 16)
    conv = pkg.checkpoint.convert_triton_packed(b.view(torch.int8))
    v = np.stack([(b.numpy() >> (2 * j)) & 3 for j in range(4)], axis=-1).astype(np.int32)
    triton_w = ((v & 1) - (v >> 1)).reshape(16, 64)
    assert np.array_equal(O.unpack_ternary(conv.numpy(), 64), triton_w)
