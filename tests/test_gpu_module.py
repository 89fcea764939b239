"""The layer-level API (Int2LinearTC / BitLinearInt2 / converters) against the oracle's composite step."""
import io

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import int2_oracle as O
from oracle import native

from helpers import make_layer_inputs, t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _make_layer(pkg, d, K, N, thr=2, order="reference", mode="per_token", hook=True):
    cls = pkg.Int2LinearTCWithGradHook if hook else pkg.Int2LinearTC
    layer = cls(K, N, threshold=thr, lr_scale=5.0, decay_rate=0.001, quant_mode=mode, hysteresis_order=order).to(DEV)
    layer.init_from_float(d["W"].to(DEV), scale=d["gamma"])
    layer.H_packed.copy_(torch.from_numpy(d["Hp"]))
    layer.train()
    return layer


@pytest.mark.parametrize("order", ["reference", "after_dx"])
@pytest.mark.parametrize("M,K,N,dtype", [(1024, 1536, 1536, torch.bfloat16), (96, 128, 80, torch.float32),
                                         (64, 100, 36, torch.bfloat16),
                                         # the awkward projections of the reference model: K=16 (dt_proj), N=48 (x_proj),
                                         # N=16 (diff_gate), K=256 (w_kv_up), and the 4096->512 MLA latent projection
                                         (64, 16, 64, torch.bfloat16), (64, 128, 48, torch.bfloat16),
                                         (64, 64, 16, torch.bfloat16), (128, 256, 1024, torch.bfloat16),
                                         (256, 4096, 512, torch.bfloat16)])
def test_layer_step_matches_oracle(pkg, order, M, K, N, dtype):
    """Forward, dX and the weight update of one layer step (benchmark configuration 0 is the first case)."""
    d = make_layer_inputs(M, K, N, seed=0, dtype=dtype, dy_std=1e-2)
    lr = 1e-2 if M >= 1024 else 0.5      # large enough for the small cases to flip weights too
    layer = _make_layer(pkg, d, K, N, thr=2, order=order)
    layer.set_lr(lr)
    assert np.array_equal(layer.W_packed.cpu().numpy(), d["Wp"])
    x = d["x"].to(DEV).requires_grad_(True)
    y = layer(x)
    y.backward(d["dY"].to(DEV))
    torch.cuda.synchronize()
    pkg.int2_tc_ops.check_device_status(torch.device(DEV))

    out = {torch.bfloat16: "bf16", torch.float32: "f32"}[dtype]
    yo, Xq, ax = O.bitlinear_forward(t2n(d["x"]), d["Wp"], d["gamma"], K, out=out)
    assert np.array_equal(t2n(y), yo)
    dWo, acc, g = O.bitlinear_dw(t2n(d["dY"]), Xq, ax)
    Wn, Hn = native.c_hysteresis_step(dWo, d["Wp"], d["Hp"], lr, 5.0, 2, 0.001, 1, K)
    assert np.array_equal(layer.W_packed.cpu().numpy(), Wn)
    assert np.array_equal(layer.H_packed.cpu().numpy(), Hn)
    # the case does move the state (the tiniest shapes may only move counters)
    assert (O.unpack_ternary(Wn, K) != O.unpack_ternary(d["Wp"], K)).any() or not np.array_equal(Hn, d["Hp"])
    w_for_dx = Wn if order == "reference" else d["Wp"]      # the reference's hook updates the weights before dX
    dxo = O.bitlinear_backward_dx(t2n(d["dY"]), w_for_dx, d["gamma"], K, out=out)
    assert np.array_equal(t2n(x.grad), dxo)
    assert layer._step_py == 1 and layer._saved_input is None


def test_per_tensor_mode_follows_the_reference_cuda_rule(pkg):
    M, K, N = 128, 256, 192
    d = make_layer_inputs(M, K, N, seed=4, dtype=torch.float16)
    layer = _make_layer(pkg, d, K, N, mode="per_tensor", hook=False)
    x = d["x"].to(DEV).requires_grad_(True)
    y = layer(x)
    assert y.dtype == torch.float16
    xq, a = O.quantize_tensor(t2n(d["x"]))
    yo = O.to_f16(O.scale_rows(O.gemm_fwd_acc(xq, d["Wp"], K), a, d["gamma"]))
    assert np.array_equal(t2n(y), yo)
    y.backward(d["dY"].to(DEV))
    dyq, ay = O.quantize_tensor(t2n(d["dY"]))
    dxo = O.to_f16(O.scale_rows(O.gemm_dx_acc(dyq, d["Wp"], K), ay, d["gamma"]))
    assert np.array_equal(t2n(x.grad), dxo)
    layer.hysteresis_update(d["dY"].to(DEV), 1e-2)
    assert layer._step_py == 1


def test_accumulation_gate_and_missing_input(pkg):
    d = make_layer_inputs(32, 64, 48, seed=2)
    layer = _make_layer(pkg, d, 64, 48)
    with pytest.raises(RuntimeError):
        layer.hysteresis_update(d["dY"].to(DEV), 1e-2)            # no forward yet
    pkg.disable_hysteresis()
    try:
        y = layer(d["x"].to(DEV).requires_grad_(True))
        y.backward(d["dY"].to(DEV))
        assert np.array_equal(layer.W_packed.cpu().numpy(), d["Wp"]) and layer._step_py == 0
        assert layer._saved_input is None
    finally:
        pkg.enable_hysteresis()
    y = layer(d["x"].to(DEV).requires_grad_(True))
    y.backward(d["dY"].to(DEV))
    assert layer._step_py == 1
    layer.eval()
    with torch.no_grad():
        layer(d["x"].to(DEV))
    assert layer._saved_input is None                              # inference keeps no activation


def test_checkpoint_roundtrip_keeps_reference_state_names(pkg):
    d = make_layer_inputs(16, 64, 32, seed=5)
    layer = _make_layer(pkg, d, 64, 32)
    layer._step_py = 7
    layer.sync_step_buffer()
    sd = layer.state_dict()
    assert set(sd) == {"gamma", "W_packed", "H_packed", "_step"}
    buf = io.BytesIO()
    torch.save(sd, buf)
    buf.seek(0)
    other = pkg.Int2LinearTCWithGradHook(64, 32).to(DEV)
    other.load_state_dict(torch.load(buf))
    assert other._step_py == 7 and other._initialized
    assert torch.equal(other.W_packed, layer.W_packed)
    with torch.no_grad():
        assert torch.equal(other.eval()(d["x"].to(DEV)), layer.eval()(d["x"].to(DEV)))


def test_convert_all_linear_to_int2(pkg):
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.w1 = nn.Linear(256, 512, bias=False)
            self.w2 = nn.Linear(512, 256, bias=True)
            self.tiny = nn.Linear(16, 8)                # below the size floor
            self.lm_head = nn.Linear(256, 300)          # excluded by name
            self.norm = nn.LayerNorm(256)

        def forward(self, x):
            return self.lm_head(self.norm(self.w2(torch.nn.functional.silu(self.w1(x)))))

    torch.manual_seed(0)
    model = Block()
    conv = pkg.convert_all_linear_to_int2(model, threshold=3, min_size=64, verbose=False)
    layers = pkg.get_int2_layers(conv)
    assert len(layers) == 2 and isinstance(conv.w1, pkg.BitLinearInt2) and isinstance(conv.tiny, nn.Linear)
    assert isinstance(conv.lm_head, nn.Linear) and isinstance(model.w1, nn.Linear)      # not in place
    assert not conv._int2_conversion_stats["errors"]
    gamma = float(max(model.w1.weight.abs().mean().item(), 1e-5))
    assert np.array_equal(conv.w1.weight_packed.cpu().numpy(),
                          O.pack_ternary(O.ternarize(model.w1.weight.detach().numpy(), gamma), pad_code=0))
    pkg.set_all_int2_lr(conv, 0.02)
    assert conv.w1.int2_layer._lr == 0.02
    n_other = len(pkg.get_non_int2_params(conv))
    assert n_other == len(list(conv.parameters())) - sum(len(list(l.parameters())) for l in layers)
    conv = conv.to(DEV).train()
    x = torch.randn(4, 10, 256, device=DEV, dtype=torch.bfloat16)
    conv.lm_head.to(torch.bfloat16); conv.norm.to(torch.bfloat16)
    out = conv(x)
    out.float().pow(2).mean().backward()
    assert out.shape == (4, 10, 300) and torch.isfinite(out.float()).all()
    assert conv.w1.int2_layer._step_py == 1 and conv.w2.int2_layer._step_py == 1


@pytest.mark.parametrize("M,K,N,dtype", [(256, 1536, 512, torch.bfloat16), (64, 256, 96, torch.float32)])
def test_bitlinear_fused_rmsnorm_matches_oracle_and_unfused_module(pkg, M, K, N, dtype):
    """BitLinearInt2 with the pre-linear RMSNorm fused into the quantiser: the step equals the oracle's composite
    (norm -> quantise -> GEMM; dX GEMM -> norm backward) bit for bit, and agrees with the same module running the norm
    as separate tensor operations within rel-err 1e-2 (torch sums the squares in another order; a one-ulp difference in
    rstd can move an activation across an int8 rounding boundary, so the bound is that of the 8-bit grid for both
    I/O types)."""
    d = make_layer_inputs(M, K, N, seed=5, dtype=dtype, dy_std=1e-2)
    io = {torch.bfloat16: "bf16", torch.float32: "f32"}[dtype]
    gen = torch.Generator().manual_seed(9)
    nw = (1.0 + 0.2 * torch.randn(K, generator=gen)).float()

    def run(fused):
        m = pkg.BitLinearInt2(K, N, threshold=2, use_grad_hook=True, hysteresis_order="after_dx").to(DEV)
        m.fuse_rmsnorm = fused
        m.int2_layer.init_from_float(d["W"].to(DEV), scale=d["gamma"])
        m.int2_layer.H_packed.copy_(torch.from_numpy(d["Hp"]))
        with torch.no_grad():
            m.extra_rmsnorm.weight.copy_(nw)
        m.train()
        m.set_lr(0.5)
        x = (d["x"] * 3.0).to(dtype).to(DEV).requires_grad_(True)
        y = m(x)
        y.backward(d["dY"].to(DEV))
        torch.cuda.synchronize()
        return m, x, y

    mf, xf, yf = run(True)
    mu, xu, yu = run(False)
    pkg.int2_tc_ops.check_device_status(torch.device(DEV))

    x_np = t2n((d["x"] * 3.0).to(dtype))
    Xq, ax, rstd = O.rmsnorm_quantize_rows(x_np, nw.numpy(), 1e-6, 1e-5, io)
    yo = O.scale_rows(O.gemm_fwd_acc(Xq, d["Wp"], K), ax, d["gamma"])
    yo = O.to_bf16(yo) if io == "bf16" else yo
    assert np.array_equal(t2n(yf), yo)
    dxn = O.bitlinear_backward_dx(t2n(d["dY"]), d["Wp"], d["gamma"], K, out=io)     # after_dx: the old weights
    dxo, dwo = O.rmsnorm_backward(dxn, x_np, nw.numpy(), rstd, io)
    assert np.array_equal(t2n(xf.grad), dxo)
    assert np.array_equal(mf.extra_rmsnorm.weight.grad.cpu().numpy(), dwo)
    dWo, _, _ = O.bitlinear_dw(t2n(d["dY"]), Xq, ax)
    Wn, Hn = native.c_hysteresis_step(dWo, d["Wp"], d["Hp"], 0.5, 5.0, 2, 0.001, 1, K)
    assert np.array_equal(mf.int2_layer.W_packed.cpu().numpy(), Wn) and np.array_equal(mf.int2_layer.H_packed.cpu().numpy(), Hn)

    tol = 1e-2

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max())

    assert rel(yf, yu) <= tol
    assert rel(xf.grad, xu.grad) <= tol
    assert rel(mf.extra_rmsnorm.weight.grad, mu.extra_rmsnorm.weight.grad) <= tol


def test_from_bitnetlinear_takes_weights_scale_and_bias_of_the_source_module(pkg):
    """The converter of BitNetLinear-style modules (core/bitnet/bitnet_int2_optimized.py:245-310): latent `master_weight`
    ternarised with the mean of the module's `scale` tensor when it has one, with the weight's absmean otherwise; a module
    without latent weights is re-initialised with scale 1/sqrt(K); the bias is carried over."""
    K, N = 128, 48
    g = torch.Generator().manual_seed(8)

    class Src(nn.Module):
        def __init__(self, with_weight, with_scale, with_bias):
            super().__init__()
            self.in_features, self.out_features = K, N
            self.master_weight = nn.Parameter(torch.randn(N, K, generator=g) * 0.05) if with_weight else None
            self.scale = nn.Parameter(torch.full((N,), 0.031)) if with_scale else None
            self.bias = nn.Parameter(torch.randn(N, generator=g)) if with_bias else None

    for with_weight, with_scale, with_bias in [(True, True, True), (True, False, False), (False, False, True)]:
        src = Src(with_weight, with_scale, with_bias)
        layer = pkg.BitLinearInt2.from_bitnetlinear(src, threshold=3)
        il = layer.int2_layer
        assert il.W_packed.is_cuda and il.threshold == 3 and (il.bias is not None) == with_bias
        if with_bias:
            assert torch.equal(il.bias.detach().cpu(), src.bias.detach())
        if with_weight:
            w = src.master_weight.detach().float().numpy()
            scale = 0.031 if with_scale else float(np.abs(w).mean())
            assert abs(il.gamma.item() - scale) < 1e-7
            want = O.pack_ternary(O.ternarize(w, np.float32(il.gamma.item())), pad_code=0)
            assert np.array_equal(il.W_packed.cpu().numpy(), want)
        else:
            assert abs(il.gamma.item() - K ** -0.5) < 1e-7
            codes = il.W_packed.cpu().numpy()
            assert len(np.unique(O.unpack_ternary(codes, K))) == 3
        assert int(il.H_packed.abs().sum().item()) == 0
