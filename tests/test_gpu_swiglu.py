"""The fused SwiGLU gate kernels (silu(gate) * up -> pre-linear norm -> per-token quantiser, and the backward pass)
against the CPU oracle bit for bit, against the reference expression's golden outputs within floating-point tolerance,
and inside the feed-forward module."""
import os

import numpy as np
import pytest
import torch

from oracle import int2_oracle as O
from oracle import native

from conftest import GOLDEN
from helpers import t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"
_IO = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}


@pytest.fixture(scope="module")
def ops(pkg):
    assert os.path.exists(pkg.LIB_PATH), "the CUDA library must be built in-tree"
    return pkg.int2_tc_ops


def _gate_up(M, H, dtype, seed, scale=2.0):
    g = torch.Generator().manual_seed(seed)
    gu = (torch.randn(M, 2 * H, generator=g) * scale).to(dtype)
    w = (1.0 + 0.3 * torch.randn(H, generator=g)).float()
    gy = (torch.randn(M, H, generator=g) * 1e-2).to(dtype)
    return gu, w, gy


@pytest.mark.parametrize("M,H", [(1, 8), (7, 64), (33, 1536), (16, 4096), (5, 11008), (3, 12544)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("norm", [True, False])
def test_swiglu_quantize_rows_bit_exact(ops, M, H, dtype, norm):
    """int8 tokens, absmax and rstd equal the oracle's bit for bit, with gate and up read in place as the two halves of
    one [M, 2H] matrix.  Covers saturated gates, an all-zero token, NaN and infinity, and rows longer than the
    register cache (12544)."""
    gu, w, _ = _gate_up(M, H, dtype, M * 17 + H)
    if M > 2:
        gu[1] = 0.0
        gu[2, :H] = torch.linspace(-120.0, 120.0, H).to(dtype)       # the whole range of the exponential
    if M > 4:
        gu[3, 0] = float("nan")
        gu[4, H + 1] = float("inf")
    d = gu.to(DEV)
    q, a, rstd = ops.swiglu_quantize_rows(d[:, :H], d[:, H:], w.to(DEV) if norm else None, 1e-6, 1e-5)
    with np.errstate(all="ignore"):
        qo, ao, ro = O.swiglu_quantize_rows(t2n(gu[:, :H]), t2n(gu[:, H:]), w.numpy() if norm else None, 1e-6, 1e-5, _IO[dtype])
    if norm:
        assert np.array_equal(rstd.cpu().numpy(), ro, equal_nan=True)
    else:
        assert rstd is None
    assert np.array_equal(a.cpu().numpy(), ao)
    assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("M,H", [(1, 8), (9, 64), (300, 1536), (700, 4096), (64, 11008)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("norm", [True, False])
def test_swiglu_backward_bit_exact(ops, M, H, dtype, norm):
    """d_gate, d_up and the norm weight's gradient equal the oracle's bit for bit; the gradients are written into the
    halves of one [M, 2H] buffer."""
    gu, w, gy = _gate_up(M, H, dtype, M * 19 + H)
    if M > 2:
        gu[2, :H] = torch.linspace(-60.0, 60.0, H).to(dtype)
    gate, up = t2n(gu[:, :H]), t2n(gu[:, H:])
    rstd = None
    if norm:
        h, _, _ = O.swiglu_hidden(gate, up, _IO[dtype])
        rstd = O.rmsnorm_rstd(h, 1e-6)
    d = gu.to(DEV)
    out = torch.full((M, 2 * H), 7.0, dtype=dtype, device=DEV)
    dg, du, dw = ops.swiglu_backward(gy.to(DEV), d[:, :H], d[:, H:], w.to(DEV) if norm else None,
                                     torch.from_numpy(rstd).to(DEV) if norm else None, out=out)
    dgo, duo, dwo = O.swiglu_backward(t2n(gy), gate, up, w.numpy() if norm else None, rstd, _IO[dtype])
    assert np.array_equal(t2n(out[:, :H]), dgo) and np.array_equal(t2n(out[:, H:]), duo)
    assert dg.data_ptr() == out.data_ptr()
    if norm:
        assert np.array_equal(dw.cpu().numpy(), dwo)
    else:
        assert dw is None
    # separate output tensors give the same values
    dg2, du2, _ = ops.swiglu_backward(gy.to(DEV), d[:, :H].contiguous(), d[:, H:].contiguous(), w.to(DEV) if norm else None,
                                      torch.from_numpy(rstd).to(DEV) if norm else None)
    assert torch.equal(dg2, out[:, :H]) and torch.equal(du2, out[:, H:])


@pytest.mark.parametrize("i", range(5))
def test_swiglu_kernels_match_reference_expression_golden(ops, i):
    """The fused kernels against what the reference's `SwiGLUFFN.forward` expression and autograd give
    (tests/golden/swiglu.npz): int8 tokens within one step on at most 0.5 % of the elements, gradients within one unit of
    the I/O type (fp32: 1e-5 of the largest element), norm weight gradient within the precision the reference sums it
    in."""
    g = np.load(os.path.join(GOLDEN, "swiglu.npz"))
    io, has_norm = str(g[f"io{i}"]), bool(g[f"norm{i}"])
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[io]
    gu = torch.from_numpy(g[f"gu{i}"]).to(dt).to(DEV)
    H = gu.shape[1] // 2
    w = torch.from_numpy(g[f"w{i}"]).to(DEV) if has_norm else None
    gy = torch.from_numpy(g[f"gy{i}"]).to(dt).to(DEV)
    q, a, rstd = ops.swiglu_quantize_rows(gu[:, :H], gu[:, H:], w, float(g[f"eps{i}"]), 1e-5)
    unit = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11, "f32": 1e-5}[io]
    assert np.allclose(a.cpu().numpy(), g[f"absmax{i}"], rtol=unit * 1.01, atol=0)
    dq = np.abs(q.cpu().numpy().astype(np.int32) - g[f"q{i}"].astype(np.int32))
    assert dq.max() <= 1 and (dq != 0).mean() <= 5e-3
    dg, du, dw = ops.swiglu_backward(gy, gu[:, :H], gu[:, H:], w, rstd)
    floor = 1.0 if io == "f32" else 1e-3
    for got, ref in ((dg, g[f"dgu{i}"][:, :H]), (du, g[f"dgu{i}"][:, H:])):
        tol = unit * np.maximum(np.abs(ref), np.abs(ref).max() * floor) * 1.01
        assert np.all(np.abs(t2n(got) - ref) <= tol)
    if has_norm:
        dw_tol = {"bf16": 1e-2, "f16": 2e-3, "f32": 1e-5}[io]
        assert np.abs(dw.cpu().numpy() - g[f"dw{i}"]).max() <= dw_tol * np.abs(g[f"dw{i}"]).max()


def test_sigmoid_fixed_bit_exact_over_the_range(ops):
    """The sigmoid of the fused kernels (fixed exponential, hardware reciprocal approximation plus one Newton step)
    equals the oracle's (C float32 arithmetic with fmaf and an IEEE division) bit for bit on 48 million gate values:
    a dense sweep of [-90, 90], every float32 in [1, 2) and in (-4, -2] (all mantissa patterns), and special values."""
    dense = torch.linspace(-90.0, 90.0, 1 << 25, dtype=torch.float64).float()
    all_mant = torch.arange(0x3F800000, 0x40000000, dtype=torch.int32).view(torch.float32)          # [1, 2)
    all_mant_neg = -torch.arange(0x40000000, 0x40800000, dtype=torch.int32).view(torch.float32)     # (-4, -2]
    special = torch.tensor([0.0, -0.0, 1e-40, -1e-40, 87.0, -87.0, 88.0, -88.0, 1e30, -1e30, float("inf"), float("-inf"),
                            float("nan")])
    g = torch.cat([dense, all_mant, all_mant_neg, special])
    got = ops.sigmoid_fixed(g.to(DEV)).cpu().numpy()
    want = O.sigmoid_fixed(g.numpy())
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("gate,norm", [(True, True), (True, False), (False, True)])
def test_prelinear_rows_bit_exact(ops, dtype, gate, norm):
    """The layer input written out for the decode call equals the oracle's normalised (gated) row bit for bit."""
    M, K = 9, 1536
    gu, w, _ = _gate_up(M, K, dtype, 5)
    d = gu.to(DEV)
    y = ops.prelinear_rows(d[:, :K], d[:, K:] if gate else None, w.to(DEV) if norm else None, 1e-6)
    io = _IO[dtype]
    h = O.swiglu_hidden(t2n(gu[:, :K]), t2n(gu[:, K:]), io)[0] if gate else t2n(gu[:, :K])
    want = O.rmsnorm_forward(h, w.numpy(), 1e-6, io)[0] if norm else h
    assert y.dtype == dtype and np.array_equal(t2n(y), want)


@pytest.mark.parametrize("M", [1, 2, 7, 33, 64, 65])
@pytest.mark.parametrize("use_norm", [True, False])
def test_inference_forward_takes_the_decode_kernels_and_matches_training_forward(pkg, ops, monkeypatch, M, use_norm):
    """Without gradient recording, calls of up to 64 tokens go through the decode kernels (one small kernel forms the
    normalised / gated input first); the output is the training-time forward's, bit for bit, for a plain layer and for
    the feed-forward block."""
    calls = []
    real = ops.linear_decode
    monkeypatch.setattr(ops, "linear_decode", lambda *a, **k: (calls.append(a[0].shape), real(*a, **k))[1])
    gen = torch.Generator().manual_seed(M)
    layer = pkg.BitLinearInt2(512, 384, use_extra_rmsnorm=use_norm).to(DEV)
    layer.int2_layer.init_from_float((torch.randn(384, 512, generator=gen) * 0.03).to(DEV))
    ffn = pkg.SwiGLUFFNInt2(256, use_extra_rmsnorm=use_norm).to(DEV)          # hidden size 768
    for l, shape in ((ffn.w1, (768, 256)), (ffn.w2, (768, 256)), (ffn.w3, (256, 768))):
        l.int2_layer.init_from_float((torch.randn(*shape, generator=gen) * 0.05).to(DEV))
    if use_norm:
        with torch.no_grad():
            layer.extra_rmsnorm.weight.copy_(1.0 + 0.2 * torch.randn(512, generator=gen))
            ffn.w3.extra_rmsnorm.weight.copy_(1.0 + 0.2 * torch.randn(768, generator=gen))
    x = torch.randn(M, 512, generator=gen).to(torch.bfloat16).to(DEV)
    xf = torch.randn(M, 256, generator=gen).to(torch.bfloat16).to(DEV)
    layer.eval(); ffn.eval()
    y_train, f_train = layer(x), ffn(xf)              # gradient recording on: the GEMM path
    assert not calls
    with torch.no_grad():
        y_inf, f_inf = layer(x), ffn(xf)
    assert len(calls) == (4 if M <= 64 else 0)
    assert torch.equal(y_train, y_inf) and torch.equal(f_train, f_inf)


def test_swiglu_rejects_what_it_cannot_run(ops, pkg):
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)        # H % 8 != 0
    with pytest.raises(pkg.ElleciError) as e:
        ops.swiglu_quantize_rows(x, x)
    assert e.value.status == pkg._lib.EL_ERR_UNSUPPORTED_SHAPE
    with pytest.raises(RuntimeError):
        ops.swiglu_quantize_rows(x, x.float())
    e0 = torch.empty(0, 64, dtype=torch.bfloat16, device=DEV)
    q, a, r = ops.swiglu_quantize_rows(e0, e0, torch.ones(64, device=DEV))
    assert q.shape == (0, 64) and a.numel() == 0 and r.numel() == 0


@pytest.mark.parametrize("dtype,use_norm", [(torch.bfloat16, True), (torch.float32, True), (torch.bfloat16, False)])
def test_swiglu_ffn_module_matches_oracle_and_unfused_module(pkg, dtype, use_norm):
    """SwiGLUFFNInt2 (the reference's `w3(silu(w1 x) * w2 x)` over INT2 layers): with the gate fused, the down
    projection's output, the gradients that reach the gate and up projections' outputs and the down projection's new
    packed state equal the oracle's composite bit for bit; the same module with the gate as tensor operations agrees
    within rel-err 1e-2 (the bound of the 8-bit grid, as for the fused norm)."""
    D, M = 192, 96                        # hidden size 512
    io = _IO[dtype]
    gen = torch.Generator().manual_seed(21)
    x = torch.randn(M, D, generator=gen).to(dtype)
    dY = (torch.randn(M, D, generator=gen) * 1e-2).to(dtype)
    Ws = [torch.randn(512, D, generator=gen) * 0.05, torch.randn(512, D, generator=gen) * 0.05,
          torch.randn(D, 512, generator=gen) * 0.05]
    nw = (1.0 + 0.2 * torch.randn(512, generator=gen)).float()
    captured = {}

    def run(fused):
        ffn = pkg.SwiGLUFFNInt2(D, threshold=2, use_extra_rmsnorm=use_norm, hysteresis_order="after_dx").to(DEV)
        assert ffn.hidden_dim == 512
        for layer, W in zip((ffn.w1, ffn.w2, ffn.w3), Ws):
            layer.int2_layer.init_from_float(W.to(DEV))
        if use_norm:
            with torch.no_grad():
                ffn.w3.extra_rmsnorm.weight.copy_(nw)
        ffn.w3.fuse_swiglu = fused
        ffn.train()
        pkg.set_all_int2_lr(ffn, 0.5)
        hooks = []
        if fused:
            for name, layer in (("gate", ffn.w1), ("up", ffn.w2)):
                def fwd_hook(_m, _inp, out, name=name):
                    captured[name] = out.detach().clone()
                    out.register_hook(lambda g, name=name: captured.__setitem__("d_" + name, g.detach().clone()))
                hooks.append(layer.register_forward_hook(fwd_hook))
            captured["Wp3"] = ffn.w3.int2_layer.W_packed.cpu().numpy().copy()
            captured["Hp3"] = ffn.w3.int2_layer.H_packed.cpu().numpy().copy()
        xin = x.to(DEV).requires_grad_(True)
        y = ffn(xin)
        y.backward(dY.to(DEV))
        torch.cuda.synchronize()
        for h in hooks:
            h.remove()
        return ffn, xin, y

    ff, xf, yf = run(True)
    fu, xu, yu = run(False)
    pkg.int2_tc_ops.check_device_status(torch.device(DEV))

    gate, up = t2n(captured["gate"]), t2n(captured["up"])
    gamma3 = float(ff.w3.int2_layer.gamma.item())
    Wp3, Hp3 = captured["Wp3"], captured["Hp3"]
    Xq, ax, rstd = O.swiglu_quantize_rows(gate, up, nw.numpy() if use_norm else None, 1e-6, 1e-5, io)
    yo = O.scale_rows(O.gemm_fwd_acc(Xq, Wp3, 512), ax, gamma3)
    yo = O.to_bf16(yo) if io == "bf16" else yo
    assert np.array_equal(t2n(yf), yo)
    dxn = O.bitlinear_backward_dx(t2n(dY), Wp3, gamma3, 512, out=io)             # after_dx: the old weights
    dgo, duo, dwo = O.swiglu_backward(dxn, gate, up, nw.numpy() if use_norm else None, rstd, io)
    assert np.array_equal(t2n(captured["d_gate"]), dgo) and np.array_equal(t2n(captured["d_up"]), duo)
    if use_norm:
        assert np.array_equal(ff.w3.extra_rmsnorm.weight.grad.cpu().numpy(), dwo)
    dWo, _, _ = O.bitlinear_dw(t2n(dY), Xq, ax)
    Wn, Hn = native.c_hysteresis_step(dWo, Wp3, Hp3, 0.5, 5.0, 2, 0.001, 1, 512)
    assert np.array_equal(ff.w3.int2_layer.W_packed.cpu().numpy(), Wn) and np.array_equal(ff.w3.int2_layer.H_packed.cpu().numpy(), Hn)
    assert ff.w1.int2_layer._step_py == 1 and ff.w2.int2_layer._step_py == 1 and ff.w3.int2_layer._step_py == 1

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max())

    assert rel(yf, yu) <= 1e-2
    assert rel(xf.grad, xu.grad) <= 2e-2          # passes through two more quantised GEMMs
