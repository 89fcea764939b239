"""The CPU oracle against the golden vectors recorded from the reference (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

from oracle import int2_oracle as O
from oracle import native

from conftest import GOLDEN


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


def test_pack_unpack_matches_reference_packers():
    g = _load("pack.npz")
    for i in range(5):
        w = g[f"w{i}"]
        K = w.shape[1]
        assert np.array_equal(O.pack_ternary(w, pad_code=1), g[f"helper_packed{i}"])
        assert np.array_equal(O.pack_ternary(w, pad_code=0), g[f"module_packed{i}"])
        assert np.array_equal(O.unpack_ternary(g[f"helper_packed{i}"], K).astype(np.float32), g[f"helper_unpacked{i}"])
        assert np.array_equal(O.unpack_ternary(g[f"module_packed{i}"], K), w)
    allb = np.arange(256, dtype=np.uint8).reshape(1, 256)
    dec = O.unpack_ternary(allb, 1024)
    assert np.array_equal(dec.astype(np.float32), g["all_bytes_unpacked"])
    assert dec.min() == -1 and dec.max() == 1          # the reserved code never decodes to +2


def test_counter_roundtrip_and_sign_extension():
    rng = np.random.default_rng(3)
    for K in (1, 2, 7, 64):
        h = rng.integers(-8, 8, (5, K)).astype(np.int8)
        assert np.array_equal(O.unpack_counters(O.pack_counters(h), K), h)
    assert O.unpack_counters(np.array([[0x8F]], dtype=np.uint8), 2).tolist() == [[-1, -8]]


def test_ternarize_matches_init_from_float_and_legacy_weight_quant():
    g = _load("ternarize.npz")
    for i in range(3):
        W = g[f"W{i}"]
        gamma = float(g[f"gamma{i}"])
        q = O.ternarize(W, gamma)
        assert np.array_equal(O.pack_ternary(q, pad_code=0), g[f"W_packed{i}"])
        lg = np.float32(g[f"legacy_gamma{i}"])
        # the legacy layer returns w + (w_quant - w): equal to q*gamma up to one float32 rounding
        wq = O.ternarize(W, lg).astype(np.float32) * lg
        assert np.abs(wq - g[f"legacy_wq{i}"]).max() <= 2e-7 * max(1.0, np.abs(W).max())
        assert np.array_equal(np.rint(g[f"legacy_wq{i}"] / lg).astype(np.int8), O.ternarize(W, lg))
        assert abs(O.absmean_scale(W) - gamma) <= 1e-6 * gamma


def test_quantize_rows_matches_legacy_activation_quant():
    g = _load("legacy_layer.npz")
    for i in range(3):
        x = g[f"x{i}"]
        q, a = O.quantize_rows(x)
        s = (np.float32(127.0) / a).astype(np.float32)
        xq = (q.astype(np.float32) / s[:, None]).astype(np.float32)
        ref = g[f"xq{i}"]
        # the legacy layer returns x + (x_quant - x) in the input dtype, one rounding away from q/s
        if bool(g[f"is_bf16_{i}"]):
            assert np.abs(O.to_bf16(xq) - ref).max() <= 2.0 ** -7 * np.abs(ref).max()
        else:
            assert np.array_equal(np.rint(ref * s[:, None]).astype(np.int8), q)
            assert np.abs(xq - ref).max() <= 2e-7 * np.abs(x).max()
        assert q.min() >= -128 and q.max() <= 127


def test_layer_forward_and_dx_within_tolerance_of_legacy_layer():
    g = _load("legacy_layer.npz")
    for i in range(3):
        x, W, dY = g[f"x{i}"], g[f"W{i}"], g[f"dY{i}"]
        K = x.shape[1]
        gamma = np.float32(max(np.abs(W).mean(dtype=np.float32), 1e-5))
        Wp = O.pack_ternary(O.ternarize(W, gamma))
        bf16 = bool(g[f"is_bf16_{i}"])
        y, Xq, a = O.bitlinear_forward(x, Wp, gamma, K, out="bf16" if bf16 else "f32")
        ref = g[f"y{i}"]
        tol = 1e-2 if bf16 else 1e-5
        assert np.abs(y - ref).max() <= tol * np.abs(ref).max()
        # dX: the legacy layer back-propagates the unquantised dY; ours quantises it per token to int8
        dx = O.bitlinear_backward_dx(dY, Wp, gamma, K, out="f32")
        refdx = g[f"dx{i}"]
        assert np.abs(dx - refdx).max() <= 1e-2 * np.abs(refdx).max()
        # dW: integer definition vs the legacy float gradient (dY^T . fake-quantised x)
        dw, acc, gmax = O.bitlinear_dw(dY, Xq, a)
        refdw = g[f"dw{i}"]
        assert np.abs(dw - refdw).max() <= 2e-2 * np.abs(refdw).max()


@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_hysteresis_matches_reference_kernel_source(impl):
    g = _load("hysteresis.npz")
    step_fn = O.hysteresis_step if impl == "numpy" else native.c_hysteresis_step
    for i in range(6):
        N, K, thr, lr, ls, dec, step = g[f"params{i}"]
        N, K, thr, step = int(N), int(K), int(thr), int(step)
        W1, H1 = step_fn(g[f"dW{i}"], g[f"W0_{i}"], g[f"H0_{i}"], lr, ls, thr, dec, step, K)
        assert np.array_equal(W1, g[f"W1_{i}"]) and np.array_equal(H1, g[f"H1_{i}"])
        W2, H2 = step_fn(g[f"dW{i}"], W1, H1, lr, ls, thr, dec, step + 1, K)
        assert np.array_equal(W2, g[f"W2_{i}"]) and np.array_equal(H2, g[f"H2_{i}"])
        assert not np.array_equal(W1, g[f"W0_{i}"]) or thr >= 7       # the cases do flip weights


def test_hysteresis_row_shards_equal_the_whole_matrix():
    rng = np.random.default_rng(5)
    N, K = 24, 52
    Wp = O.pack_ternary(rng.integers(-1, 2, (N, K)).astype(np.int8))
    Hp = O.pack_counters(rng.integers(-3, 4, (N, K)).astype(np.int8))
    dW = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    Wf, Hf = O.hysteresis_step(dW, Wp, Hp, 1e-2, 5.0, 3, 0.1, 9, K)
    for g in (2, 3, 4):
        rows = N // g
        Ws, Hs = [], []
        for r in range(g):
            sl = slice(r * rows, (r + 1) * rows)
            w, h = native.c_hysteresis_step(dW[sl], Wp[sl], Hp[sl], 1e-2, 5.0, 3, 0.1, 9, K, idx_base=r * rows * K)
            Ws.append(w); Hs.append(h)
        assert np.array_equal(np.concatenate(Ws), Wf) and np.array_equal(np.concatenate(Hs), Hf)


def test_quantize_tensor_matches_reference_kernel_source():
    g = _load("quant_tensor.npz")
    for i in range(5):
        x = g[f"x_bits{i}"].view(np.float16).astype(np.float32)
        q, am = O.quantize_tensor(x)
        assert np.float32(am) == g[f"absmax{i}"][0]
        assert np.array_equal(q, g[f"q{i}"])
        deq = O.to_f16(O.dequantize_tensor(q, am))
        assert np.array_equal(deq, g[f"deq_bits{i}"].view(np.float16).astype(np.float32))


def test_c_restatement_agrees_with_numpy_on_quant_and_gemms():
    rng = np.random.default_rng(7)
    lib = native.oracle_lib()
    M, N, K = 9, 13, 50
    x = rng.standard_normal((M, K)).astype(np.float32)
    q = np.zeros((M, K), np.int8); a = np.zeros(M, np.float32)
    lib.oracle_quantize_rows(x, q, a, M, K, 1e-5)
    q2, a2 = O.quantize_rows(x)
    assert np.array_equal(q, q2) and np.array_equal(a, a2)
    Wp = O.pack_ternary(rng.integers(-1, 2, (N, K)).astype(np.int8))
    Wq = np.zeros((N, K), np.int8)
    lib.oracle_unpack_ternary(Wp, Wq, N, K)
    assert np.array_equal(Wq, O.unpack_ternary(Wp, K))
    acc = np.zeros((M, N), np.int32)
    lib.oracle_gemm_nt_i8(q, Wq, acc, M, N, K)
    assert np.array_equal(acc, O.gemm_fwd_acc(q, Wp, K))
    dYq = rng.integers(-127, 128, (M, N)).astype(np.int8)
    accx = np.zeros((M, K), np.int32)
    lib.oracle_gemm_tn_i8(np.ascontiguousarray(dYq.T), Wq, accx, N, M, K)
    assert np.array_equal(accx, O.gemm_dx_acc(dYq, Wp, K))
    accw = np.zeros((N, K), np.int32)
    lib.oracle_gemm_tn_i8(dYq, q, accw, M, N, K)
    assert np.array_equal(accw, O.gemm_dw_acc(dYq, q))


# ---- pre-linear RMSNorm: the restatement against the reference module's own outputs --------------------------------

@pytest.mark.parametrize("i", range(4))
def test_rmsnorm_restatement_matches_reference_module(i):
    """bf16/fp16 outputs and input gradients: identical values up to the rare rounding flip that torch's own float32
    summation order causes (tolerance one unit of the I/O type on at most 0.5 % of the elements); fp32: rel-err 1e-5.
    The weight gradient is summed in the I/O type by the reference and exactly here: bf16 rel-err 1e-2, fp16 2e-3."""
    g = np.load(os.path.join(GOLDEN, "rmsnorm.npz"))
    io = str(g[f"io{i}"])
    x, w, gy, eps = g[f"x{i}"], g[f"w{i}"], g[f"gy{i}"], float(g[f"eps{i}"])
    y, rstd = O.rmsnorm_forward(x, w, eps, io)
    dx, dw = O.rmsnorm_backward(gy, x, w, rstd, io)
    unit = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11, "f32": 1e-5}[io]

    def close(a, b):
        tol = unit * np.maximum(np.abs(b), np.abs(b).max() * 1e-3) * 1.01
        assert np.all(np.abs(a - b) <= tol)
        if io != "f32":
            assert (a != b).mean() <= 5e-3

    close(y, g[f"y{i}"])
    close(dx, g[f"dx{i}"])
    dw_tol = {"bf16": 1e-2, "f16": 2e-3, "f32": 1e-5}[io]
    assert np.abs(dw - g[f"dw{i}"]).max() <= dw_tol * np.abs(g[f"dw{i}"]).max()
    q, a, _ = O.rmsnorm_quantize_rows(x, w, eps, 1e-5, io)
    assert np.allclose(a, g[f"absmax{i}"], rtol=unit * 1.01, atol=0)
    dq = np.abs(q.astype(np.int32) - g[f"q{i}"].astype(np.int32))
    assert dq.max() <= 1 and (dq != 0).mean() <= 5e-3


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_package_unfused_rmsnorm_module_agrees_with_restatement(dtype):
    """The package's own `_ExtraRMSNorm` (the tensor-operation form that `fuse_rmsnorm=False` runs, and the fallback
    for shapes the fused kernel does not take) against the oracle on the CPU: outputs and input gradients equal up to
    the rare one-unit difference torch's float32 summation order causes, weight gradient to its summation precision."""
    import torch
    from conftest import load_package
    pkg = load_package()
    dt = {"bf16": torch.bfloat16, "f32": torch.float32}[dtype]
    g = torch.Generator().manual_seed(5)
    M, K = 48, 768
    x = (torch.randn(M, K, generator=g) * 1.7).to(dt).requires_grad_(True)
    norm = pkg.bitnet_int2_optimized._ExtraRMSNorm(K, eps=1e-6)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.25 * torch.randn(K, generator=g))
    gy = (torch.randn(M, K, generator=g) * 1e-2).to(dt)
    y = norm(x)
    y.backward(gy)
    xn = x.detach().float().numpy()
    yo, rstd = O.rmsnorm_forward(xn, norm.weight.detach().numpy(), 1e-6, dtype)
    dxo, dwo = O.rmsnorm_backward(gy.float().numpy(), xn, norm.weight.detach().numpy(), rstd, dtype)
    unit = {"bf16": 2.0 ** -8, "f32": 1e-5}[dtype]
    for a, b in ((yo, y.detach().float().numpy()), (dxo, x.grad.float().numpy())):
        assert np.all(np.abs(a - b) <= unit * np.maximum(np.abs(b), np.abs(b).max() * 1e-3) * 1.01)
    ref_dw = norm.weight.grad.numpy()
    assert np.abs(dwo - ref_dw).max() <= (1e-2 if dtype == "bf16" else 1e-5) * np.abs(ref_dw).max()


# ---- SwiGLU gate: the restatement against the reference's feed-forward expression -----------------------------------

@pytest.mark.parametrize("i", range(5))
def test_swiglu_restatement_matches_reference_expression(i):
    """tests/golden/swiglu.npz holds what the reference's `SwiGLUFFN.forward` expression and autograd give for
    gate|up inputs (followed by the INT2 layer's pre-linear norm, except in the last case).  The restatement fixes the
    exponential and the order of the row sums, so values may differ by one unit of the I/O type on a small fraction of
    the elements (bf16/fp16; the gate gradient passes through two more roundings: 2 %), fp32 within 1e-5."""
    g = np.load(os.path.join(GOLDEN, "swiglu.npz"))
    io, has_norm = str(g[f"io{i}"]), bool(g[f"norm{i}"])
    gu, gy, eps = g[f"gu{i}"], g[f"gy{i}"], float(g[f"eps{i}"])
    H = gu.shape[1] // 2
    gate, up = np.ascontiguousarray(gu[:, :H]), np.ascontiguousarray(gu[:, H:])
    w = g[f"w{i}"] if has_norm else None
    unit = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11, "f32": 1e-5}[io]

    def close(a, b, frac=5e-3):
        floor = 1.0 if io == "f32" else 1e-3        # fp32: error relative to the largest element
        tol = unit * np.maximum(np.abs(b), np.abs(b).max() * floor) * 1.01
        assert np.all(np.abs(a - b) <= tol)
        if io != "f32":
            assert (a != b).mean() <= frac

    h, _, _ = O.swiglu_hidden(gate, up, io)
    if has_norm:
        y, rstd = O.rmsnorm_forward(h, w, eps, io)
    else:
        y, rstd = h, None
    close(y, g[f"y{i}"])
    q, a, rstd_q = O.swiglu_quantize_rows(gate, up, w, eps, 1e-5, io)
    assert np.allclose(a, g[f"absmax{i}"], rtol=unit * 1.01, atol=0)
    dq = np.abs(q.astype(np.int32) - g[f"q{i}"].astype(np.int32))
    assert dq.max() <= 1 and (dq != 0).mean() <= 5e-3
    if has_norm:
        assert np.array_equal(rstd, rstd_q)
    dg, du, dw = O.swiglu_backward(gy, gate, up, w, rstd, io)
    close(du, g[f"dgu{i}"][:, H:], 1e-2)
    close(dg, g[f"dgu{i}"][:, :H], 2e-2)
    if has_norm:
        dw_tol = {"bf16": 1e-2, "f16": 2e-3, "f32": 1e-5}[io]
        assert np.abs(dw - g[f"dw{i}"]).max() <= dw_tol * np.abs(g[f"dw{i}"]).max()


def test_sigmoid_fixed_accuracy_and_edges():
    """The fixed exponential: within 3 float32 ulps of the exact sigmoid over the whole normal range, limits at the clamps."""
    x = np.linspace(-87, 87, 400001).astype(np.float32)
    s = O.sigmoid_fixed(x)
    ref = 1.0 / (1.0 + np.exp(-x.astype(np.float64)))
    assert np.all(np.abs(s - ref) <= 3 * np.spacing(ref.astype(np.float32)).astype(np.float64))
    e = O.sigmoid_fixed(np.array([0.0, -0.0, 104.0, 1e30, np.inf, -104.0, -1e30, -np.inf], np.float32))
    assert e[0] == 0.5 and e[1] == 0.5 and np.all(e[2:5] == 1.0) and np.all((e[5:] > 1.1e-38) & (e[5:] < 2e-38)) and e[5] == e[7]
    # a NaN gate is clamped away inside the exponential; silu = gate * sigmoid brings it back
    assert O.sigmoid_fixed(np.array([np.nan], np.float32))[0] == 1.0
    assert np.isnan(O.swiglu_hidden(np.array([[np.nan]], np.float32), np.ones((1, 1), np.float32), "f32")[0][0, 0])
