"""Parity of the CUDA kernels with the CPU oracle, through the package's operator surface (which ends in the
C ABI).  Integer results are compared bit for bit; scaled outputs share the oracle's float32 arithmetic and are
compared exactly too (the tolerances the path promises, 1e-2 for bf16 and 1e-5 for fp32, are asserted against
the reference's own legacy layer in test_oracle_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import int2_oracle as O
from oracle import native

from conftest import GOLDEN
from helpers import make_layer_inputs, random_packed, t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops(pkg):
    assert os.path.exists(pkg.LIB_PATH), "the CUDA library must be built in-tree"
    return pkg.int2_tc_ops


def _cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t if dtype is None else t.to(dtype)).to(DEV)


# ---- weight format ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("N,K", [(8, 8), (5, 7), (16, 130), (3, 1), (33, 64), (130, 126), (256, 256)])
def test_pack_unpack_bit_exact(ops, N, K):
    rng = np.random.default_rng(N * 1000 + K)
    w = rng.integers(-1, 2, (N, K)).astype(np.int8)
    for pad in (0, 1):
        got = ops.pack_int2(_cuda(w), pad_code=pad).cpu().numpy()
        assert np.array_equal(got, O.pack_ternary(w, pad_code=pad))
    Wp = rng.integers(0, 256, (N, (K + 3) // 4)).astype(np.uint8)       # every code, also the reserved one
    for dt in (torch.float16, torch.bfloat16, torch.float32, torch.int8):
        out = torch.empty(N, K, dtype=dt, device=DEV)
        ops.unpack_int2(_cuda(Wp), out, K)
        assert np.array_equal(t2n(out).astype(np.int8), O.unpack_ternary(Wp, K))


def test_ternarize_pack_matches_golden_init_from_float(ops):
    g = np.load(os.path.join(GOLDEN, "ternarize.npz"))
    for i in range(3):
        got = ops.ternarize_pack(_cuda(g[f"W{i}"]), float(g[f"gamma{i}"])).cpu().numpy()
        assert np.array_equal(got, g[f"W_packed{i}"])


# ---- activation quantisation -----------------------------------------------------------------------------------

@pytest.mark.parametrize("M,K", [(1, 255), (7, 64), (16, 1536), (33, 100), (4, 11008), (5, 8)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quantize_rows_bit_exact(ops, M, K, dtype):
    g = torch.Generator().manual_seed(M * 7 + K)
    x = (torch.randn(M, K, generator=g) * 3.0).to(dtype)
    x[0, : min(K, 3)] = 0.0
    if M > 2:
        x[1] = 0.0                      # all-zero token: absmax clamps to eps
        x[2, 0] = float("inf")          # non-finite values count as zero
        x[2, K - 1] = float("nan")
    if M > 4:
        x[3, K // 2] = float("nan")     # NaN alone: the row keeps the unchecked conversion
        x[4, K // 3] = float("-inf")
    q, a = ops.quantize_rows(x.to(DEV))
    qo, ao = O.quantize_rows(t2n(x))
    assert np.array_equal(a.cpu().numpy(), ao)
    assert np.array_equal(q.cpu().numpy(), qo)


# ---- pre-linear RMSNorm fused with the quantiser ---------------------------------------------------------------

_IO = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}


@pytest.mark.parametrize("M,K", [(1, 8), (7, 64), (33, 1536), (16, 4096), (5, 11008)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rmsnorm_quantize_rows_bit_exact(ops, M, K, dtype):
    """int8 tokens, absmax and rstd equal the oracle's (RMSNorm as the reference writes it, then the per-token
    quantiser) bit for bit: row sums are accumulated in float64 on both sides."""
    g = torch.Generator().manual_seed(M * 11 + K)
    x = (torch.randn(M, K, generator=g) * 2.5).to(dtype)
    w = (1.0 + 0.3 * torch.randn(K, generator=g)).float()
    if M > 2:
        x[1] = 0.0                          # all-zero token: rstd = 1/sqrt(eps), absmax clamps to the quantiser's eps
        x[2, 0] = float("nan")              # a NaN poisons the token's sum of squares: the whole token quantises to 0
    if M > 4:
        x[3, K - 1] = float("inf")
    q, a, rstd = ops.rmsnorm_quantize_rows(x.to(DEV), w.to(DEV), 1e-6, 1e-5)
    with np.errstate(all="ignore"):
        qo, ao, ro = O.rmsnorm_quantize_rows(t2n(x), w.numpy(), 1e-6, 1e-5, _IO[dtype])
    assert np.array_equal(rstd.cpu().numpy(), ro, equal_nan=True)
    assert np.array_equal(a.cpu().numpy(), ao)
    assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("i", range(4))
def test_rmsnorm_kernels_match_reference_module_golden(ops, i):
    """The fused kernels against the reference module's own outputs (tests/golden/rmsnorm.npz): int8 tokens within
    one step on at most 0.5 % of the elements (torch's float32 summation order differs), input gradient within one
    unit of the I/O type, weight gradient within the precision the reference sums it in."""
    g = np.load(os.path.join(GOLDEN, "rmsnorm.npz"))
    io = str(g[f"io{i}"])
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[io]
    x = torch.from_numpy(g[f"x{i}"]).to(dt).to(DEV)
    w = torch.from_numpy(g[f"w{i}"]).to(DEV)
    gy = torch.from_numpy(g[f"gy{i}"]).to(dt).to(DEV)
    q, a, rstd = ops.rmsnorm_quantize_rows(x, w, float(g[f"eps{i}"]), 1e-5)
    unit = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11, "f32": 1e-5}[io]
    assert np.allclose(a.cpu().numpy(), g[f"absmax{i}"], rtol=unit * 1.01, atol=0)
    dq = np.abs(q.cpu().numpy().astype(np.int32) - g[f"q{i}"].astype(np.int32))
    assert dq.max() <= 1 and (dq != 0).mean() <= 5e-3
    dx, dw = ops.rmsnorm_backward(gy, x, w, rstd)
    ref_dx = g[f"dx{i}"]
    tol = unit * np.maximum(np.abs(ref_dx), np.abs(ref_dx).max() * 1e-3) * 1.01
    assert np.all(np.abs(t2n(dx) - ref_dx) <= tol)
    dw_tol = {"bf16": 1e-2, "f16": 2e-3, "f32": 1e-5}[io]
    assert np.abs(dw.cpu().numpy() - g[f"dw{i}"]).max() <= dw_tol * np.abs(g[f"dw{i}"]).max()


@pytest.mark.parametrize("M,K", [(1, 8), (9, 64), (300, 1536), (1200, 4096), (64, 11008)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rmsnorm_backward_bit_exact(ops, M, K, dtype):
    """dx and dweight equal the oracle's bit for bit (float64 row and column sums on both sides)."""
    g = torch.Generator().manual_seed(M * 13 + K)
    x = (torch.randn(M, K, generator=g) * 1.5).to(dtype)
    gy = (torch.randn(M, K, generator=g) * 1e-2).to(dtype)
    w = (1.0 + 0.3 * torch.randn(K, generator=g)).float()
    rstd = torch.from_numpy(O.rmsnorm_rstd(t2n(x), 1e-6))
    dx, dw = ops.rmsnorm_backward(gy.to(DEV), x.to(DEV), w.to(DEV), rstd.to(DEV))
    dxo, dwo = O.rmsnorm_backward(t2n(gy), t2n(x), w.numpy(), rstd.numpy(), _IO[dtype])
    assert np.array_equal(t2n(dx), dxo)
    assert np.array_equal(dw.cpu().numpy(), dwo)


def test_rmsnorm_rejects_what_it_cannot_run(ops, pkg):
    x = torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV)        # K % 8 != 0
    with pytest.raises(pkg.ElleciError) as e:
        ops.rmsnorm_quantize_rows(x, torch.ones(100, device=DEV))
    assert e.value.status == pkg._lib.EL_ERR_UNSUPPORTED_SHAPE
    assert not ops.rmsnorm_supported(x)
    q, a, r = ops.rmsnorm_quantize_rows(torch.empty(0, 64, dtype=torch.bfloat16, device=DEV), torch.ones(64, device=DEV))
    assert q.shape == (0, 64) and a.numel() == 0 and r.numel() == 0


def test_quantize_rows_empty_inputs(ops):
    q, a = ops.quantize_rows(torch.empty(0, 64, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (0, 64) and a.numel() == 0
    q, a = ops.quantize_rows(torch.empty(3, 0, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (3, 0) and np.allclose(a.cpu().numpy(), 1e-5)


@pytest.mark.parametrize("i", range(5))
def test_quantize_tensor_matches_reference_kernel_golden(ops, i):
    g = np.load(os.path.join(GOLDEN, "quant_tensor.npz"))
    x = torch.from_numpy(g[f"x_bits{i}"].view(np.float16).copy()).to(DEV)
    q, am = ops.quantize_activation_async(x, torch.zeros(1, device=DEV))
    assert am.cpu().numpy()[0] == g[f"absmax{i}"][0]
    assert np.array_equal(q.cpu().numpy(), g[f"q{i}"])
    deq = ops.dequantize_activation(q, am)
    assert np.array_equal(deq.cpu().numpy().view(np.uint16), g[f"deq_bits{i}"])


@pytest.mark.parametrize("special", [False, True])
def test_grad_quantisation_bit_exact(ops, special):
    d = make_layer_inputs(37, 96, 80, seed=3, dy_std=1e-3)
    x, dY = d["x"], d["dY"]
    if special:                         # non-finite gradients count as zero
        dY = dY.clone()
        dY[0, 0], dY[5, 79], dY[36, 40], dY[7, 7] = float("nan"), float("inf"), float("-inf"), -0.0
    _, ax = ops.quantize_rows(x.to(DEV))
    dYq, ady, gmax = ops.quantize_rows(dY.to(DEV), 1e-30, fold_absmax=ax)
    Gq = ops.quantize_grad(dY.to(DEV), ax, gmax)
    _, axo = O.quantize_rows(t2n(x))
    dYqo, adyo = O.quantize_rows(t2n(dY), eps=1e-30)
    Gqo, go = O.grad_quantize(t2n(dY), axo)
    assert np.array_equal(dYq.cpu().numpy(), dYqo) and np.array_equal(ady.cpu().numpy(), adyo)
    assert gmax.cpu().numpy()[0] == go
    assert np.array_equal(Gq.cpu().numpy(), Gqo)


# ---- hysteresis ---------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("i", range(6))
def test_hysteresis_matches_reference_kernel_golden(ops, i):
    g = np.load(os.path.join(GOLDEN, "hysteresis.npz"))
    N, K, thr, lr, ls, dec, step = g[f"params{i}"]
    N, K, thr, step = int(N), int(K), int(thr), int(step)
    W, H = _cuda(g[f"W0_{i}"]), _cuda(g[f"H0_{i}"])
    dW = _cuda(g[f"dW{i}"])
    ops.hysteresis_step_v2(dW, W, H, lr, ls, thr, dec, step)
    assert np.array_equal(W.cpu().numpy(), g[f"W1_{i}"]) and np.array_equal(H.cpu().numpy(), g[f"H1_{i}"])
    ops.hysteresis_step_v2(dW, W, H, lr, ls, thr, dec, step + 1)
    assert np.array_equal(W.cpu().numpy(), g[f"W2_{i}"]) and np.array_equal(H.cpu().numpy(), g[f"H2_{i}"])


@pytest.mark.parametrize("N,K,thr", [(64, 64, 2), (37, 50, 3), (5, 7, 7), (16, 130, 1), (8, 20, 2), (1536, 1536, 2)])
def test_hysteresis_bit_exact_with_special_values(ops, N, K, thr):
    rng = np.random.default_rng(N + K)
    Wp = rng.integers(0, 256, (N, (K + 3) // 4)).astype(np.uint8)
    Hp = O.pack_counters(rng.integers(-7, 8, (N, K)).astype(np.int8))
    dW = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    flat = dW.reshape(-1)
    flat[0], flat[1 % flat.size], flat[2 % flat.size] = np.nan, np.inf, -np.inf
    flat[3 % flat.size], flat[4 % flat.size] = 1e-42, -0.0
    for step, ftz in ((1, True), (77, False), (4000000000, True)):
        W, H = _cuda(Wp), _cuda(Hp)
        ops.hysteresis_step_v2(_cuda(dW), W, H, 3e-3, 5.0, thr, 0.2, step, ftz=ftz)
        Wo, Ho = native.c_hysteresis_step(dW, Wp, Hp, 3e-3, 5.0, thr, 0.2, step, K, ftz=ftz)
        assert np.array_equal(W.cpu().numpy(), Wo) and np.array_equal(H.cpu().numpy(), Ho)


def test_hysteresis_row_shards_equal_whole(ops):
    rng = np.random.default_rng(11)
    N, K = 48, 64
    Wp, _ = random_packed(N, K, 1)
    Hp = O.pack_counters(rng.integers(-3, 4, (N, K)).astype(np.int8))
    dW = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    Wf, Hf = native.c_hysteresis_step(dW, Wp, Hp, 1e-2, 5.0, 3, 0.1, 5, K)
    for g in (2, 4):
        rows = N // g
        for r in range(g):
            sl = slice(r * rows, (r + 1) * rows)
            W, H = _cuda(Wp[sl]), _cuda(Hp[sl])
            ops.hysteresis_step_v2(_cuda(dW[sl]), W, H, 1e-2, 5.0, 3, 0.1, 5, idx_base=r * rows * K)
            assert np.array_equal(W.cpu().numpy(), Wf[sl]) and np.array_equal(H.cpu().numpy(), Hf[sl])


def test_hysteresis_rejects_bad_arguments(ops):
    W = torch.zeros(4, 2, dtype=torch.uint8, device=DEV)
    H = torch.zeros(4, 4, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError):
        ops.hysteresis_step_v2(torch.zeros(4, 8, device=DEV).half(), W, H, 1e-3, 5.0, 2, 0.0, 1)       # dtype
    with pytest.raises(RuntimeError):
        ops.hysteresis_step_v2(torch.zeros(4, 9, device=DEV), W, H, 1e-3, 5.0, 2, 0.0, 1)              # packed shape
    with pytest.raises(RuntimeError):
        ops.hysteresis_step_v2(torch.zeros(32, device=DEV), W, H, 1e-3, 5.0, 2, 0.0, 1)                # not 2-D


# ---- GEMMs --------------------------------------------------------------------------------------------------------

# the reference's own edge grid (kernels/tests/test_correctness.py:17-42) plus shapes the layer really has
SIMPLE_SHAPES = [(8, 8, 8), (256, 256, 256), (256, 260, 256), (128, 128, 130), (64, 48, 200), (33, 16, 16), (130, 126, 126),
                 (1, 64, 64)]
# tensor-core constraints: K % 64 == 0 (packed pitch), N % 16 == 0 (dYq / Gq pitch); M is free
TC_SHAPES = [(128, 256, 128), (128, 256, 256), (256, 512, 384), (100, 304, 192), (1024, 1536, 1536), (160, 272, 1088),
             (37, 64, 64), (300, 1376, 4096), (129, 16, 64), (700, 528, 320),
             # a handful of rows (the tile is mostly padding): what a small batch with gradients, or more than 64 tokens at
             # inference, sends here
             (1, 256, 128), (8, 512, 256), (31, 304, 192),
             # ragged tiles on a deeper reduction; more tiles (81) than CTA pairs, i.e. a partial second wave
             (600, 2000, 2048), (2304, 2304, 2048)]


def _gemm_inputs(M, N, K, seed):
    rng = np.random.default_rng(seed)
    Xq = rng.integers(-128, 128, (M, K)).astype(np.int8)
    dYq = rng.integers(-128, 128, (M, N)).astype(np.int8)
    Wp, w = random_packed(N, K, seed)
    ax = (rng.random(M).astype(np.float32) * 4 + 0.5)
    ay = (rng.random(M).astype(np.float32) * 1e-2 + 1e-4)
    return Xq, dYq, Wp, ax, ay


def _check_gemms(ops, M, N, K, path, seed=0):
    Xq, dYq, Wp, ax, ay = _gemm_inputs(M, N, K, seed)
    gamma = 0.0173
    dXq, ddY, dWp, dax, day = _cuda(Xq), _cuda(dYq), _cuda(Wp), _cuda(ax), _cuda(ay)
    acc_f = O.gemm_fwd_acc(Xq, Wp, K)
    acc_x = O.gemm_dx_acc(dYq, Wp, K)
    acc_w = O.gemm_dw_acc(dYq, Xq)
    # raw int32 accumulators: bit-exact
    assert np.array_equal(ops.matmul_rows(dXq, dWp, dax, gamma, torch.int32, path).cpu().numpy(), acc_f)
    assert np.array_equal(ops.backward_input_rows(ddY, dWp, day, gamma, K, torch.int32, path).cpu().numpy(), acc_x)
    g1 = torch.tensor([0.37], device=DEV)
    assert np.array_equal(ops.weight_grad(ddY, dXq, g1, raw=True, path=path).cpu().numpy(), acc_w)
    # scaled outputs: the oracle's float32 arithmetic, then the output rounding
    for dt, rnd in ((torch.float32, lambda v: v), (torch.bfloat16, O.to_bf16), (torch.float16, O.to_f16)):
        y = ops.matmul_rows(dXq, dWp, dax, gamma, dt, path)
        assert np.array_equal(t2n(y), rnd(O.scale_rows(acc_f, ax, gamma)))
        dx = ops.backward_input_rows(ddY, dWp, day, gamma, K, dt, path)
        assert np.array_equal(t2n(dx), rnd(O.scale_rows(acc_x, ay, gamma)))
    # per-tensor scale (the reference extension's calling convention)
    s1 = torch.tensor([2.5], device=DEV)
    y = ops.matmul_int8(dXq, dWp, s1, gamma, path=path)
    assert np.array_equal(t2n(y), O.to_f16(O.scale_rows(acc_f, np.float32(2.5), gamma)))
    dw = ops.weight_grad(ddY, dXq, g1, path=path)
    assert np.array_equal(dw.cpu().numpy(), O.dw_from_acc(acc_w, np.float32(0.37)))


@pytest.mark.parametrize("M,N,K", SIMPLE_SHAPES)
def test_gemms_cuda_core_path_bit_exact(ops, pkg, M, N, K):
    _check_gemms(ops, M, N, K, pkg._lib.EL_PATH_SIMPLE, seed=M + N + K)


@pytest.mark.parametrize("single_cta", [False, True])
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemms_tensor_core_path_bit_exact(ops, pkg, M, N, K, single_cta):
    """Forward and dX run on CTA pairs (cta_group::2) or, on request, on the single-CTA kernel; dW has one kernel."""
    _check_gemms(ops, M, N, K, pkg._lib.EL_PATH_TC_SINGLE if single_cta else pkg._lib.EL_PATH_TC, seed=M + N + K)
    ops.check_device_status(torch.device(DEV))


def test_pair_kernel_banded_tile_order_bit_exact(ops, pkg):
    """A reduction so deep (65536) that the pair kernel orders its tiles in bands of two 256-row tiles: five row
    tiles give the bands 2 + 2 + 1 (ragged last band), two column tiles each."""
    rng = np.random.default_rng(21)
    M, big, small = 1280, 65536, 512
    Xq = rng.integers(-128, 128, (M, big)).astype(np.int8)
    Wp, _ = random_packed(small, big, 3)                     # forward: K = 65536, N = 512
    a = _cuda(np.ones(M, np.float32))
    y = ops.matmul_rows(_cuda(Xq), _cuda(Wp), a, 1.0, torch.int32, pkg._lib.EL_PATH_TC)
    assert np.array_equal(y.cpu().numpy(), O.gemm_fwd_acc(Xq, Wp, big))
    del Xq, Wp
    dYq = rng.integers(-128, 128, (M, big)).astype(np.int8)
    Wp2, _ = random_packed(big, small, 4)                    # dX: reduction over N = 65536, K = 512 output columns
    dx = ops.backward_input_rows(_cuda(dYq), _cuda(Wp2), a, 1.0, small, torch.int32, pkg._lib.EL_PATH_TC)
    assert np.array_equal(dx.cpu().numpy(), O.gemm_dx_acc(dYq, Wp2, small))
    ops.check_device_status(torch.device(DEV))


def test_tensor_core_forward_with_ragged_n(ops, pkg):
    """The forward GEMM alone has no constraint on N (only dX and dW read a pitch of N bytes)."""
    M, N, K = 200, 300, 320
    Xq, _, Wp, ax, _ = _gemm_inputs(M, N, K, 5)
    y = ops.matmul_rows(_cuda(Xq), _cuda(Wp), _cuda(ax), 0.02, torch.bfloat16, pkg._lib.EL_PATH_TC)
    assert np.array_equal(t2n(y), O.to_bf16(O.scale_rows(O.gemm_fwd_acc(Xq, Wp, K), ax, 0.02)))
    ops.check_device_status(torch.device(DEV))


def test_tensor_core_path_refuses_unaligned_shapes(ops, pkg):
    Xq = torch.zeros(128, 100, dtype=torch.int8, device=DEV)      # K % 64 != 0
    Wp = torch.zeros(64, 25, dtype=torch.uint8, device=DEV)
    a = torch.ones(128, device=DEV)
    with pytest.raises(pkg.ElleciError) as e:
        ops.matmul_rows(Xq, Wp, a, 1.0, torch.bfloat16, pkg._lib.EL_PATH_TC)
    assert e.value.status == pkg._lib.EL_ERR_UNSUPPORTED_SHAPE
    # the automatic path takes the same problem through the CUDA-core kernel
    assert ops.matmul_rows(Xq, Wp, a, 1.0, torch.bfloat16).shape == (128, 64)
    with pytest.raises(RuntimeError):
        ops.matmul_rows(Xq, torch.zeros(64, 26, dtype=torch.uint8, device=DEV), a, 1.0)     # packed_K mismatch


@pytest.mark.parametrize("M,N,K,thr", [(128, 128, 256, 2), (200, 272, 96, 3), (1024, 1536, 1536, 2)])
def test_fused_dw_hysteresis_bit_exact(ops, M, N, K, thr):
    rng = np.random.default_rng(M + N)
    Gq = rng.integers(-127, 128, (M, N)).astype(np.int8)
    Xq = rng.integers(-128, 128, (M, K)).astype(np.int8)
    Wp, _ = random_packed(N, K, 5)
    Hp = O.pack_counters(rng.integers(-3, 4, (N, K)).astype(np.int8))
    g = np.float32(3e-3 if M < 1000 else 4e-4)
    W, H = _cuda(Wp), _cuda(Hp)
    ops.dw_hysteresis(_cuda(Gq), _cuda(Xq), torch.tensor([g], device=DEV), W, H, 1e-2, 5.0, thr, 0.01, 3, idx_base=1000)
    ops.check_device_status(torch.device(DEV))
    dW = O.dw_from_acc(O.gemm_dw_acc(Gq, Xq), g)
    Wo, Ho = native.c_hysteresis_step(dW, Wp, Hp, 1e-2, 5.0, thr, 0.01, 3, K, idx_base=1000)
    assert np.array_equal(W.cpu().numpy(), Wo) and np.array_equal(H.cpu().numpy(), Ho)
    assert (O.unpack_ternary(Wo, K) != O.unpack_ternary(Wp, K)).mean() > 0.01      # the case does flip weights


# ---- small-M decode path -------------------------------------------------------------------------------------------

@pytest.fixture
def gemv_threshold(ops):
    """Lets a test choose between the few-token CUDA-core GEMV (up to `v` tokens), the warp-MMA kernel (up to `mma`
    tokens: one launch up to 8, quantiser + kernel on the quantised tokens beyond) and the tcgen05 stream-K kernel (the
    rest)."""
    def set_(v, mma=0):
        assert ops._lib.lib().el_set_decode_gemv_max_tokens(v) == 0
        assert ops._lib.lib().el_set_decode_mma_max_tokens(mma) == 0
    yield set_
    set_(2, 64)


@pytest.mark.parametrize("gemv_max", [0, 8, "mma"])
@pytest.mark.parametrize("M", [1, 3, 8, 17, 32, 64])
@pytest.mark.parametrize("K,N", [(4096, 11008), (11008, 4096), (256, 384), (192, 100)])
def test_linear_decode_bit_exact(ops, gemv_threshold, M, K, N, gemv_max):
    """The weight-streaming small-M kernel gives the integers and the rounding of quantize_rows + the forward GEMM;
    run twice on one workspace to show that a call leaves the workspace clean."""
    g = torch.Generator().manual_seed(M + K + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    Wp, _ = random_packed(N, K, seed=K + N)
    gamma = 0.0161
    Xq, ax = O.quantize_rows(t2n(x))
    want = O.to_bf16(O.scale_rows(O.gemm_fwd_acc(Xq, Wp, K), ax, gamma))
    # 0: tcgen05 kernel for every M; 8: CUDA-core GEMV up to 8 tokens; "mma": warp-MMA kernel wherever the tokens fit
    if gemv_max == "mma":
        gemv_threshold(0, 64)
    else:
        gemv_threshold(gemv_max)
    ws = torch.zeros(ops._lib.lib().el_decode_workspace_bytes(N), dtype=torch.uint8, device=DEV)
    Wd = _cuda(Wp)
    for _ in range(2):
        y = ops.linear_decode(x.to(DEV), Wd, gamma, workspace=ws)
        assert np.array_equal(t2n(y), want)
    assert int(ws.view(torch.int32).abs().sum().item()) == 0
    ops.check_device_status(torch.device(DEV))


@pytest.mark.parametrize("gemv_max", [0, 8, "mma"])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_linear_decode_counts_non_finite_tokens_as_zero(ops, gemv_threshold, M, gemv_max):
    """NaN and infinities in the tokens quantise to 0 and do not enter the absmax (NaN alone keeps the GEMV's fast
    path, an infinity sends it through the checked one)."""
    K, N = 1024, 328
    g = torch.Generator().manual_seed(90 + M)
    if gemv_max == "mma":
        gemv_threshold(0, 64)
    else:
        gemv_threshold(gemv_max)
    Wp, _ = random_packed(N, K, seed=77)
    Wd = _cuda(Wp)
    for kind in ("nan", "inf", "both"):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        if kind in ("nan", "both"):
            x[0, 5] = float("nan")
            x[M - 1, K - 1] = float("nan")
        if kind in ("inf", "both"):
            x[M // 2, 17] = float("inf")
            x[0, 900] = float("-inf")
        Xq, ax = O.quantize_rows(t2n(x))
        want = O.to_bf16(O.scale_rows(O.gemm_fwd_acc(Xq, Wp, K), ax, 0.02))
        y = ops.linear_decode(x.to(DEV), Wd, 0.02)
        assert np.array_equal(t2n(y), want), kind
    ops.check_device_status(torch.device(DEV))


@pytest.mark.parametrize("M", [1, 4, 12])
def test_linear_decode_chain_with_overlap_equals_plain_chain(ops, M):
    """Dependent-launch overlap: a chain of calls in which every call's tokens are the previous call's output (so a
    call that started too early would read stale tokens) gives bit-identical results with the overlap on, in plain
    stream order and replayed from a CUDA graph."""
    K = N = 2048
    g = torch.Generator().manual_seed(11 + M)
    x0 = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    Ws = [_cuda(random_packed(N, K, seed=50 + i)[0]) for i in range(6)]

    def chain(x):
        outs = []
        for W in Ws:
            x = ops.linear_decode(x, W, 0.05)
            outs.append(x)
        return outs

    ops.set_decode_overlap(False)
    want = [o.clone() for o in chain(x0)]
    assert float(want[-1].float().abs().max()) > 0
    try:
        ops.set_decode_overlap(True)
        got = chain(x0)
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            got_g = chain(x0)
        for o in got_g:
            o.zero_()
        graph.replay()
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(got_g, want):
            assert torch.equal(a, b)
    finally:
        ops.set_decode_overlap(False)
    ops.check_device_status(torch.device(DEV))


def test_linear_decode_rejects_what_it_cannot_run(ops, pkg):
    Wp = torch.zeros(64, 25, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError):
        ops.linear_decode(torch.zeros(65, 100, dtype=torch.bfloat16, device=DEV), Wp, 1.0)       # more than 64 tokens
    with pytest.raises(pkg.ElleciError) as e:
        ops.linear_decode(torch.zeros(4, 100, dtype=torch.bfloat16, device=DEV), Wp, 1.0)        # K % 64 != 0
    assert e.value.status == pkg._lib.EL_ERR_UNSUPPORTED_SHAPE


# ---- N-sharded dX: scatter of the partial sums, the ranks emulated one after the other on one GPU ------------------

@pytest.mark.parametrize("g,M,K,N", [(2, 512, 256, 512), (4, 2048, 512, 1024), (8, 4096, 256, 2048), (8, 256, 128, 512)])
def test_dx_scatter_of_all_ranks_adds_up_to_the_unsharded_sums(ops, g, M, K, N):
    """Every rank's shard of the dX GEMM stores its int32 partial sums into slot `rank` of the owners' staging buffers
    (each rank walks the row tiles from its own rows on); launched rank after rank on one device with local buffers,
    the slots must add up to the unsharded integer sums, row block by row block."""
    rng = np.random.default_rng(g * 1000 + M)
    dYq = rng.integers(-128, 128, (M, N)).astype(np.int8)
    Wp, _ = random_packed(N, K, 9)
    Mr, Ns = M // g, N // g
    parts = [torch.full((g, Mr, K), -7, dtype=torch.int32, device=DEV) for _ in range(g)]       # owner d: [source rank, rows, K]
    ptrs = [p.data_ptr() for p in parts]
    for r in range(g):
        shard = _cuda(np.ascontiguousarray(dYq[:, r * Ns:(r + 1) * Ns]))
        ops.backward_input_scatter(shard, _cuda(Wp[r * Ns:(r + 1) * Ns]), K, ptrs, r)
    ops.check_device_status(torch.device(DEV))
    want = O.gemm_dx_acc(dYq, Wp, K)
    for d in range(g):
        for r in range(g):
            part = O.gemm_dx_acc(np.ascontiguousarray(dYq[d * Mr:(d + 1) * Mr, r * Ns:(r + 1) * Ns]), Wp[r * Ns:(r + 1) * Ns], K)
            assert np.array_equal(parts[d][r].cpu().numpy(), part), (d, r)
        assert np.array_equal(parts[d].sum(0).cpu().numpy(), want[d * Mr:(d + 1) * Mr])


# ---- N-sharded forward and the owner's half of the dX exchange, ranks emulated one after the other on one GPU --------

@pytest.mark.parametrize("g,M,K,N", [(2, 512, 256, 512), (4, 300, 512, 1024), (8, 1024, 256, 2048), (8, 256, 128, 256)])
def test_fwd_gather_of_all_ranks_fills_every_output_buffer(ops, g, M, K, N):
    """Every rank's shard of the forward GEMM writes its [M, N/g] block at column r*N/g of ALL g output buffers (the
    all-gather is the epilogue's TMA stores).  Launched rank after rank on one device with g local buffers standing in
    for the ranks' buffers, every buffer must end up holding the unsharded layer's output, and nothing else is touched."""
    rng = np.random.default_rng(g * 100 + M)
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(torch.bfloat16)
    Wp, _ = random_packed(N, K, 21)
    gamma = 0.0173
    Xq, ax = O.quantize_rows(t2n(x))
    want = O.to_bf16(O.scale_rows(O.gemm_fwd_acc(Xq, Wp, K), ax, gamma))
    Ns = N // g
    pad = 64                                                    # guard columns right of the matrix: must stay untouched
    bufs = [torch.full((M, N + pad), 3.0, dtype=torch.bfloat16, device=DEV) for _ in range(g)]
    Xd, ad = _cuda(Xq), _cuda(ax)
    for r in range(g):
        ops.matmul_rows_gather(Xd, _cuda(Wp[r * Ns:(r + 1) * Ns]), ad, gamma, [b.data_ptr() for b in bufs], N + pad, r * Ns,
                               torch.bfloat16)
    ops.check_device_status(torch.device(DEV))
    for d in range(g):
        got = t2n(bufs[d])
        assert np.array_equal(got[:, :N], want), d
        assert np.all(got[:, N:] == 3.0), d


@pytest.mark.parametrize("g,M,K", [(2, 512, 256), (4, 2048, 512), (8, 256, 128), (8, 4096, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_reduce_scale_gather_of_all_owners_completes_dx(ops, g, M, K, dtype):
    """Owner d adds the g slots of its staging buffer, scales the rows it owns and writes them into every rank's dX.
    With all owners launched one after the other on one device, every dX buffer must equal scale_rows of the summed
    partial sums (integer addition first, one rounding at the end), whichever owner produced a row."""
    rng = np.random.default_rng(g + M + K)
    Mr = M // g
    parts = rng.integers(-(1 << 20), 1 << 20, (g, g, Mr, K)).astype(np.int32)          # [owner, source rank, rows, K]
    ax = (rng.random(M).astype(np.float32) + 0.25)
    gamma = 0.0211
    total = parts.astype(np.int64).sum(1).reshape(M, K)
    assert np.abs(total).max() < 2 ** 31
    want = O.scale_rows(total.astype(np.int32), ax, gamma)
    want = O.to_bf16(want) if dtype == torch.bfloat16 else want.astype(np.float32)
    outs = [torch.full((M, K), -5.0, dtype=dtype, device=DEV) for _ in range(g)]
    ad = _cuda(ax)
    for d in range(g):
        ops.reduce_scale_gather(_cuda(parts[d]), [o.data_ptr() for o in outs], d, ad, gamma, M, K, dtype)
    for r in range(g):
        assert np.array_equal(t2n(outs[r]), want), r


# ---- bounded device-side waits and first calls from several host threads -----------------------------------------

def test_peer_barrier_reports_a_rank_that_never_arrives_and_leaves_the_device_usable(ops, pkg):
    """Two ranks' flag arrays live on this one device; only rank 0 ever launches.  With the wait limit set to a
    millisecond the barrier must come back by itself, name the missing rank (code 40 + 1) in the status word and leave
    the context healthy.  A barrier whose partner has already signalled (its flag written beforehand) passes at once."""
    dev = torch.device(DEV)
    handle = pkg._lib.lib()
    flags = [torch.zeros(8, dtype=torch.int32, device=DEV) for _ in range(2)]
    ptrs = [f.data_ptr() for f in flags]
    status = ops.device_status(dev)
    status.zero_()
    assert handle.el_set_peer_barrier_limit_us(1000) == 0
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        ops.peer_barrier(ptrs, 0, 1, dev)                   # rank 1 never signals
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0                  # a millisecond of cycles, not the default of seconds
        assert int(status.item()) == 41
        with pytest.raises(pkg.ElleciError):
            ops.check_device_status(dev)                    # raises and clears the word
        assert int(status.item()) == 0
        assert flags[0][0].item() == 1 and flags[1][0].item() == 1      # rank 0 did publish its epoch everywhere
        # the partner's arrival written by hand: epoch 2 passes without a wait
        flags[0][1] = 2
        ops.peer_barrier(ptrs, 0, 2, dev)
        torch.cuda.synchronize()
        ops.check_device_status(dev)
        # a barrier that carries a word: rank 0's value lands at its offset of every rank's buffer before the epoch does
        word = torch.tensor([3.25], dtype=torch.float32, device=DEV)
        slots = [torch.zeros(8, dtype=torch.float32, device=DEV) for _ in range(2)]
        flags[0][1] = 3
        ops.peer_barrier_put(ptrs, 0, 3, dev, word, [s_.data_ptr() for s_ in slots], 4 * 5)
        torch.cuda.synchronize()
        ops.check_device_status(dev)
        for s_ in slots:
            assert s_[5].item() == 3.25 and float(s_.sum()) == 3.25
        assert flags[0][0].item() == 3 and flags[1][0].item() == 3
        # and the device still computes
        Wp, w = random_packed(64, 64, 5)
        out = torch.empty(64, 64, dtype=torch.int8, device=DEV)
        ops.unpack_int2(_cuda(Wp), out, 64)
        assert np.array_equal(out.cpu().numpy(), w)
    finally:
        assert handle.el_set_peer_barrier_limit_us(0) == 0
        status.zero_()
    assert handle.el_set_peer_barrier_limit_us(-1) == pkg._lib.EL_ERR_INVALID_ARG


def test_calls_from_two_host_threads_agree_with_one(ops):
    """The library promises re-entrancy across host threads, including the per-device set-up a launcher does on its
    first call.  Two threads, each on its own stream, run the forward and dX GEMMs and a decode call at shapes no other
    test of this file uses first; both must return what the oracle gives."""
    import threading
    M, N, K = 384, 640, 320
    Xq, dYq, Wp, ax, ay = _gemm_inputs(M, N, K, seed=4242)
    gamma = 0.019
    want_y = O.to_bf16(O.scale_rows(O.gemm_fwd_acc(Xq, Wp, K), ax, gamma))
    want_dx = O.to_bf16(O.scale_rows(O.gemm_dx_acc(dYq, Wp, K), ay, gamma))
    xs = torch.from_numpy(np.random.default_rng(1).standard_normal((5, K)).astype(np.float32)).to(torch.bfloat16)
    q5, a5 = O.quantize_rows(t2n(xs))
    want_dec = O.to_bf16(O.scale_rows(O.gemm_fwd_acc(q5, Wp, K), a5, gamma))
    Xd, Yd, Wd, axd, ayd, xsd = _cuda(Xq), _cuda(dYq), _cuda(Wp), _cuda(ax), _cuda(ay), xs.to(DEV)
    torch.cuda.synchronize()
    results, errors = [None, None], []
    gate = threading.Barrier(2)

    def worker(i):
        try:
            torch.cuda.set_device(0)
            s = torch.cuda.Stream()
            gate.wait()
            with torch.cuda.stream(s):
                y = ops.matmul_rows(Xd, Wd, axd, gamma, torch.bfloat16)
                dx = ops.backward_input_rows(Yd, Wd, ayd, gamma, K, torch.bfloat16)
                ws = torch.zeros(ops._lib.lib().el_decode_workspace_bytes(N), dtype=torch.uint8, device=DEV)
                dec = ops.linear_decode(xsd, Wd, gamma, workspace=ws)
            s.synchronize()
            results[i] = (t2n(y), t2n(dx), t2n(dec))
        except Exception as e:  # noqa: BLE001 - reported by the asserting thread
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for y, dx, dec in results:
        assert np.array_equal(y, want_y) and np.array_equal(dx, want_dx) and np.array_equal(dec, want_dec)
    ops.check_device_status(torch.device(DEV))


# ---- token-parallel layer: its exchange kernels with the ranks emulated one after the other on one GPU ---------------

@pytest.mark.parametrize("nbytes,offset", [(4, 8), (48, 16), (4096, 0), (1 << 20, 4096), (100, 4), (3 * (1 << 20) + 16, 32)])
def test_peer_put_copies_the_block_into_every_destination(ops, nbytes, offset):
    """The push half of an all-gather: one local block lands at the same byte offset of every destination buffer (16-byte
    stores when everything is aligned, 4-byte stores otherwise) and nothing around it changes."""
    src = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=DEV)
    dsts = [torch.full((offset + nbytes + 64,), 7, dtype=torch.uint8, device=DEV) for _ in range(3)]
    ops.peer_put(src, [d.data_ptr() for d in dsts], offset, max_ctas=5)
    ops.peer_put(src, [dsts[2].data_ptr()], offset)                      # default grid size
    for d in dsts:
        assert torch.equal(d[offset:offset + nbytes], src)
        assert bool((d[:offset] == 7).all()) and bool((d[offset + nbytes:] == 7).all())


@pytest.mark.parametrize("nbytes,offset", [(4096, 0), (70001, 13), (3 << 20, 4096)])
def test_peer_put_through_the_copy_engines(ops, nbytes, offset):
    """The same push as one copy-engine copy per destination (max_ctas < 0): any size and alignment, the same bytes in
    every destination, nothing around them touched; ordered with kernels of the stream (the source is written by a
    kernel queued just before, and a kernel queued after reads the destinations)."""
    src = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    dsts = [torch.full((offset + nbytes + 64,), 7, dtype=torch.uint8, device=DEV) for _ in range(3)]
    src.copy_(torch.arange(nbytes, device=DEV, dtype=torch.int64).remainder(251).to(torch.uint8))
    ops.peer_put(src, [d.data_ptr() for d in dsts], offset, max_ctas=-1)
    sums = [int(d[offset:offset + nbytes].to(torch.int64).sum().item()) for d in dsts]
    want = int(src.to(torch.int64).sum().item())
    for d, s_ in zip(dsts, sums):
        assert s_ == want and torch.equal(d[offset:offset + nbytes], src)
        assert bool((d[:offset] == 7).all()) and bool((d[offset + nbytes:] == 7).all())


def test_peer_put_rejects_misaligned_blocks(ops, pkg):
    src = torch.zeros(64, dtype=torch.uint8, device=DEV)
    dst = torch.zeros(64, dtype=torch.uint8, device=DEV)
    for args in ((src[1:9], [dst.data_ptr()], 0), (src[:8], [dst.data_ptr()], 2), (src[:6], [dst.data_ptr()], 0)):
        with pytest.raises(pkg.ElleciError) as e:
            ops.peer_put(*args)
        assert e.value.status == pkg._lib.EL_ERR_ALIGNMENT


@pytest.mark.parametrize("g,Ml,K,N,thr", [(2, 128, 256, 512, 2), (4, 64, 128, 256, 3), (8, 96, 256, 1024, 2)])
def test_token_parallel_update_of_all_ranks_equals_the_single_gpu_update(ops, g, Ml, K, N, thr):
    """The weight update of a token-parallel layer, its g ranks emulated one after the other on one device with local
    buffers standing in for the peers': every rank quantises its own tokens into its row block of the gathered token
    buffers, leaves its partial gradient maximum in its slot, scatters the column windows of its quantised gradient to
    the owners (el_quantize_grad_scatter), and every owner runs the fused weight-gradient + hysteresis kernel on its rows
    of a replica.  The assembled weights and counters must equal the single-GPU update over all g*Ml tokens bit for bit,
    and so must the intermediate integers against the oracle."""
    M = g * Ml
    d = make_layer_inputs(M, K, N, seed=g + Ml, dtype=torch.bfloat16, dy_std=1e-2, counters=thr)
    x, dY = d["x"].to(DEV), d["dY"].to(DEV)
    Nl = N // g
    lr, lr_scale, decay, step = 0.5, 5.0, 0.001, 3
    # single-GPU update
    Xq1, ax1 = ops.quantize_rows(x)
    _, _, gmax1 = ops.quantize_rows(dY, ops.GRAD_EPS, fold_absmax=ax1)
    Gq1 = ops.quantize_grad(dY, ax1, gmax1)
    W1, H1 = _cuda(d["Wp"]), _cuda(d["Hp"])
    ops.dw_hysteresis(Gq1, Xq1, gmax1, W1, H1, lr, lr_scale, thr, decay, step)
    # emulated ranks
    xq_all = [torch.zeros(M, K, dtype=torch.int8, device=DEV) for _ in range(g)]           # every rank's gathered tokens
    gq_recv = [torch.full((M, Nl), 99, dtype=torch.int8, device=DEV) for _ in range(g)]    # owner d: [source rank * Ml + token, window]
    slots = [torch.zeros(8, dtype=torch.float32, device=DEV) for _ in range(g)]
    axs = []
    for r in range(g):
        rows = slice(r * Ml, (r + 1) * Ml)
        own = xq_all[r][rows]
        _, ax = ops.quantize_rows(x[rows], out=own)
        ops.peer_put(own, [xq_all[p].data_ptr() for p in range(g) if p != r], r * Ml * K)
        _, _, gloc = ops.quantize_rows(dY[rows], ops.GRAD_EPS, fold_absmax=ax)
        ops.peer_put(gloc, [s.data_ptr() for s in slots], 4 * r)
        axs.append(ax)
    gmaxes = []
    for r in range(g):
        rows = slice(r * Ml, (r + 1) * Ml)
        gmax = torch.zeros(1, dtype=torch.float32, device=DEV)
        ops.quantize_grad_scatter(dY[rows], axs[r], slots[r][:g], [b.data_ptr() for b in gq_recv], r * Ml, gmax)
        gmaxes.append(gmax)
    Wr = [_cuda(d["Wp"]) for _ in range(g)]                                                # one replica per rank
    Hr = [_cuda(d["Hp"][r * Nl:(r + 1) * Nl]) for r in range(g)]
    for r in range(g):
        own_rows = Wr[r][r * Nl:(r + 1) * Nl]
        ops.dw_hysteresis(gq_recv[r], xq_all[r], gmaxes[r], own_rows, Hr[r], lr, lr_scale, thr, decay, step, idx_base=r * Nl * K)
        ops.peer_put(own_rows, [Wr[p].data_ptr() for p in range(g) if p != r], r * Nl * (K // 4))
    ops.check_device_status(torch.device(DEV))
    for r in range(g):
        assert torch.equal(xq_all[r], Xq1), r
        assert float(gmaxes[r].item()) == float(gmax1.item())
        assert torch.equal(gq_recv[r], Gq1[:, r * Nl:(r + 1) * Nl].contiguous()), r
        assert torch.equal(Wr[r], W1), r
        assert torch.equal(Hr[r], H1[r * Nl:(r + 1) * Nl]), r
    # the intermediate integers against the oracle
    xq_o, ax_o = O.quantize_rows(t2n(d["x"]))
    assert np.array_equal(Xq1.cpu().numpy(), xq_o)
    Gq_o, g_o = O.grad_quantize(t2n(d["dY"]), ax_o)
    assert np.array_equal(Gq1.cpu().numpy(), Gq_o) and np.float32(gmax1.item()) == g_o
    assert not torch.equal(W1.cpu(), torch.from_numpy(d["Wp"]))


# ---- split reduction of GEMMs with few output tiles ---------------------------------------------------------------------

@pytest.mark.parametrize("M,N,K", [(512, 4096, 11008), (512, 11008, 4096), (256, 512, 8192), (300, 520, 8192), (1024, 8192, 1024)])
def test_split_reduction_gemms_equal_the_unsplit_ones(ops, pkg, M, N, K):
    """Shapes with at most 37 output tiles (forward, dX or both) run with their reduction cut into parts on otherwise
    idle CTA pairs, the int32 partial sums added by a second kernel: the outputs must equal the oracle's and the unsplit
    kernel's bit for bit (bf16 and float32), also for ragged edges and per-tensor scales."""
    lib = pkg._lib.lib()
    Xq, dYq, Wp, ax, ay = _gemm_inputs(M, N, K, seed=M + N)
    gamma = 0.0173
    assert lib.el_gemm_workspace_bytes(0, M, N, K) > 0 or lib.el_gemm_workspace_bytes(1, M, N, K) > 0
    dXq, ddY, dWp, dax, day = _cuda(Xq), _cuda(dYq), _cuda(Wp), _cuda(ax), _cuda(ay)
    acc_f, acc_x = O.gemm_fwd_acc(Xq, Wp, K), O.gemm_dx_acc(dYq, Wp, K)
    for dt, rnd in ((torch.float32, lambda v: v), (torch.bfloat16, O.to_bf16)):
        y = ops.matmul_rows(dXq, dWp, dax, gamma, dt)
        assert np.array_equal(t2n(y), rnd(O.scale_rows(acc_f, ax, gamma)))
        dx = ops.backward_input_rows(ddY, dWp, day, gamma, K, dt)
        assert np.array_equal(t2n(dx), rnd(O.scale_rows(acc_x, ay, gamma)))
        # the same calls without a workspace run unsplit
        y0 = torch.empty_like(y)
        dx0 = torch.empty_like(dx)
        st = ops.device_status(torch.device(DEV))
        cs = torch.cuda.current_stream().cuda_stream
        edt = pkg._lib.EL_F32 if dt == torch.float32 else pkg._lib.EL_BF16
        pkg._lib.call("el_gemm_fwd", dXq.data_ptr(), dWp.data_ptr(), y0.data_ptr(), edt, dax.data_ptr(), 1, gamma, M, N, K, 0,
                      st.data_ptr(), cs)
        pkg._lib.call("el_gemm_dx", ddY.data_ptr(), dWp.data_ptr(), dx0.data_ptr(), edt, day.data_ptr(), 1, gamma, M, N, K, 0,
                      st.data_ptr(), cs)
        assert torch.equal(y, y0) and torch.equal(dx, dx0)
    s1 = torch.tensor([2.5], device=DEV)
    yt = ops.matmul_int8(dXq, dWp, s1, gamma)
    assert np.array_equal(t2n(yt), O.to_f16(O.scale_rows(acc_f, np.float32(2.5), gamma)))
    ops.check_device_status(torch.device(DEV))


def test_split_reduction_is_chosen_for_the_shapes_it_is_meant_for(pkg):
    lib = pkg._lib.lib()
    assert lib.el_gemm_workspace_bytes(0, 4096, 512, 4096) == 0                            # 32 tiles but only 32 reduction blocks
    assert lib.el_gemm_workspace_bytes(0, 4096, 11008, 4096) == 0                          # 688 tiles: no split
    assert lib.el_gemm_workspace_bytes(1, 512, 11008, 4096) == 2 * 512 * 4096 * 4         # dX of 512 tokens: 32 tiles, 86 blocks
    assert lib.el_gemm_workspace_bytes(0, 512, 4096, 11008) == 2 * 512 * 4096 * 4         # 86 reduction blocks = 2 x 43
    assert lib.el_gemm_workspace_bytes(0, 256, 256, 8192) == 4 * 256 * 256 * 4            # one tile, 64 blocks: four parts of 16
    assert lib.el_gemm_workspace_bytes(0, 0, 64, 64) == 0 and lib.el_gemm_workspace_bytes(7, 64, 64, 64) == 0


@pytest.mark.parametrize("M,N,K", [(600, 2000, 2048), (2304, 2304, 2048), (512, 4096, 11008)])
def test_register_lean_pair_kernels_bit_exact(ops, pkg, M, N, K):
    """EL_FLAG_LEAN selects the form of the CTA-pair kernels that leaves register-file room for a co-resident push kernel:
    same integers, same rounding (also through the split reduction)."""
    Xq, dYq, Wp, ax, ay = _gemm_inputs(M, N, K, seed=7 + M)
    gamma = 0.0173
    path = pkg._lib.EL_PATH_TC | pkg._lib.EL_FLAG_LEAN
    dXq, ddY, dWp, dax, day = _cuda(Xq), _cuda(dYq), _cuda(Wp), _cuda(ax), _cuda(ay)
    acc_f, acc_x = O.gemm_fwd_acc(Xq, Wp, K), O.gemm_dx_acc(dYq, Wp, K)
    assert np.array_equal(ops.matmul_rows(dXq, dWp, dax, gamma, torch.int32, path).cpu().numpy(), acc_f)
    assert np.array_equal(ops.backward_input_rows(ddY, dWp, day, gamma, K, torch.int32, path).cpu().numpy(), acc_x)
    assert np.array_equal(t2n(ops.matmul_rows(dXq, dWp, dax, gamma, torch.bfloat16, path)), O.to_bf16(O.scale_rows(acc_f, ax, gamma)))
    assert np.array_equal(t2n(ops.backward_input_rows(ddY, dWp, day, gamma, K, torch.bfloat16, path)),
                          O.to_bf16(O.scale_rows(acc_x, ay, gamma)))
    ops.check_device_status(torch.device(DEV))


def test_barrier_and_weight_update_replayed_from_a_cuda_graph(ops, pkg):
    """What a recorded training step needs: a barrier whose number comes from the flag array and a weight update whose
    step number comes from a device counter.  One rank on one device: three replays of a graph holding
    [barrier_next + word, counter_add, dW + hysteresis with the step pointer] must leave the flag at the right epoch,
    mix with an explicitly numbered barrier, and update the weights exactly as three ordinary calls with steps 6, 7, 8."""
    dev = torch.device(DEV)
    M, N, K = 256, 128, 128
    g = torch.Generator().manual_seed(77)
    Gq = torch.randint(-127, 128, (M, N), generator=g, dtype=torch.int8).to(DEV)
    Xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(DEV)
    gmax = torch.tensor([3.0e-3], dtype=torch.float32, device=DEV)
    Wp, _ = random_packed(N, K, seed=9)
    W_ref, W_rec = _cuda(Wp).clone(), _cuda(Wp).clone()
    H_ref = torch.zeros(N, K // 2, dtype=torch.uint8, device=DEV)
    H_rec = H_ref.clone()
    for step in (6, 7, 8):
        ops.dw_hysteresis(Gq, Xq, gmax, W_ref, H_ref, 0.8, 5.0, 2, 0.01, step, 64)
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    slots = torch.zeros(8, dtype=torch.float32, device=DEV)
    word = torch.tensor([1.5], dtype=torch.float32, device=DEV)
    counter = torch.tensor([5], dtype=torch.int32, device=DEV)
    ops.peer_barrier([flags.data_ptr()], 0, 1, dev)                  # explicit epochs 1 and 2 first
    ops.peer_barrier([flags.data_ptr()], 0, 2, dev)
    ops.peer_barrier_next([flags.data_ptr()], 0, dev)                # 3, queued directly
    torch.cuda.synchronize()
    assert flags[0].item() == 3
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.peer_barrier_next([flags.data_ptr()], 0, dev, word, [slots.data_ptr()], 4 * 2)
        ops.counter_add(counter, 1)
        ops.dw_hysteresis(Gq, Xq, gmax, W_rec, H_rec, 0.8, 5.0, 2, 0.01, counter, 64)
    torch.cuda.synchronize()
    assert flags[0].item() == 3 and counter.item() == 5 and torch.equal(W_rec, _cuda(Wp))     # recording ran nothing
    for i in range(3):
        word.fill_(2.0 + i)
        graph.replay()
    torch.cuda.synchronize()
    assert flags[0].item() == 6 and counter.item() == 8 and slots[2].item() == 4.0
    assert torch.equal(W_rec, W_ref) and torch.equal(H_rec, H_ref)
    assert not torch.equal(W_rec, _cuda(Wp))
    ops.peer_barrier([flags.data_ptr()], 0, 7, dev)                  # the host kept counting: explicit 7, then next = 8
    ops.peer_barrier_next([flags.data_ptr()], 0, dev)
    torch.cuda.synchronize()
    assert flags[0].item() == 8
    ops.check_device_status(dev)
