"""Parity at the benchmark's full sizes (M = 4096 with 4096 <-> 11008, and M = 65536 with 4096 -> 16384), where a CPU
oracle of the whole result would take minutes.  Three size-independent checks stand in for it:
  * checksums over the whole result: for the integer GEMMs, the sum of every output row and of every output column
    must equal what the linearity of the product predicts from the sums of the operands (computed independently, in
    float64 / int64, never with the kernels under test) - an error in any tile changes one of them;
  * exact comparison with the oracle on sampled rows (GEMMs) and on sampled contiguous blocks of weight rows (the fused
    weight-gradient + hysteresis update, whose per-weight random numbers depend on the global weight index);
  * invariants of the packed state after an update (counters within the threshold, codes valid, a plausible share of
    flips).
The quantisers are compared with the oracle in full (NumPy handles 45 M elements in a second)."""
import numpy as np
import pytest
import torch

from oracle import int2_oracle as O
from oracle import native

from helpers import t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"

SIZES = [pytest.param(4096, 4096, 11008, id="config2-4096x11008"), pytest.param(4096, 11008, 4096, id="config2-11008x4096"),
         pytest.param(65536, 4096, 16384, id="config4-65536x4096x16384")]


@pytest.fixture(scope="module")
def ops(pkg):
    return pkg.int2_tc_ops


def _ternary_packed(N, K, seed):
    """Packed ternary weights with about one third zeros, generated on the GPU; returns (packed uint8 on the GPU,
    the int8 values on the GPU)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = torch.randint(-1, 2, (N, K), generator=g, device=DEV, dtype=torch.int8)
    c = (w + 1).to(torch.uint8).view(N, K // 4, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).contiguous(), w


def _rows(M, n, seed):
    rng = np.random.default_rng(seed)
    return np.sort(np.concatenate([[0, M - 1], rng.choice(np.arange(1, M - 1), n - 2, replace=False)]))


@pytest.mark.parametrize("M,K,N", SIZES)
def test_forward_and_dx_gemms_at_full_size(ops, M, K, N):
    g = torch.Generator(device=DEV).manual_seed(M + K)
    Wp, w = _ternary_packed(N, K, 7)
    ones = torch.ones(M, device=DEV)
    # ---- forward: acc[m,n] = sum_k Xq[m,k] * w[n,k]
    Xq = torch.randint(-128, 128, (M, K), generator=g, device=DEV, dtype=torch.int8)
    acc = ops.matmul_rows(Xq, Wp, ones, 1.0, torch.int32)
    ops.check_device_status(torch.device(DEV))
    w_col_sum = w.to(torch.float64).sum(0)                         # [K]: sum over n
    x_col_sum = Xq.to(torch.float64).sum(0)                        # [K]: sum over m
    assert torch.equal(acc.sum(1, dtype=torch.int64), (Xq.to(torch.float64) @ w_col_sum).to(torch.int64))      # row checksums
    assert torch.equal(acc.sum(0, dtype=torch.int64), (w.to(torch.float64) @ x_col_sum).to(torch.int64))       # column checksums
    rows = _rows(M, 48, 1)
    want = O.gemm_fwd_acc(Xq[rows].cpu().numpy(), Wp.cpu().numpy(), K)
    assert np.array_equal(acc[rows].cpu().numpy(), want)
    # the scaled bf16 output on the sampled rows: the oracle's float32 epilogue
    ax = (torch.rand(M, generator=g, device=DEV) * 4 + 0.5)
    y = ops.matmul_rows(Xq, Wp, ax, 0.0173, torch.bfloat16)
    assert np.array_equal(t2n(y[rows]), O.to_bf16(O.scale_rows(want, ax[rows].cpu().numpy(), 0.0173)))
    del acc, y, Xq
    # ---- dX: acc[m,k] = sum_n dYq[m,n] * w[n,k]
    dYq = torch.randint(-128, 128, (M, N), generator=g, device=DEV, dtype=torch.int8)
    acc = ops.backward_input_rows(dYq, Wp, ones, 1.0, K, torch.int32)
    ops.check_device_status(torch.device(DEV))
    w_row_sum = w.to(torch.float64).sum(1)                         # [N]: sum over k
    dy_col_sum = dYq.to(torch.float64).sum(0)                      # [N]: sum over m
    assert torch.equal(acc.sum(1, dtype=torch.int64), (dYq.to(torch.float64) @ w_row_sum).to(torch.int64))
    assert torch.equal(acc.sum(0, dtype=torch.int64), (dy_col_sum @ w.to(torch.float64)).to(torch.int64))
    want = O.gemm_dx_acc(dYq[rows].cpu().numpy(), Wp.cpu().numpy(), K)
    assert np.array_equal(acc[rows].cpu().numpy(), want)


@pytest.mark.parametrize("M,K,N", SIZES)
def test_fused_weight_update_at_full_size(ops, M, K, N):
    """The fused dW + hysteresis kernel on the whole layer; the oracle re-computes sampled blocks of 16 weight rows (their
    int32 sums from the same int8 operands, then the C restatement of the update with the block's global index base)."""
    thr, lr, step = 3, 1e-2, 5
    g = torch.Generator(device=DEV).manual_seed(N + 3)
    Wp, w = _ternary_packed(N, K, 11)
    h = torch.randint(-3, 4, (N, K), generator=g, device=DEV, dtype=torch.int16)
    Hp = ((h[:, 0::2] & 0xF) | ((h[:, 1::2] & 0xF) << 4)).to(torch.uint8).contiguous()
    Gq = torch.randint(-127, 128, (M, N), generator=g, device=DEV, dtype=torch.int8)
    Xq = torch.randint(-128, 128, (M, K), generator=g, device=DEV, dtype=torch.int8)
    gmax = np.float32(2e-4 * 4096 / M)               # puts |dW * lr * lr_scale * thr| around 1: about a fifth of the weights flip
    Wp0, Hp0 = Wp.clone(), Hp.clone()
    ops.dw_hysteresis(Gq, Xq, torch.tensor([gmax], device=DEV), Wp, Hp, lr, 5.0, thr, 0.001, step)
    ops.check_device_status(torch.device(DEV))
    rng = np.random.default_rng(N)
    Xd = Xq.to(torch.float64)
    for n0 in [0, N - 16] + [int(v) * 16 for v in rng.choice(N // 16 - 2, 6, replace=False) + 1]:
        acc = (Gq[:, n0:n0 + 16].to(torch.float64).t() @ Xd).cpu().numpy()       # exact: |acc| < 2^31
        dW = O.dw_from_acc(acc.astype(np.int64).astype(np.int32), gmax)
        Wo, Ho = native.c_hysteresis_step(dW, Wp0[n0:n0 + 16].cpu().numpy(), Hp0[n0:n0 + 16].cpu().numpy(), lr, 5.0, thr, 0.001,
                                          step, K, idx_base=n0 * K)
        assert np.array_equal(Wp[n0:n0 + 16].cpu().numpy(), Wo), n0
        assert np.array_equal(Hp[n0:n0 + 16].cpu().numpy(), Ho), n0
    # invariants of the whole packed state
    codes = torch.stack([(Wp >> s) & 3 for s in (0, 2, 4, 6)], dim=-1).view(N, K)
    assert int((codes == 3).sum()) == 0
    lo, hi = (Hp & 0xF).to(torch.int16), (Hp >> 4).to(torch.int16)
    cnt = torch.stack([lo, hi], dim=-1).view(N, K)
    cnt = torch.where(cnt > 7, cnt - 16, cnt)
    assert int(cnt.abs().max()) <= thr
    flipped = float((codes.to(torch.int8) - 1 != w).float().mean())
    assert 0.05 < flipped < 0.6, flipped


@pytest.mark.parametrize("M,K", [pytest.param(4096, 4096, id="4096x4096"), pytest.param(4096, 11008, id="4096x11008")])
def test_quantisers_at_full_size(ops, M, K):
    """Per-token quantiser (with the fold for the gradient scale) and gradient quantiser against the oracle, every
    element."""
    g = torch.Generator().manual_seed(K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    dY = (torch.randn(M, K, generator=g) * 1e-3).to(torch.bfloat16)
    q, a = ops.quantize_rows(x.to(DEV))
    qo, ao = O.quantize_rows(t2n(x))
    assert np.array_equal(q.cpu().numpy(), qo) and np.array_equal(a.cpu().numpy(), ao)
    dq, da, gmax = ops.quantize_rows(dY.to(DEV), ops.GRAD_EPS, a)
    dqo, dao = O.quantize_rows(t2n(dY), eps=O.GRAD_ABSMAX_FLOOR)
    assert np.array_equal(dq.cpu().numpy(), dqo) and np.array_equal(da.cpu().numpy(), dao)
    Gq = ops.quantize_grad(dY.to(DEV), a, gmax)
    Gqo, go = O.grad_quantize(t2n(dY), ao)
    assert np.float32(gmax.item()) == np.float32(go) and np.array_equal(Gq.cpu().numpy(), Gqo)


def test_swiglu_gate_at_full_size(ops):
    """The fused SwiGLU gate of the 11008 -> 4096 down projection on 4096 tokens; tokens are independent of one another,
    so the oracle re-computes 256 sampled tokens (every int8 value of theirs).  The backward kernel on 512 of the tokens
    (the norm weight's gradient is a sum over the tokens given)."""
    M, H = 4096, 11008
    g = torch.Generator().manual_seed(31)
    gu = (torch.randn(M, 2 * H, generator=g) * 1.5).to(torch.bfloat16)
    w = (1.0 + 0.2 * torch.randn(H, generator=g)).float()
    d = gu.to(DEV)
    q, a, rstd = ops.swiglu_quantize_rows(d[:, :H], d[:, H:], w.to(DEV))
    rows = _rows(M, 256, 2)
    gate, up = t2n(gu[rows, :H]), t2n(gu[rows, H:])
    qo, ao, ro = O.swiglu_quantize_rows(gate, up, w.numpy(), 1e-6, 1e-5, "bf16")
    assert np.array_equal(rstd.cpu().numpy()[rows], ro) and np.array_equal(a.cpu().numpy()[rows], ao)
    assert np.array_equal(q.cpu().numpy()[rows], qo)
    Mb = 512
    gy = (torch.randn(Mb, H, generator=g) * 1e-2).to(torch.bfloat16)
    dg, du, dw = ops.swiglu_backward(gy.to(DEV), d[:Mb, :H], d[:Mb, H:], w.to(DEV), rstd[:Mb].contiguous())
    dgo, duo, dwo = O.swiglu_backward(t2n(gy), t2n(gu[:Mb, :H]), t2n(gu[:Mb, H:]), w.numpy(), rstd[:Mb].cpu().numpy(), "bf16")
    assert np.array_equal(t2n(dg), dgo) and np.array_equal(t2n(du), duo) and np.array_equal(dw.cpu().numpy(), dwo)
