"""The decode entry point that allocates nothing (el_linear_decode_static), called through the C ABI.

Some hosts cannot give the library device memory at call time: a serving process that bans cudaMalloc once it is
live, a runtime that owns the whole memory pool, a job already at its memory budget.  For them the library keeps the
scratch of the small-M decode call in a static device array.  This test checks that the variant returns exactly what
the regular entry point (el_linear_decode, caller-owned scratch) returns, on two calls in a row that share the array,
and that sizes beyond the array's capacity are refused.  It is collected last so that a failure here cannot hide
another test's result; it passes on its own in a fresh process as well as after the rest of the suite."""
import numpy as np
import pytest
import torch

from oracle import int2_oracle as O

from helpers import random_packed, t2n

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _regular(pkg, x, W, gamma, out_dtype):
    """el_linear_decode through the C ABI, with scratch owned by this test."""
    lib = pkg._lib
    M, K = x.shape
    N = W.shape[0]
    ws = torch.zeros(lib.lib().el_decode_workspace_bytes(N), dtype=torch.uint8, device=DEV)
    xq = torch.empty(M, K, dtype=torch.int8, device=DEV)
    a = torch.empty(M, dtype=torch.float32, device=DEV)
    y = torch.empty(M, N, dtype=out_dtype, device=DEV)
    dt = {torch.bfloat16: lib.EL_BF16, torch.float16: lib.EL_F16, torch.float32: lib.EL_F32}
    lib.call("el_linear_decode", x.data_ptr(), dt[x.dtype], W.data_ptr(), y.data_ptr(), dt[out_dtype], gamma, xq.data_ptr(),
             a.data_ptr(), ws.data_ptr(), ws.numel(), M, N, K, None, torch.cuda.current_stream().cuda_stream)
    return y


def _static(pkg, x, W, gamma, out_dtype):
    """el_linear_decode_static through the C ABI: inputs and the output buffer only."""
    lib = pkg._lib
    M, K = x.shape
    N = W.shape[0]
    y = torch.empty(M, N, dtype=out_dtype, device=DEV)
    dt = {torch.bfloat16: lib.EL_BF16, torch.float16: lib.EL_F16, torch.float32: lib.EL_F32}
    lib.call("el_linear_decode_static", x.data_ptr(), dt[x.dtype], W.data_ptr(), y.data_ptr(), dt[out_dtype], gamma, M, N, K,
             None, torch.cuda.current_stream().cuda_stream)
    return y


def test_static_scratch_decode_matches_regular_entry_point_twice_in_a_row(pkg):
    cases = [(8, 4096, 11008, torch.bfloat16), (33, 1024, 640, torch.float32), (1, 11008, 4096, torch.bfloat16)]
    for M, K, N, out_dtype in cases:
        g = torch.Generator().manual_seed(M + K + N)
        Wp, _ = random_packed(N, K, seed=N)
        W = torch.from_numpy(Wp).to(DEV)
        x1 = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        x2 = (torch.randn(M, K, generator=g) * 3.0).to(torch.bfloat16).to(DEV)
        # two calls in a row on the shared array, different inputs; bit-exact against the regular entry point
        y1 = _static(pkg, x1, W, 0.017, out_dtype)
        y2 = _static(pkg, x2, W, 0.017, out_dtype)
        torch.cuda.synchronize()
        r1 = _regular(pkg, x1, W, 0.017, out_dtype)
        r2 = _regular(pkg, x2, W, 0.017, out_dtype)
        torch.cuda.synchronize()
        assert torch.equal(y1, r1) and torch.equal(y2, r2)
        assert not torch.equal(y1, y2) and float(y1.float().abs().max()) > 0.0


@pytest.mark.parametrize("mma_max", [64, 0])
def test_static_scratch_is_really_used_and_shared_between_shapes(pkg, mma_max):
    """Calls that need the array (more than 8 tokens): the stated capacity M=64 at N=16384, a 40-token call, then a
    small-N call whose tile counters sit where the large call kept partial sums, then the large one again, then tokens
    that do not fit in shared memory.  With the default limits the quantised tokens and their scales live in the array
    and the warp-MMA kernel reads them (the last case takes the tcgen05 kernel and its partial-sum area); with the
    warp-MMA kernel switched off (`mma_max` 0) every case takes the tcgen05 kernel.  The first call of the sequence is
    a one-token call, which touches no scratch but must already have resolved the array's address.  Every result is
    checked against the regular entry point and against the CPU oracle."""
    assert pkg._lib.lib().el_set_decode_mma_max_tokens(mma_max) == 0
    try:
        _static_sequence(pkg)
    finally:
        assert pkg._lib.lib().el_set_decode_mma_max_tokens(64) == 0


def _static_sequence(pkg):
    gamma = 0.0157
    seq = [(1, 4096, 16384), (64, 4096, 16384), (33, 1024, 640), (40, 4096, 16384), (48, 256, 128), (64, 4096, 16384),
           (40, 11008, 512)]
    weights = {}
    for i, (M, K, N) in enumerate(seq):
        if (K, N) not in weights:
            Wp, _ = random_packed(N, K, seed=K + N)
            weights[(K, N)] = (Wp, torch.from_numpy(Wp).to(DEV))
        Wp, W = weights[(K, N)]
        x = (torch.randn(M, K, generator=torch.Generator().manual_seed(100 + i)) * (1.0 + i)).to(torch.bfloat16)
        xd = x.to(DEV)
        y = _static(pkg, xd, W, gamma, torch.bfloat16)
        r = _regular(pkg, xd, W, gamma, torch.bfloat16)
        torch.cuda.synchronize()
        Xq, ax = O.quantize_rows(t2n(x))
        want = O.to_bf16(O.scale_rows(O.gemm_fwd_acc(Xq, Wp, K), ax, gamma))
        assert torch.equal(y, r), (M, K, N)
        assert np.array_equal(t2n(y), want), (M, K, N)
    pkg.int2_tc_ops.check_device_status(torch.device(DEV))


def test_static_scratch_decode_refuses_sizes_beyond_its_capacity(pkg):
    lib = pkg._lib
    x = torch.zeros(1, 64, dtype=torch.bfloat16, device=DEV)
    W = torch.zeros(4, 16, dtype=torch.uint8, device=DEV)
    y = torch.zeros(1, 4, dtype=torch.bfloat16, device=DEV)
    handle = lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    for M, N, K in [(65, 128, 128), (1, 16385, 128), (1, 128, 16448)]:
        rc = handle.el_linear_decode_static(x.data_ptr(), lib.EL_BF16, W.data_ptr(), y.data_ptr(), lib.EL_BF16, 1.0, M, N, K,
                                            None, st)
        assert rc == lib.EL_ERR_TOO_LARGE
        assert b"capacity" in handle.el_status_string(rc)
    with pytest.raises(pkg.ElleciError):
        pkg.int2_tc_ops.linear_decode_static(torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV), W,
                                             1.0, torch.zeros(65, 4, dtype=torch.bfloat16, device=DEV))
