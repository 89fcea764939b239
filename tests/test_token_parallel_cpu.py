"""The token-parallel layer's host logic on CPU ranks (gloo, world size 2 and 4): which rank quantises which tokens,
the exchange of int8 tokens / partial maxima / gradient windows / updated weight rows, the row ownership and the
random-number indexing, with the CPU oracle standing in for the CUDA operators.  Several consecutive steps must
reproduce the single-rank layer bit for bit: every rank's output and input-gradient rows, every replica of the packed
weights, and the owner's counters."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_package
from helpers import make_layer_inputs

HERE = os.path.dirname(os.path.abspath(__file__))
M, K, N, STEPS = 48, 64, 96, 3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs():
    d = make_layer_inputs(M, K, N, seed=5, dtype=torch.float32, dy_std=1e-2, counters=1)
    g = torch.Generator().manual_seed(99)
    xs = [d["x"]] + [torch.randn(M, K, generator=g) for _ in range(STEPS - 1)]
    dys = [d["dY"]] + [torch.randn(M, N, generator=g) * 1e-2 for _ in range(STEPS - 1)]
    return d, xs, dys


def _single_rank(pkg, order):
    import oracle_ops
    d, xs, dys = _inputs()
    layer = pkg.token_parallel.TokenParallelInt2Linear(K, N, threshold=2, hysteresis_order=order, ops=oracle_ops)
    layer.load_full(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
    layer.set_lr(0.5)
    ys, dxs = [], []
    for x, dy in zip(xs, dys):
        x = x.clone().requires_grad_(True)
        y = layer.train()(x)
        y.backward(dy)
        ys.append(y.detach())
        dxs.append(x.grad.detach())
    return ys, dxs, layer.W_packed.clone(), layer.H_packed.clone(), layer.state_dict()


def _worker(rank, world, port, order, out_dir):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle_ops
        pkg = load_package()
        d, xs, dys = _inputs()
        layer = pkg.token_parallel.TokenParallelInt2Linear(K, N, threshold=2, hysteresis_order=order, ops=oracle_ops)
        assert (layer.row_start, layer.row_stop) == (rank * N // world, (rank + 1) * N // world)
        layer.load_full(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
        layer.set_lr(0.5)
        Ml = M // world
        ys, dxs = [], []
        for i, (x, dy) in enumerate(zip(xs, dys)):
            if i == STEPS - 1:
                # a checkpoint in the middle of training: a fresh layer restored from state_dict() continues bit for bit
                fresh = pkg.token_parallel.TokenParallelInt2Linear(K, N, threshold=2, hysteresis_order=order, ops=oracle_ops)
                fresh.load_state_dict(layer.state_dict())
                fresh.set_lr(0.5)
                assert fresh._step_py == STEPS - 1
                layer = fresh
            xl = x[rank * Ml:(rank + 1) * Ml].clone().requires_grad_(True)         # this rank's tokens
            y = layer.train()(xl)
            y.backward(dy[rank * Ml:(rank + 1) * Ml])
            ys.append(y.detach())
            dxs.append(xl.grad.detach())
        torch.save({"ys": ys, "dxs": dxs, "W": layer.W_packed, "H": layer.H_packed, "rows": (layer.row_start, layer.row_stop),
                    "step": int(layer._step.item())}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("order", ["reference", "after_dx"])
def test_token_parallel_steps_equal_single_rank(tmp_path, world, order):
    pkg = load_package()
    sys.path.insert(0, HERE)
    ys1, dxs1, W1, H1, _ = _single_rank(pkg, order)
    d, _, _ = _inputs()
    assert not torch.equal(W1, torch.from_numpy(d["Wp"]))          # the steps flip weights
    mp.spawn(_worker, args=(world, _free_port(), order, str(tmp_path)), nprocs=world, join=True)
    Ml = M // world
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        a, b = res["rows"]
        for i in range(STEPS):
            assert torch.equal(res["ys"][i], ys1[i][r * Ml:(r + 1) * Ml]), (r, i)        # token rows of the output
            assert torch.equal(res["dxs"][i], dxs1[i][r * Ml:(r + 1) * Ml]), (r, i)      # and of the input gradient
        assert torch.equal(res["W"], W1)                           # every replica holds all updated rows
        assert torch.equal(res["H"], H1[a:b])                      # the owner's counters
        assert res["step"] == STEPS


def test_token_parallel_single_rank_equals_the_n_sharded_single_rank_layer():
    """With one rank both partitions are the plain layer: same outputs, gradients and state."""
    pkg = load_package()
    sys.path.insert(0, HERE)
    import oracle_ops
    d, xs, dys = _inputs()
    ys1, dxs1, W1, H1, _ = _single_rank(pkg, "reference")
    ref = pkg.sharded.ShardedInt2Linear(K, N, threshold=2, hysteresis_order="reference", ops=oracle_ops)
    ref.load_shard(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
    ref.set_lr(0.5)
    for i, (x, dy) in enumerate(zip(xs, dys)):
        x = x.clone().requires_grad_(True)
        y = ref.train()(x)
        y.backward(dy)
        assert torch.equal(y.detach(), ys1[i]) and torch.equal(x.grad, dxs1[i])
    assert torch.equal(ref.W_packed, W1) and torch.equal(ref.H_packed, H1)
    assert int(ref._step.item()) == STEPS


def test_push_policy_and_peer_order():
    """Host-side choices of the fused path that need no GPU: the peers are listed from the rank's successor on (so that
    copy-engine pushes of all ranks never meet at one destination), pushes of 8 MiB and more per destination go through
    the copy engines, smaller ones through the peer-store kernel with one CTA per SM, and the register-lean GEMM form is
    only chosen beside a push kernel, from four ranks on."""
    import oracle_ops
    pkg = load_package()
    tp = pkg.token_parallel
    layer = tp.TokenParallelInt2Linear(4096, 11008, threshold=2, ops=oracle_ops)
    layer.world, layer.rank = 8, 5
    assert layer._successors(list("abcdefgh")) == list("ghabcde")
    # every rank r sends to (r + j) mod g at position j: at a given position all destinations differ
    for j in range(1, 8):
        dests = set()
        for r in range(8):
            layer.rank = r
            dests.add(layer._successors(list(range(8)))[j - 1])
        assert dests == set(range(8))
    assert layer._push_mode(tp.PUSH_DMA_MIN_BYTES) < 0 and layer._push_mode(tp.PUSH_DMA_MIN_BYTES - 1) == 148
    layer.push_ctas = 37
    assert layer._push_mode(1) == 37 and layer._push_mode(1 << 30) == 37
    layer.push_ctas = -1
    assert layer._push_mode(1) < 0
    layer.push_ctas, layer._lean = 0, 0x100
    assert layer._gemm_flags(512) == 0x100            # 512 x 4096 = 2 MiB per destination: kernel push, lean GEMM beside it
    assert layer._gemm_flags(8192) == 0               # 32 MiB: copy engines, the GEMM keeps its faster form
