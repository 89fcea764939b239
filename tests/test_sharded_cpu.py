"""The N-sharded layer's host logic on CPU ranks (gloo, world size 2 and 4): the collectives, the shard
arithmetic and the random-number indexing, with the CPU oracle standing in for the CUDA operators.
A sharded step must reproduce the single-rank step bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_package
from helpers import make_layer_inputs

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _single_rank_step(pkg, d, K, N, order):
    import oracle_ops
    layer = pkg.sharded.ShardedInt2Linear(K, N, threshold=2, hysteresis_order=order, ops=oracle_ops)
    layer.load_shard(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
    layer.set_lr(0.5)
    x = d["x"].clone().requires_grad_(True)
    y = layer.train()(x)
    y.backward(d["dY"])
    return y.detach(), x.grad.detach(), layer.W_packed.clone(), layer.H_packed.clone()


def _worker(rank, world, port, order, out_dir):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle_ops
        pkg = load_package()
        M, K, N = 48, 64, 96
        d = make_layer_inputs(M, K, N, seed=1, dtype=torch.float32, dy_std=1e-2, counters=1)
        layer = pkg.sharded.ShardedInt2Linear(K, N, threshold=2, hysteresis_order=order, ops=oracle_ops)
        assert (layer.row_start, layer.row_stop) == (rank * N // world, (rank + 1) * N // world)
        layer.load_shard(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
        layer.set_lr(0.5)
        x = d["x"].clone().requires_grad_(True)
        y = layer.train()(x)
        y.backward(d["dY"])
        torch.save({"y": y.detach(), "dx": x.grad.detach(), "W": layer.W_packed, "H": layer.H_packed,
                    "rows": (layer.row_start, layer.row_stop)}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("order", ["reference", "after_dx"])
def test_sharded_step_equals_single_rank(tmp_path, world, order):
    pkg = load_package()
    M, K, N = 48, 64, 96
    d = make_layer_inputs(M, K, N, seed=1, dtype=torch.float32, dy_std=1e-2, counters=1)
    sys.path.insert(0, HERE)
    y1, dx1, W1, H1 = _single_rank_step(pkg, d, K, N, order)
    assert not torch.equal(W1, torch.from_numpy(d["Wp"]))          # the step flips weights
    mp.spawn(_worker, args=(world, _free_port(), order, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        a, b = res["rows"]
        assert torch.equal(res["y"], y1)                           # every rank holds the full gathered output
        assert torch.equal(res["dx"], dx1)                         # integer partial sums add exactly
        assert torch.equal(res["W"], W1[a:b]) and torch.equal(res["H"], H1[a:b])


def test_shard_rows_rejects_uneven_split():
    pkg = load_package()
    with pytest.raises(ValueError):
        pkg.sharded.shard_rows(100, 8, 0)
    assert pkg.sharded.shard_rows(11008, 8, 3) == (4128, 5504)


def test_sharded_layer_resumes_from_plain_state_dict():
    """The `_step` buffer follows the Python counter, so state_dict() -> load_state_dict() on a fresh layer continues
    with the next step's random numbers instead of replaying the first step's."""
    pkg = load_package()
    sys.path.insert(0, HERE)
    import oracle_ops
    M, K, N = 32, 64, 64
    d = make_layer_inputs(M, K, N, seed=2, dtype=torch.float32, dy_std=1e-2, counters=1)

    def make():
        layer = pkg.sharded.ShardedInt2Linear(K, N, threshold=2, ops=oracle_ops)
        layer.set_lr(0.5)
        return layer.train()

    def step(layer):
        x = d["x"].clone().requires_grad_(True)
        layer(x).backward(d["dY"])

    a = make()
    a.load_shard(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
    step(a)
    assert int(a._step.item()) == 1
    b = make()
    b.load_state_dict(a.state_dict())
    assert b._step_py == 1 and abs(b.gamma_value() - d["gamma"]) < 1e-9
    step(a)
    step(b)
    assert torch.equal(a.W_packed, b.W_packed) and torch.equal(a.H_packed, b.H_packed)
    c = make()                                   # a layer that replays step 1's random numbers ends up elsewhere
    c.load_state_dict(b.state_dict())
    c._step_py = 0
    step(c)
    step(a)
    assert not torch.equal(a.H_packed, c.H_packed)
