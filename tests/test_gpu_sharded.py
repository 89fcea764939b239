"""The N-sharded layer on real GPUs (NCCL, one process per GPU): a sharded step must reproduce the single-GPU layer
step bit for bit.  Skipped on a box with one GPU (the CPU-rank test covers the host logic there)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_package
from helpers import make_layer_inputs

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
M, K, N = 512, 1024, 2048
STEPS = 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, order, out_dir, fused):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = load_package()
        d = make_layer_inputs(M, K, N, seed=3, dtype=torch.bfloat16, dy_std=1e-2, counters=1)
        layer = pkg.sharded.ShardedInt2Linear(K, N, threshold=2, hysteresis_order=order, fused_gather=bool(fused),
                                              own_barrier=(fused == "own_barrier")).to(dev)
        layer.load_shard(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
        layer.set_lr(0.5)
        x = d["x"].to(dev).requires_grad_(True)
        for _ in range(STEPS):                       # several steps: the symmetric buffers alternate between calls
            x.grad = None
            y = layer.train()(x)
            y.backward(d["dY"].to(dev))
        torch.cuda.synchronize()
        pkg.int2_tc_ops.check_device_status(dev)
        torch.save({"y": y.detach().cpu(), "dx": x.grad.cpu(), "W": layer.W_packed.cpu(), "H": layer.H_packed.cpu(),
                    "rows": (layer.row_start, layer.row_stop)}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused", [False, True, "own_barrier"])
@pytest.mark.parametrize("order", ["reference", "after_dx"])
def test_sharded_step_on_gpus_equals_single_gpu(tmp_path, order, fused):
    """fused: the output all-gather and the dX reduce-scatter happen as stores from the GEMM epilogues into symmetric
    memory, with the symmetric-memory handle's barrier between them (True) or el_peer_barrier ("own_barrier")."""
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    pkg = load_package()
    d = make_layer_inputs(M, K, N, seed=3, dtype=torch.bfloat16, dy_std=1e-2, counters=1)
    ref = pkg.Int2LinearTCWithGradHook(K, N, threshold=2, hysteresis_order=order).to("cuda:0")
    ref.W_packed.copy_(torch.from_numpy(d["Wp"]))
    ref.H_packed.copy_(torch.from_numpy(d["Hp"]))
    ref.gamma.data.fill_(d["gamma"])
    ref._gamma_cached = d["gamma"]
    ref._initialized = True
    ref.set_lr(0.5)
    x = d["x"].to("cuda:0").requires_grad_(True)
    for _ in range(STEPS):
        x.grad = None
        y = ref.train()(x)
        y.backward(d["dY"].to("cuda:0"))
    torch.cuda.synchronize()
    assert not torch.equal(ref.W_packed.cpu(), torch.from_numpy(d["Wp"]))
    mp.spawn(_worker, args=(world, _free_port(), order, str(tmp_path), fused), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        a, b = res["rows"]
        assert torch.equal(res["y"], y.detach().cpu())
        assert torch.equal(res["dx"], x.grad.cpu())
        assert torch.equal(res["W"], ref.W_packed.cpu()[a:b]) and torch.equal(res["H"], ref.H_packed.cpu()[a:b])


# ---- token-parallel layer ---------------------------------------------------------------------------------------------

def _tp_worker(rank, world, port, order, out_dir, fused):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = load_package()
        d = make_layer_inputs(M, K, N, seed=3, dtype=torch.bfloat16, dy_std=1e-2, counters=1)
        layers = []
        for li in range(2):                              # two layers share the barrier group (and each other's barriers)
            layer = pkg.token_parallel.TokenParallelInt2Linear(K, N, threshold=2, hysteresis_order=order, fused=bool(fused),
                                                               graph_steps=(fused == "graph")).to(dev)
            layer.load_full(torch.from_numpy(d["Wp"]), torch.from_numpy(d["Hp"]), d["gamma"])
            layer.set_lr(0.5 + li)
            layers.append(layer.train())
        Ml = M // world
        rows = slice(rank * Ml, (rank + 1) * Ml)
        outs = []
        for li, layer in enumerate(layers):
            x = d["x"][rows].to(dev).requires_grad_(True)
            outs.append([layer, x, None])
        dy = d["dY"][rows].to(dev)
        grads = [None, None]
        for _ in range(STEPS):
            for li, o in enumerate(outs):
                layer, x, _ = o
                if li == 0:                              # through autograd
                    x.grad = None
                    y = layer(x)
                    y.backward(dy)
                    o[2], grads[li] = y.detach(), x.grad
                else:                                    # the same step issued directly (from the prepared plan when fused)
                    o[2], grads[li] = layer.train_step(x.detach(), dy)
        for o in outs:
            o[0]._weights_ready()                        # the last pushes of updated rows have landed in this replica
        torch.cuda.synchronize()
        pkg.int2_tc_ops.check_device_status(dev)
        torch.save([{"y": y.cpu(), "dx": grads[li].cpu(), "W": layer.W_packed.cpu(), "H": layer.H_packed.cpu(),
                     "rows": (layer.row_start, layer.row_stop), "step": int(layer.state_dict()["_step"])}
                    for li, (layer, x, y) in enumerate(outs)], os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused", [False, True, "graph"])
@pytest.mark.parametrize("order", ["reference", "after_dx"])
def test_token_parallel_steps_on_gpus_equal_single_gpu(tmp_path, order, fused):
    """Every rank runs forward and dX on its own tokens against its replica of the weights and updates its own rows from
    all ranks' tokens; after the steps each rank's rows of Y and dX, every replica of W_packed and the owners' counters
    must equal the single-GPU layer's.  fused: the exchanges are the library's own peer stores and barrier.  "graph": the
    directly issued layer also replays its step from a recorded CUDA graph from the second step on (barrier numbers and
    the hysteresis step then come from device memory), next to a layer that queues its launches one by one and shares
    the barrier group with it."""
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    pkg = load_package()
    d = make_layer_inputs(M, K, N, seed=3, dtype=torch.bfloat16, dy_std=1e-2, counters=1)
    refs = []
    for li in range(2):
        ref = pkg.Int2LinearTCWithGradHook(K, N, threshold=2, hysteresis_order=order).to("cuda:0")
        ref.W_packed.copy_(torch.from_numpy(d["Wp"]))
        ref.H_packed.copy_(torch.from_numpy(d["Hp"]))
        ref.gamma.data.fill_(d["gamma"])
        ref._gamma_cached = d["gamma"]
        ref._initialized = True
        ref.set_lr(0.5 + li)
        x = d["x"].to("cuda:0").requires_grad_(True)
        for _ in range(STEPS):
            x.grad = None
            y = ref.train()(x)
            y.backward(d["dY"].to("cuda:0"))
        torch.cuda.synchronize()
        refs.append((ref, x, y))
    assert not torch.equal(refs[0][0].W_packed, refs[1][0].W_packed)       # different learning rates, different flips
    mp.spawn(_tp_worker, args=(world, _free_port(), order, str(tmp_path), fused), nprocs=world, join=True)
    Ml = M // world
    for r in range(world):
        res = torch.load(os.path.join(tmp_path, f"rank{r}.pt"))
        for li, (ref, x, y) in enumerate(refs):
            a, b = res[li]["rows"]
            assert torch.equal(res[li]["y"], y.detach().cpu()[r * Ml:(r + 1) * Ml]), (r, li)
            assert torch.equal(res[li]["dx"], x.grad.cpu()[r * Ml:(r + 1) * Ml]), (r, li)
            assert torch.equal(res[li]["W"], ref.W_packed.cpu()), (r, li)
            assert torch.equal(res[li]["H"], ref.H_packed.cpu()[a:b]), (r, li)
            assert res[li]["step"] == STEPS
