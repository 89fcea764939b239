"""Benchmark of the INT2 linear layer step on B200: forward + dX + dW/hysteresis tokens per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload config2|config4|config1|config3|hbm|ffn] [--partition both|tokens|features]

One "step" is one pass of the hot path over one batch of synthetic tokens: for every layer of the workload,
per-token int8 quantisation of the activations, the forward GEMM, per-token quantisation of the output gradient,
the dX GEMM, and the weight-gradient GEMM fused with the hysteresis update of the packed weights and counters.

  config2 (default)  M = 4096 tokens through the two 7B MLP projections 4096->11008 and 11008->4096,
                     counters seeded uniformly in [-3, 3], threshold 3, dY ~ N(0, 1e-3)
  config4            M = 65536 tokens through one 4096->16384 projection (also a sub-record of the default line)

With N > 1 (launched by torch.distributed.run, one rank per GPU; strong scaling: the problem is fixed) the step is
measured under two partitions of the work and `value` is the faster one, the other is reported beside it:
  tokens    every rank runs forward and dX on M/N tokens against a replica of the weights and updates 1/N of the rows
  features  the weights are sharded along their output features, activations are replicated (BASELINE config 4's wording)

Rank 0 prints one JSON line.  `value` is timed with CUDA events, inputs resident in HBM, L2 flushed between steps;
`e2e` goes through the module API with pinned host buffers copied in and results copied out every step.  The default
single-GPU line also carries: the measured int8 ceiling of the box (library GEMM), config 1 (forward sweep), config 3
(decode) and config 4 summaries, the stand-alone hysteresis kernel, the reference's own CUDA kernels timed on the same
GPU, and the CPU port timed on the host cores.  `--impl reference` times the CPU port of the reference layer
(oracle/cpu_baseline.py) alone.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "config2": dict(M=4096, layers=[(4096, 11008), (11008, 4096)], threshold=3, counters=3, dy_std=1e-3,
                    desc="config2: M=4096 tokens, layers 4096->11008 + 11008->4096, fwd + dX + dW/hysteresis"),
    "config4": dict(M=65536, layers=[(4096, 16384)], threshold=3, counters=3, dy_std=1e-3,
                    desc="config4: M=65536 tokens, layer 4096->16384, fwd + dX + dW/hysteresis"),
}
LR, LR_SCALE, DECAY = 1e-2, 5.0, 0.001
METRIC = "BitLinear fwd+bwd+hysteresis tokens/s at 7B shapes"


def load_package():
    name = "elleci_training_vast_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = os.path.join(ROOT, "elleci-training-vast_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ------------------------------------------------------------------------------------------------------------------
# clock sampling (read-only NVML queries from a thread during the timed region)
# ------------------------------------------------------------------------------------------------------------------

class ClockSampler:
    def __init__(self, device_index: int):
        self.samples, self.reasons, self.sm_max = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[device_index]) if visible and visible.split(",")[device_index].isdigit() else device_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001 - no NVML: the clocks key says so
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.004)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------------------------
# reference arm: the CPU port of the reference layer on the host cores
# ------------------------------------------------------------------------------------------------------------------

CPU_FULL_TOKENS_MAX = 8192      # workloads up to this many tokens are timed whole on the CPU; larger ones on a sample


def cpu_baseline_run(wl, steps: int, warmup: int):
    """Times the CPU port on the host cores: every step runs forward, dX, dW and the hysteresis update of every weight
    on all tokens of the workload (a 4096-token sample, scaled, only for workloads above 8192 tokens).  The warm-up
    steps alternate between bfloat16 and float32; the timed steps use the faster of the two."""
    import torch
    from oracle import cpu_baseline as cb
    from oracle import native
    native.build_oracle_lib()
    cores = cb.use_all_cores()
    M = wl["M"]
    Mt = M if M <= CPU_FULL_TOKENS_MAX else 4096
    layers = [cb.CpuLayer(K, N, seed=i, counters=wl["counters"]) for i, (K, N) in enumerate(wl["layers"])]
    dtypes = {"bf16": torch.bfloat16, "fp32": torch.float32}
    seen = {k: [] for k in dtypes}
    t_begin = time.perf_counter()
    warmup = max(warmup, 4)             # two steps per dtype at least: the first one of each pays one-time set-up
    for i in range(warmup):
        name = list(dtypes)[i % 2]
        seen[name].append(cb.time_step(layers, Mt, dtypes[name], lr=LR, threshold=wl["threshold"], seed=i, dy_std=wl["dy_std"]))
    best = min(seen, key=lambda k: min(seen[k]))
    # K steps as asked while they fit in about four minutes of CPU time
    per_step = min(seen[best])
    steps_run = max(1, min(steps, int(240.0 / max(per_step, 1e-3))))
    times = [cb.time_step(layers, Mt, dtypes[best], lr=LR, threshold=wl["threshold"], seed=100 + i, dy_std=wl["dy_std"])
             for i in range(steps_run)]
    sec = sum(times) / len(times) * (M / Mt)
    sample = (f"{steps_run} timed steps after {warmup} warm-up steps, each on "
              + (f"all {M} tokens" if Mt == M else f"{Mt} of {M} tokens, scaled by {M // Mt}")
              + f": forward + dX + dW (torch, {best}) and the hysteresis update of every weight (C, OpenMP); "
              + "warm-up best per step: " + ", ".join(f"{k} {min(v):.2f} s" for k, v in seen.items() if v))
    return {"value": M / sec, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample,
            "ms_per_step": sec * 1e3, "steps": steps_run, "warmup": warmup, "dtype": best, "extrapolated": Mt != M,
            "wall_seconds": time.perf_counter() - t_begin}


def run_reference(args, wl):
    if int(os.environ.get("RANK", "0")) != 0:
        return                          # under torch.distributed.run only rank 0 measures the host
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(n)      # the launcher exports 1; must change before torch and the C library load
    os.environ["MKL_NUM_THREADS"] = str(n)
    base = cpu_baseline_run(wl, max(1, args.steps), args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": base["steps"], "warmup": base["warmup"], "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": f"{base['dtype']} (CPU torch) + int (hysteresis)", "data": "synthetic",
        "config": {"workload": wl["desc"], "M": wl["M"], "layers": wl["layers"], "threshold": wl["threshold"],
                   "parallelism": f"host CPU, {base['cores']} threads"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------------

class Timer:
    """CUDA-event pairs on the current stream, grouped by name; read after a synchronize."""

    def __init__(self, torch):
        self.torch, self.pairs, self.enabled = torch, {}, False

    def run(self, name, fn, *a, **k):
        if not self.enabled:
            return fn(*a, **k)
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*a, **k)
        e1.record()
        self.pairs.setdefault(name, []).append((e0, e1))
        return out

    def totals(self):
        return {n: (sum(a.elapsed_time(b) for a, b in ps), len(ps)) for n, ps in self.pairs.items()}


GEMM_NAMES = ("gemm_fwd", "gemm_dx", "gemm_dw_hysteresis")
# torch / NCCL work and copy-engine copies: not this library's kernel launches
LIBRARY_NAMES = ("all_", "barrier_post", "barrier_dx", "permute_y", "push_tokens_dma", "push_weights_dma")


class Env:
    """What every leg of the benchmark needs: torch, the package, the device, the process group, the L2 flush buffer."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.pkg = load_package()
        self.ops = self.pkg.int2_tc_ops
        if not os.path.exists(self.pkg.LIB_PATH):
            raise SystemExit("libelleci_int2.so is not built; there is no fallback path")
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)      # larger than the 126 MB L2
        self.peaks, self.peak_kind = measured_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


class StepBench:
    """The layer step of one workload under one partition of the work over the ranks:

      single    one GPU: quantise X, forward, quantise dY (+ fold), quantise G, dW + hysteresis, dX (the reference's order)
      features  N-sharded weights, activations replicated: Y gathered and dX partial sums reduce-scattered by TMA stores
                from the GEMM epilogues into symmetric memory (what BASELINE config 4 describes)
      tokens    token-parallel: every rank runs forward and dX on M/g tokens against a replica of the weights and updates
                N/g rows from all ranks' int8 tokens and gradient windows (token_parallel.TokenParallelInt2Linear, fused)
    """

    def __init__(self, env: Env, wl: dict, partition: str):
        torch, pkg, ops, dev = env.torch, env.pkg, env.ops, env.dev
        self.env, self.wl, self.partition = env, wl, partition
        world, rank = env.world, env.rank
        self.timer = Timer(torch)
        M, thr = wl["M"], wl["threshold"]
        self.M = M
        gen = torch.Generator(device=dev).manual_seed(1234)          # the same stream of numbers on every rank
        self.layers = []

        class L:
            pass

        for li, (K, N) in enumerate(wl["layers"]):
            lay = L()
            lay.K, lay.N = K, N
            lay.gamma = 0.0160
            Wfull = ops.ternarize_pack(torch.randn(N, K, generator=gen, device=dev) * 0.02, lay.gamma)
            h = torch.randint(-wl["counters"], wl["counters"] + 1, (N, K), generator=gen, device=dev, dtype=torch.int8)
            hb = (h & 0xF).to(torch.uint8).view(N, K // 2, 2)
            Hfull = (hb[:, :, 0] | (hb[:, :, 1] << 4)).contiguous()
            del h, hb
            x = torch.randn(M, K, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            # dY in row blocks: a float32 [65536, 16384] temporary would be 4 GB
            dY = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            for r0 in range(0, M, 8192):
                r1 = min(M, r0 + 8192)
                dY[r0:r1] = (torch.randn(r1 - r0, N, generator=gen, device=dev) * wl["dy_std"]).to(torch.bfloat16)
            lay.step = 0
            if partition == "tokens":
                Ml = M // world
                lay.x = x[rank * Ml:(rank + 1) * Ml].contiguous()
                lay.dY = dY[rank * Ml:(rank + 1) * Ml].contiguous()
                del x, dY
                mod = pkg.token_parallel.TokenParallelInt2Linear(K, N, threshold=thr, lr_scale=LR_SCALE, decay_rate=DECAY,
                                                                 hysteresis_order="after_dx", fused=True,
                                                                 push_ctas=env.args.push_ctas).to(dev)
                mod.load_full(Wfull, Hfull, lay.gamma)
                mod.set_lr(LR)
                mod.train()
                mod._run = self.timer.run
                lay.mod = mod
                lay.n0, lay.n1, lay.Nl = mod.row_start, mod.row_stop, mod.local_out_features
                lay.W0 = Wfull[lay.n0:lay.n1].clone()
                lay.current_rows = mod.owned_rows
            else:
                lay.n0, lay.n1 = pkg.sharded.shard_rows(N, world, rank)
                lay.Nl = lay.n1 - lay.n0
                lay.x, lay.dY = x, dY
                lay.Wp = Wfull[lay.n0:lay.n1].clone()
                lay.Hp = Hfull[lay.n0:lay.n1].clone()
                lay.W0, lay.H0 = lay.Wp.clone(), lay.Hp.clone()
                lay.current_rows = (lambda l=lay: l.Wp)
                lay.symm = None
                if partition == "features" and world > 1:
                    import torch.distributed._symmetric_memory as symm_mem
                    grp = env.dist.group.WORLD
                    lay.symm, lay.symm_dx = [], []
                    for _ in range(2):      # two sets of buffers alternate between steps: no barrier guards their reuse
                        ybuf = symm_mem.empty((M, N), dtype=torch.bfloat16, device=dev)
                        lay.symm.append((ybuf, symm_mem.rendezvous(ybuf, grp)))
                        parts = symm_mem.empty((world, M // world, K), dtype=torch.int32, device=dev)
                        dxbuf = symm_mem.empty((M, K), dtype=torch.bfloat16, device=dev)
                        lay.symm_dx.append((parts, symm_mem.rendezvous(parts, grp), dxbuf, symm_mem.rendezvous(dxbuf, grp)))
            del Wfull, Hfull
            self.layers.append(lay)
        self.side = torch.cuda.Stream(device=dev) if partition == "features" and world > 1 else None

    # ---- one layer step per partition -------------------------------------------------------------------------------
    def _step_single(self, lay):
        ops, timer, thr = self.env.ops, self.timer, self.wl["threshold"]
        torch = self.env.torch
        Xq, ax = timer.run("quantize_rows", ops.quantize_rows, lay.x)
        y = timer.run("gemm_fwd", ops.matmul_rows, Xq, lay.Wp, ax, lay.gamma, torch.bfloat16)
        dYq, ady, gmax = timer.run("quantize_rows_dy", ops.quantize_rows, lay.dY, ops.GRAD_EPS, ax)
        lay.step += 1
        Gq = timer.run("quantize_grad", ops.quantize_grad, lay.dY, ax, gmax)
        timer.run("gemm_dw_hysteresis", ops.dw_hysteresis, Gq, Xq, gmax, lay.Wp, lay.Hp, LR, LR_SCALE, thr, DECAY, lay.step, 0)
        dX = timer.run("gemm_dx", ops.backward_input_rows, dYq, lay.Wp, ady, lay.gamma, lay.K, torch.bfloat16)
        return y, dX

    def _step_features(self, lay):
        env, ops, timer, thr = self.env, self.env.ops, self.timer, self.wl["threshold"]
        torch, dist, rank, M, K = env.torch, env.dist, env.rank, self.M, lay.K
        Xq, ax = timer.run("quantize_rows", ops.quantize_rows, lay.x)
        ybuf, hdl = lay.symm[lay.step & 1]
        # forward GEMM fused with the all-gather: the epilogue stores into every rank's Y over NVLink
        timer.run("gemm_fwd", ops.matmul_rows_gather, Xq, lay.Wp, ax, lay.gamma, hdl.buffer_ptrs, lay.N, lay.n0, torch.bfloat16)
        timer.run("barrier_post", hdl.barrier, channel=1)
        window = lay.dY[:, lay.n0:lay.n1]
        if lay.dY.numel() * 2 <= (256 << 20):
            raw = timer.run("absmax_rows", ops.absmax_rows, lay.dY)      # replicated dY: scan all of it, no collective
        else:
            raw = timer.run("absmax_rows", ops.absmax_rows, window)
            timer.run("all_reduce_absmax", dist.all_reduce, raw, op=dist.ReduceOp.MAX)
        dYq, ady, gmax = timer.run("quantize_rows_dy", ops.quantize_rows, window, ops.GRAD_EPS, ax, raw)
        lay.step += 1
        # order "forward, dX, weight update": the dX GEMM scatters its int32 partial sums to the owners; after the barrier
        # the owner's sum + scale + gather pass and its barrier run on a side stream, under the local dW + hysteresis kernel
        parts, hp, dxbuf, hd = lay.symm_dx[lay.step & 1]
        timer.run("gemm_dx", ops.backward_input_scatter, dYq, lay.Wp, K, hp.buffer_ptrs, rank)
        timer.run("barrier_dx1", hp.barrier, channel=3)
        main = torch.cuda.current_stream()
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            timer.run("reduce_scale_gather", ops.reduce_scale_gather, parts, hd.buffer_ptrs, rank, ady, lay.gamma, M, K, torch.bfloat16)
            timer.run("barrier_dx2", hd.barrier, channel=4)
        Gq = timer.run("quantize_grad", ops.quantize_grad, window, ax, gmax)
        timer.run("gemm_dw_hysteresis", ops.dw_hysteresis, Gq, Xq, gmax, lay.Wp, lay.Hp, LR, LR_SCALE, thr, DECAY, lay.step, lay.n0 * K)
        main.wait_stream(self.side)
        return ybuf, dxbuf

    def step(self):
        for lay in self.layers:
            if self.partition == "tokens":
                lay.mod.train_step(lay.x, lay.dY)
            elif self.partition == "features" and self.env.world > 1:
                self._step_features(lay)
            else:
                self._step_single(lay)

    # ---- the measurement -----------------------------------------------------------------------------------------------
    def run(self, steps: int, warmup: int, sample_clocks: bool):
        env, torch, timer = self.env, self.env.torch, self.timer
        # Token partition: the step is replayed from a recorded CUDA graph (one host launch per layer and step); the
        # per-kernel pass below queues the same launches one by one, with an event pair around each.
        self.graphed = self.partition == "tokens" and env.world > 1 and not env.args.no_graph
        for lay in self.layers:
            if hasattr(lay, "mod"):
                lay.mod.graph_steps = self.graphed
        for _ in range(max(warmup, 3)):
            self.step()
        env.barrier()
        env.ops.check_device_status(env.dev)
        sampler = ClockSampler(env.local_rank) if sample_clocks else None
        timer.enabled = env.args.inline_kernel_events
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        env.barrier()
        if sampler:
            sampler.start()
        host_s = 0.0
        for i in range(steps):
            env.flush.zero_()
            ev[i][0].record()
            h0 = time.perf_counter()
            self.step()
            host_s += time.perf_counter() - h0
            ev[i][1].record()
        env.barrier()
        clocks = sampler.stop() if sampler else None
        timer.enabled = False
        total_ms = env.max_over_ranks(sum(a.elapsed_time(b) for a, b in ev))
        env.ops.check_device_status(env.dev)
        if not env.args.inline_kernel_events:
            # The per-kernel event pairs (roofline, breakdown) come from a second pass of the same K steps: inside the
            # headline region the extra event records per step cost about 5 % of it.
            timer.enabled = True
            for lay in self.layers:
                if hasattr(lay, "mod"):
                    lay.mod.graph_steps = False
            for i in range(steps):
                env.flush.zero_()
                self.step()
            env.barrier()
            timer.enabled = False
        totals = timer.totals()
        ms = total_ms / steps
        out = {"partition": self.partition, "ms_per_step": ms, "tokens_per_s": self.M / (ms * 1e-3), "steps": steps,
               "clocks": clocks, "totals": totals,
               # host time spent queueing one step's launches: a step whose device time is close to it is bound by the host
               "host_enqueue_ms_per_step": env.max_over_ranks(host_s * 1e3) / steps, "cuda_graph": self.graphed}
        out["gemm_modes"] = self.gemm_modes(totals, steps)
        out["kernels_ms_per_step"] = {n: t / steps for n, (t, c) in sorted(totals.items())}
        out["own_launches"] = sum(c for n, (t, c) in totals.items() if not n.startswith(LIBRARY_NAMES))
        out["nvlink"] = self.nvlink_bytes_per_step()
        return out

    def gemm_ops_per_mode(self) -> float:
        """2*M*N*K summed over the layers, divided by the ranks: what each of the three GEMM launches of a rank computes."""
        return sum(2.0 * self.M * lay.Nl * lay.K for lay in self.layers)

    def gemm_modes(self, totals, steps):
        per_mode, ops_ = {}, self.gemm_ops_per_mode()
        for n in GEMM_NAMES:
            if n in totals:
                ms, cnt = totals[n]
                per_mode[n] = {"ms_per_launch": ms / cnt, "tops": ops_ * steps / (ms * 1e-3) / 1e12}
        return per_mode

    def nvlink_bytes_per_step(self):
        """Bytes one rank sends to its peers per step (what the partition's exchange costs on NVLink)."""
        g = self.env.world
        if g == 1:
            return None
        total, parts = 0, {}
        for lay in self.layers:
            M, K, N, Nl = self.M, lay.K, lay.N, lay.Nl
            if self.partition == "tokens":
                b = {"tokens_int8": (g - 1) * (M // g) * K, "grad_windows_int8": (g - 1) * (M // g) * Nl,
                     "weight_rows": (g - 1) * Nl * (K // 4)}
            else:
                b = {"y_bf16": (g - 1) * M * Nl * 2, "dx_partials_int32": (g - 1) * (M // g) * K * 4,
                     "dx_rows_bf16": (g - 1) * (M // g) * K * 2}
            for k, v in b.items():
                parts[k] = parts.get(k, 0) + v
                total += v
        return {"sent_bytes_per_rank": total, "by_kind": parts}

    def changed_fraction(self):
        lay, ops, torch = self.layers[0], self.env.ops, self.env.torch
        now = lay.current_rows().contiguous()
        a = torch.empty(lay.Nl, lay.K, dtype=torch.int8, device=self.env.dev)
        b = torch.empty_like(a)
        ops.unpack_int2(now, a, lay.K)
        ops.unpack_int2(lay.W0, b, lay.K)
        return float((a != b).float().mean().item())


def int8_ceiling(env: Env, n: int = 8192, reps: int = 10):
    """The library int8 GEMM (cuBLASLt through torch._int_mm) at n^3, best of `reps`, in TOP/s: a measured ceiling of the
    int8 tensor pipe on this box, taken outside every timed region of the layer step."""
    torch = env.torch
    try:
        a = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=env.dev)
        b = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=env.dev).t()
        for _ in range(3):
            torch._int_mm(a, b)
        best = float("inf")
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception as e:  # noqa: BLE001 - the ceiling is context, not a dependency of the measurement
        return {"unavailable": repr(e)[:200]}


def traffic_from_profile(kernel_key: str):
    """DRAM bytes per launch of the dominant kernel as captured by ncu, read from the committed summary that holds it
    (a line `traffic_bytes_per_launch[<key>]: <number>`), so that the figure and its source stay together."""
    prof_dir = os.path.join(ROOT, "profiles")
    if not os.path.isdir(prof_dir):
        return None, None
    tag = f"traffic_bytes_per_launch[{kernel_key}]:"
    for name in sorted(os.listdir(prof_dir)):
        try:
            with open(os.path.join(prof_dir, name)) as f:
                for line in f:
                    if tag in line:
                        return float(line.split(tag, 1)[1].split()[0]), f"profiles/{name}"
        except (OSError, ValueError):
            continue
    return None, None


def measure_config1(env: Env, reps: int = 20):
    """BASELINE config 1: the forward GEMM alone at M=4096 for the four 7B projections, bf16 out.  Each launch is timed by
    its own event pair after an (untimed) L2 flush; int8 tokens and scales are made once per shape."""
    torch, ops, dev = env.torch, env.ops, env.dev
    M, out = 4096, []
    gen = torch.Generator(device=dev).manual_seed(11)
    for K, N in ((4096, 4096), (4096, 11008), (11008, 4096), (4096, 512)):
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        Wp = ops.ternarize_pack(torch.randn(N, K, generator=gen, device=dev) * 0.02, 0.016)
        Xq, ax = ops.quantize_rows(x)
        for _ in range(3):
            ops.matmul_rows(Xq, Wp, ax, 0.016, torch.bfloat16)
        total = 0.0
        for _ in range(reps):
            env.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.matmul_rows(Xq, Wp, ax, 0.016, torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ms = total / reps
        xq_ms = 0.0
        for _ in range(reps):
            env.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ops.quantize_rows(x)
            e1.record()
            torch.cuda.synchronize()
            xq_ms += e0.elapsed_time(e1)
        out.append({"K": K, "N": N, "gemm_ms": ms, "tops": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "quantize_ms": xq_ms / reps,
                    "tokens_per_s_forward": M / ((ms + xq_ms / reps) * 1e-3)})
        del x, Wp, Xq
    env.ops.check_device_status(dev)
    return {"M": M, "l2": "flushed before every timed launch", "shapes": out}


def measure_config3(env: Env, reps: int = 10, nbuf: int = 16):
    """BASELINE config 3 in brief: the decode call at M in {1, 8, 32, 64} for both MLP shapes, sixteen weight buffers
    (more than L2) rotated inside one CUDA graph so that every call streams its weights from HBM; time per call = graph
    time / 16.  Default kernel selection of el_linear_decode, dependent-launch overlap off."""
    torch, ops, dev = env.torch, env.ops, env.dev
    cases = []
    for (K, N) in ((4096, 11008), (11008, 4096)):
        gen = torch.Generator(device=dev).manual_seed(K)
        Ws = [torch.randint(0, 256, (N, K // 4), generator=gen, device=dev, dtype=torch.uint8) for _ in range(nbuf)]
        for M in (1, 8, 32, 64):
            x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
            for W in Ws[:3]:
                ops.linear_decode(x, W, 0.016)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for W in Ws:
                    y = ops.linear_decode(x, W, 0.016)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * nbuf)
            nbytes = N * K // 4 + 2 * M * K + 2 * M * N
            gbs = nbytes / (us * 1e-6) / 1e9
            cases.append({"M": M, "K": K, "N": N, "us_per_call": us, "GBps": gbs, "frac_of_hbm": gbs / env.peaks["hbm_gbs"]})
            del graph, y
        del Ws
    ops.check_device_status(dev)
    return {"cases": cases, "peak": env.peaks["hbm_gbs"], "peak_source": f"hbm_gbs ({env.peak_kind})",
            "method": f"{nbuf} rotating weight buffers in one CUDA graph, {reps} replays"}


def measure_hysteresis(env: Env, reps: int = 10):
    """The stand-alone hysteresis update (float32 gradient in, the reference-compatible entry point) at 11008 x 4096,
    L2 flushed before every launch; 5.5 algorithmic bytes per weight."""
    torch, ops, dev = env.torch, env.ops, env.dev
    N, K = 11008, 4096
    gen = torch.Generator(device=dev).manual_seed(3)
    Wp = ops.ternarize_pack(torch.randn(N, K, generator=gen, device=dev) * 0.02, 0.016)
    Hp = torch.randint(0, 256, (N, K // 2), generator=gen, device=dev, dtype=torch.uint8)
    dW = torch.randn(N, K, generator=gen, device=dev) * 1e-3
    for s in range(3):
        ops.hysteresis_step_v2(dW, Wp, Hp, 1e-2, 5.0, 3, 0.001, s + 1)
    total = 0.0
    for s in range(reps):
        env.flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.hysteresis_step_v2(dW, Wp, Hp, 1e-2, 5.0, 3, 0.001, s + 10)
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    ms = total / reps
    gbs = N * K * 5.5 / (ms * 1e-3) / 1e9
    return {"N": N, "K": K, "ms": ms, "GBps": gbs, "frac_of_hbm": gbs / env.peaks["hbm_gbs"], "algorithmic_bytes": N * K * 5.5}


def measure_ref_cuda(env: Env):
    """The reference's own CUDA extension (compiled unmodified for sm_100a into oracle/_ref/, when present) on this same
    GPU at the 4096 <-> 11008 shapes, timed the way its own benchmark does (kernels/tests/test_perf.py:19-58: 10
    warm-up calls, then 50 calls between one event pair, no cache flush), next to this library's kernels timed the
    same way.  Runs outside every timed region of the layer step."""
    torch, ops, dev = env.torch, env.ops, env.dev
    try:
        from oracle import ref_cuda
        ref = ref_cuda.load()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"loading oracle/_ref/int2_tc_ops_ref.so failed: {repr(e)[:160]}"}
    if ref is None:
        return {"unavailable": "oracle/_ref/int2_tc_ops_ref.so is not built on this box"}

    def time_ms(fn, iters=50, warmup=10):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    M, gamma = 4096, 0.016
    gen = torch.Generator(device=dev).manual_seed(5)
    rows = []
    for K, N in ((4096, 11008), (11008, 4096)):
        X = torch.randn(M, K, generator=gen, device=dev).half()
        dY = (torch.randn(M, N, generator=gen, device=dev) * 1e-3).half()
        Wp = ops.ternarize_pack(torch.randn(N, K, generator=gen, device=dev) * 0.02, gamma)
        Hp = torch.zeros(N, K // 2, dtype=torch.uint8, device=dev)
        dW = torch.randn(N, K, generator=gen, device=dev) * 1e-3
        scratch = torch.zeros(1, dtype=torch.float32, device=dev)
        Xq, sx = ref.quantize_activation_async(X, scratch)
        dYq, sy = ref.quantize_activation_async(dY, scratch)
        Wr, Hr = Wp.clone(), Hp.clone()
        step = [0]

        def ref_hyst():
            step[0] += 1
            ref.hysteresis_step_v2(dW, Wr, Hr, 1e-2, 5.0, 3, 0.001, step[0])

        def our_hyst():
            step[0] += 1
            ops.hysteresis_step_v2(dW, Wp, Hp, 1e-2, 5.0, 3, 0.001, step[0])

        gop = 2.0 * M * N * K
        pairs = {
            "matmul_int8": (lambda: ref.matmul_int8(Xq, Wr, sx, gamma), lambda: ops.matmul_int8(Xq, Wp, sx, gamma), gop),
            "backward_input_int8": (lambda: ref.backward_input_int8(dYq, Wr, sy, gamma, K),
                                    lambda: ops.backward_input_int8(dYq, Wp, sy, gamma, K), gop),
            "quantize_activation_async": (lambda: ref.quantize_activation_async(X, scratch),
                                          lambda: ops.quantize_activation_async(X, scratch), None),
            "hysteresis_step_v2": (ref_hyst, our_hyst, None),
        }
        for name, (fr, fo, work) in pairs.items():
            r_ms, o_ms = time_ms(fr), time_ms(fo)
            row = {"op": name, "K": K, "N": N, "reference_ms": r_ms, "ours_ms": o_ms, "speedup": r_ms / o_ms}
            if work:
                row["reference_tops"], row["ours_tops"] = work / (r_ms * 1e-3) / 1e12, work / (o_ms * 1e-3) / 1e12
            rows.append(row)
        del X, dY, Wp, Hp, dW, Wr, Hr
    ops.check_device_status(dev)
    return {"M": M, "method": "10 warm-up calls, 50 calls between one CUDA-event pair, no cache flush (the reference benchmark's own)",
            "rows": rows}


def gpu_local_cpus(torch, index: int):
    """The CPUs on the NUMA node the GPU's PCIe slot hangs off (from sysfs), restricted to those this process may use;
    None when the system does not say."""
    try:
        pr = torch.cuda.get_device_properties(index)
        path = f"/sys/bus/pci/devices/{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0/local_cpulist"
        with open(path) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        cpus &= os.sched_getaffinity(0)
        return cpus or None
    except (OSError, ValueError, AttributeError):
        return None


def measure_e2e(env: Env, bench: StepBench, steps: int):
    """The same step through the module API with HOST buffers: every step copies the layers' inputs (X and dY of each
    layer) from pinned host memory to the device and copies each layer's results (Y and dX) back to pinned host memory,
    all inside the timed region.  With several GPUs every rank moves its own tokens (token-parallel layer)."""
    torch, pkg, dev = env.torch, env.pkg, env.dev
    wl, thr = bench.wl, bench.wl["threshold"]
    mods = []
    # The pinned host buffers are allocated from a thread that runs on the GPU's own NUMA node, so that their pages sit
    # next to the GPU's PCIe root: on a two-socket host, pages on the other socket put the inter-socket link into every
    # copy.  (What a trainer's data loader does with its staging buffers.)  The affinity is put back afterwards.
    old_affinity = os.sched_getaffinity(0)
    local = gpu_local_cpus(torch, dev.index)
    if local:
        os.sched_setaffinity(0, local)
    for lay in bench.layers:
        if bench.partition == "tokens":
            m = lay.mod
            m._run = lambda name, fn, *a, **k: fn(*a, **k)
        else:
            m = pkg.Int2LinearTCWithGradHook(lay.K, lay.N, threshold=thr, lr_scale=LR_SCALE, decay_rate=DECAY).to(dev)
            m.W_packed.copy_(lay.W0)
            m.H_packed.copy_(lay.H0)
            m.gamma.data.fill_(lay.gamma)
            m._gamma_cached = lay.gamma
            m._initialized = True
            m.set_lr(LR)
            m.train()
        xh, dyh = lay.x.cpu().pin_memory(), lay.dY.cpu().pin_memory()
        yh = torch.empty(xh.shape[0], lay.N, dtype=torch.bfloat16).pin_memory()
        dxh = torch.empty(xh.shape[0], lay.K, dtype=torch.bfloat16).pin_memory()
        mods.append((m, xh, dyh, yh, dxh))
    if local:
        os.sched_setaffinity(0, old_affinity)
    h2d = sum(x.numel() * 2 + dy.numel() * 2 for _, x, dy, _, _ in mods)
    d2h = sum(y.numel() * 2 + dx.numel() * 2 for _, _, _, y, dx in mods)
    copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_step():
        # A training step's order: forward through the layers, backward through them in reverse.  The host->device
        # copies go out on a copy stream in the order the step needs them (inputs first, then the output gradients,
        # last layer's first), results leave on a second copy stream as they appear; PCIe is full duplex, so Y of the
        # first layer already travels back while the later inputs still arrive.  What arrives last (the first layer's
        # gradient) feeds the smallest result (its dX), which keeps the tail after the last arrival short.
        main = torch.cuda.current_stream()
        copy_in.wait_stream(main)                  # copies start inside the timed region
        xs, dys = [], {}
        with torch.cuda.stream(copy_in):
            for i, (m, xh, dyh, yh, dxh) in enumerate(mods):
                x = xh.to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                xs.append((x, ev))
            for i in reversed(range(len(mods))):
                dy = mods[i][2].to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                dys[i] = (dy, ev)
        ys = []
        for (m, xh, dyh, yh, dxh), (x, ev) in zip(mods, xs):
            main.wait_event(ev)
            x.record_stream(main)
            x.requires_grad_(True)
            y = m(x)
            copy_out.wait_stream(main)
            with torch.cuda.stream(copy_out):
                yh.copy_(y.detach(), non_blocking=True)
            y.record_stream(copy_out)
            ys.append(y)
        for i in reversed(range(len(mods))):
            (m, xh, dyh, yh, dxh), (x, _), (dy, ev) = mods[i], xs[i], dys[i]
            main.wait_event(ev)
            dy.record_stream(main)
            ys[i].backward(dy)
            copy_out.wait_stream(main)
            with torch.cuda.stream(copy_out):
                dxh.copy_(x.grad, non_blocking=True)
            x.grad.record_stream(copy_out)
        main.wait_stream(copy_out)                 # the step ends when its results are on the host

    def e2e_step_per_layer():
        # the other order (--e2e-order layer): each layer's forward and backward back to back, all inputs copied first
        main = torch.cuda.current_stream()
        copy_in.wait_stream(main)
        staged = []
        with torch.cuda.stream(copy_in):
            for m, xh, dyh, yh, dxh in mods:
                x = xh.to(dev, non_blocking=True)
                dy = dyh.to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_in)
                staged.append((m, x, dy, ev, yh, dxh))
        for m, x, dy, ev, yh, dxh in staged:
            main.wait_event(ev)
            x.record_stream(main)
            dy.record_stream(main)
            x.requires_grad_(True)
            y = m(x)
            copy_out.wait_stream(main)
            with torch.cuda.stream(copy_out):
                yh.copy_(y.detach(), non_blocking=True)
            y.record_stream(copy_out)
            y.backward(dy)
            copy_out.wait_stream(main)
            with torch.cuda.stream(copy_out):
                dxh.copy_(x.grad, non_blocking=True)
            x.grad.record_stream(copy_out)
        main.wait_stream(copy_out)

    if env.args.e2e_order == "layer":
        e2e_step = e2e_step_per_layer
    e_steps = max(3, min(steps, 20))
    for _ in range(3):
        e2e_step()
    env.barrier()
    ee = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(e_steps)]
    for i in range(e_steps):
        env.flush.zero_()
        ee[i][0].record()
        e2e_step()
        ee[i][1].record()
    env.barrier()
    e_ms = env.max_over_ranks(sum(a.elapsed_time(b) for a, b in ee)) / e_steps
    env.ops.check_device_status(dev)
    per_rank = " per rank" if env.world > 1 else ""
    return {"value": bench.M / (e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": e_ms, "steps": e_steps,
            "bound": (f"host link: {(h2d + d2h) / 1e6:.0f} MB{per_rank} cross PCIe per step (X, dY in; Y, dX out); "
                      f"the link moved {max(h2d, d2h) / (e_ms * 1e-3) / 1e9:.1f} GB/s in its busier direction"),
            "api": "token_parallel.TokenParallelInt2Linear (autograd)" if bench.partition == "tokens"
                   else "Int2LinearTCWithGradHook (autograd, gradient hook)",
            "host_buffers": ("pinned, allocated on the GPU's NUMA node" if local else "pinned (the GPU's NUMA node is not known)")}


def run_ours(args, wl):
    env = Env(args)
    torch, world = env.torch, env.world
    if world > 1 and wl["M"] % (32 * world) != 0:
        raise SystemExit("the token count must divide by 32 x the number of GPUs")
    partitions = ["single"] if world == 1 else (["tokens", "features"] if args.partition == "both" else [args.partition])
    results, benches = {}, {}
    for part in partitions:
        b = StepBench(env, wl, part)
        results[part] = b.run(args.steps, args.warmup, sample_clocks=True)
        results[part]["weights_changed_after_run"] = b.changed_fraction()
        benches[part] = b
        if part != partitions[-1] or world > 1:
            pass
    best = max(results, key=lambda p: results[p]["tokens_per_s"])
    res, bench = results[best], benches[best]
    for p in partitions:                       # free the partition that is not the headline before the other legs
        if p != best:
            del benches[p]
    torch.cuda.empty_cache()

    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(env, bench, args.steps)

    # ---- sub-records (rank 0 measures the single-GPU ones; config 4 runs on all ranks) ---------------------------------
    config4 = None
    if args.workload == "config2" and not args.no_config4:
        del bench, benches
        torch.cuda.empty_cache()
        b4 = StepBench(env, WORKLOADS["config4"], "single" if world == 1 else "tokens")
        r4 = b4.run(min(args.steps, 10), 3, sample_clocks=False)
        config4 = {"workload": WORKLOADS["config4"]["desc"], "partition": r4["partition"], "ms_per_step": r4["ms_per_step"],
                   "tokens_per_s": r4["tokens_per_s"], "steps": r4["steps"], "gemm_modes": r4["gemm_modes"],
                   "kernels_ms_per_step": r4["kernels_ms_per_step"], "nvlink": r4["nvlink"],
                   "tops_whole_step": 3 * 2.0 * 65536 * 16384 * 4096 / (r4["ms_per_step"] * 1e-3) / 1e12}
        if r4["nvlink"]:
            config4["nvlink"]["GBps_if_serial"] = r4["nvlink"]["sent_bytes_per_rank"] / (r4["ms_per_step"] * 1e-3) / 1e9
        del b4
        torch.cuda.empty_cache()

    if env.rank != 0:
        if world > 1:
            env.dist.barrier()
            env.dist.destroy_process_group()
        return

    extras = {}
    if world == 1 and not args.brief:
        extras["int8_ceiling_tops"] = int8_ceiling(env)
        extras["config1"] = measure_config1(env)
        extras["config3"] = measure_config3(env)
        extras["hysteresis_standalone"] = measure_hysteresis(env)
        extras["pre_norm"] = measure_pre_norm(torch, env.pkg, wl["M"], wl["layers"][0][0], env.dev, env.flush, env.peaks)
        extras["ref_cuda_same_box"] = measure_ref_cuda(env)
    elif not args.brief:
        extras["int8_ceiling_tops"] = int8_ceiling(env)

    # ---- roofline of the dominant kernel (the tcgen05 GEMM in its three modes) -----------------------------------------
    peaks = env.peaks
    totals = res["totals"]
    gemm_ms = sum(totals[n][0] for n in GEMM_NAMES)
    gemm_launches = sum(totals[n][1] for n in GEMM_NAMES)
    ops_per_mode = sum(2.0 * wl["M"] * N * K for K, N in wl["layers"]) / world
    achieved = 3.0 * ops_per_mode * res["steps"] / (gemm_ms * 1e-3) / 1e12
    # The timed region is tens of milliseconds at full clock, far from the power-capped regime of the sustained figure:
    # the burst row applies.  int8 runs at twice the bf16 rate on this part; MEASURED_PEAKS.json has no int8 row.
    int8_peak = 2.0 * peaks["bf16_tflops"]
    traffic, traffic_src = traffic_from_profile("gemm_config2")
    if args.workload != "config2" or world > 1:
        traffic, traffic_src = None, None
    ceiling = extras.get("int8_ceiling_tops")
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s", "frac": achieved / int8_peak,
        "traffic": traffic, "traffic_source": traffic_src,
        "algorithmic_bytes_per_launch": sum(wl["M"] * K + N * K // 4 + 2 * wl["M"] * N for K, N in wl["layers"]) / len(wl["layers"]),
        "kernel": "gemm_tc2_kernel / gemm_tc_kernel (tcgen05 kind::i8; forward, dX and dW+hysteresis launches)",
        "launches": gemm_launches, "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
        "timing": ("CUDA event pair around every launch, " + ("inside the headline region" if args.inline_kernel_events else
                   "second pass of the same K steps right after the headline region (the headline has one pair per step)")),
        "peak_source": f"2 x bf16_tflops (burst) of MEASURED_PEAKS.json ({env.peak_kind}); of measured",
        "frac_of_nominal_int8": achieved / 4500.0,
        "int8_ceiling_tops": ceiling,
        "frac_of_int8_ceiling": (achieved / ceiling) if isinstance(ceiling, float) else None,
        "whole_step_tops": 3.0 * ops_per_mode * world / (res["ms_per_step"] * 1e-3) / 1e12,
    }
    hbm = {}
    Mq = wl["M"] // world if best == "tokens" else wl["M"]
    bytes_per_step = {
        "quantize_rows": sum(Mq * lay.K * 3 + 4 * Mq for lay in bench_layers_meta(wl, world, best)),
        "quantize_rows_dy": sum(Mq * lay.Nq * 3 + 8 * Mq for lay in bench_layers_meta(wl, world, best)),
        "quantize_grad": sum(Mq * lay.Nq * 3 + 4 * Mq for lay in bench_layers_meta(wl, world, best)),
    }
    for n, b in bytes_per_step.items():
        if n in totals:
            ms, cnt = totals[n]
            gbs = b * res["steps"] / (ms * 1e-3) / 1e9
            hbm[n] = {"ms_per_launch": ms / cnt, "GBps": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"]}
    if "hysteresis_standalone" in extras:
        hbm["hysteresis_from_dw (stand-alone, outside the step)"] = extras.pop("hysteresis_standalone")

    cpu = cpu_baseline_run(wl, steps=3, warmup=4) if world == 1 and not args.no_cpu else None

    par = {"single": "single GPU (order: forward, weight update, dX - the reference's hook order)",
           "tokens": (f"token-parallel x{world}: every rank runs forward and dX on {wl['M'] // world} tokens against a replica of "
                      "W_packed and updates N/g rows from all ranks' int8 tokens and gradient windows; exchanges are this "
                      "library's peer stores + barrier (order: forward, dX, weight update)"
                      + ("" if args.no_graph else "; each layer's step replayed from a recorded CUDA graph")),
           "features": (f"N-sharded x{world}, activations replicated: Y gathered and dX partial sums reduce-scattered by TMA "
                        "stores from the GEMM epilogues, dX rows summed and re-gathered by peer stores on a side stream")}
    line = {
        "metric": METRIC, "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 x int2 -> int32 (bf16 in/out)", "data": "synthetic",
        "config": {"workload": wl["desc"], "M": wl["M"], "layers": wl["layers"], "threshold": wl["threshold"],
                   "parallelism": par[best], "l2": "256 MiB written between timed steps (untimed)",
                   "weights_changed_after_run": res["weights_changed_after_run"]},
        "clocks": res["clocks"], "e2e": e2e, "gpu_launches": res["own_launches"],
        "roofline": roofline, "gemm_modes": res["gemm_modes"], "hbm_kernels": hbm,
        "kernels_ms_per_step": res["kernels_ms_per_step"],
        "host_enqueue_ms_per_step": res["host_enqueue_ms_per_step"],
    }
    if res["nvlink"]:
        line["nvlink"] = res["nvlink"]
    if len(results) > 1:
        line["partitions"] = {p: {"ms_per_step": r["ms_per_step"], "tokens_per_s": r["tokens_per_s"], "gemm_modes": r["gemm_modes"],
                                  "kernels_ms_per_step": r["kernels_ms_per_step"], "nvlink": r["nvlink"], "parallelism": par[p],
                                  "host_enqueue_ms_per_step": r["host_enqueue_ms_per_step"], "cuda_graph": r["cuda_graph"]}
                              for p, r in results.items()}
    if config4 is not None:
        line["config4"] = config4
    for k, v in extras.items():
        line[k] = v
    if cpu is not None:
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))
    if world > 1:
        env.dist.barrier()
        env.dist.destroy_process_group()


def bench_layers_meta(wl, world, partition):
    """(K, columns of dY a rank quantises) per layer: all N columns of its own tokens (single, tokens) or its N/g window."""
    class Meta:
        pass
    out = []
    for K, N in wl["layers"]:
        m = Meta()
        m.K, m.Nq = K, (N // world if partition == "features" else N)
        out.append(m)
    return out


def measure_pre_norm(torch, pkg, M, K, dev, flush, peaks, reps=10):
    """The pre-linear RMSNorm row of the path (outside the headline step): the fused norm + quantise kernel and the
    fused norm backward on the first layer's activation shape, next to the same work done as the reference does it
    (the norm as separate tensor operations, then the quantiser).  Each is captured in a CUDA graph over rotating
    input buffers that together exceed L2 and timed per call with CUDA events around the replays."""
    ops = pkg.int2_tc_ops
    gen = torch.Generator().manual_seed(77)
    nbuf = max(2, (192 << 20) // (M * K * 2) + 1)
    xs = [torch.randn(M, K, generator=gen).to(torch.bfloat16).to(dev) for _ in range(nbuf)]
    gs = [(torch.randn(M, K, generator=gen) * 1e-2).to(torch.bfloat16).to(dev) for _ in range(nbuf)]
    norm = pkg.bitnet_int2_optimized._ExtraRMSNorm(K).to(dev)
    w = norm.weight.detach()
    rstd = [ops.rmsnorm_quantize_rows(x, w)[2] for x in xs]

    def timed(fn):
        for i in range(nbuf):
            fn(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = [fn(i) for i in range(nbuf)]
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        del keep
        return e0.elapsed_time(e1) / (reps * nbuf)

    fwd_ms = timed(lambda i: ops.rmsnorm_quantize_rows(xs[i], w))
    bwd_ms = timed(lambda i: ops.rmsnorm_backward(gs[i], xs[i], w, rstd[i]))
    with torch.no_grad():
        unfused_ms = timed(lambda i: ops.quantize_rows(norm(xs[i])))
    fwd_bytes = M * K * 3 + 8 * M + 4 * K
    bwd_bytes = M * K * 6 + 4 * M + 8 * K
    return {"shape": [M, K], "dtype": "bf16", "buffers": nbuf,
            "rmsnorm_quantize_rows": {"ms": fwd_ms, "GBps": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                      "frac_of_hbm": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "rmsnorm_backward": {"ms": bwd_ms, "GBps": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
                                 "frac_of_hbm": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "unfused_forward_ms": unfused_ms}


def run_decode(args):
    """config3: the small-M layer call at decode shapes, measured against the HBM roofline.  Sixteen distinct weight
    buffers (180 MB, more than L2) are rotated inside one CUDA graph so that every call streams its weights from
    HBM; time per call = graph time / 16, CUDA events around the replays."""
    import torch
    pkg = load_package()
    ops = pkg.int2_tc_ops
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks, peak_kind = measured_peaks()
    cases = []
    stream_us = {}
    nbuf = 16
    for (K, N) in [(4096, 11008), (11008, 4096)]:
        gen = torch.Generator().manual_seed(K)
        Ws = [torch.randint(0, 256, (N, K // 4), generator=gen, dtype=torch.uint8).to(dev) for _ in range(nbuf)]
        # yardstick of the harness itself: a device-to-device copy of the same 16 weight buffers (one copy each, 11 MB
        # read and 11 MB written) in the same kind of graph - what moving one weight matrix per launch costs here
        # before any decode work
        dst = torch.empty_like(Ws[0])
        for W in Ws[:3]:
            dst.copy_(W)
        torch.cuda.synchronize()
        sgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(sgraph):
            for W in Ws:
                dst.copy_(W)
        for _ in range(3):
            sgraph.replay()
        torch.cuda.synchronize()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(max(args.steps, 10)):
            sgraph.replay()
        s1.record()
        torch.cuda.synchronize()
        stream_us[f"{K}x{N}"] = s0.elapsed_time(s1) * 1e3 / (max(args.steps, 10) * nbuf)
        del sgraph, dst
        # overlap: the GEMV issued as a programmatic dependent launch (weights constant, as at inference), so that a
        # call's weight loads start under the tail of the previous call
        # columns: tokens, limit of the CUDA-core GEMV, limit of the warp-MMA kernel (tcgen05 stream-K above it), overlap
        for M, gemv_max, mma_max, overlap in ((1, 1, 64, False), (1, 1, 64, True), (1, 0, 64, True), (2, 2, 64, True),
                                              (2, 1, 64, True), (4, 4, 64, True), (4, 1, 64, False), (4, 1, 64, True),
                                              (8, 8, 64, True), (8, 1, 64, False), (8, 1, 64, True), (8, 0, 0, False),
                                              (16, 1, 64, True), (16, 0, 0, False), (32, 1, 64, True), (32, 1, 0, False),
                                              (64, 1, 64, False), (64, 1, 0, False)):
            pkg._lib.lib().el_set_decode_gemv_max_tokens(gemv_max)
            pkg._lib.lib().el_set_decode_mma_max_tokens(mma_max)
            ops.set_decode_overlap(overlap)
            x = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(dev)
            for W in Ws[:3]:
                ops.linear_decode(x, W, 0.016)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for W in Ws:
                    y = ops.linear_decode(x, W, 0.016)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            reps = max(args.steps, 10)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * nbuf)
            nbytes = N * K // 4 + 2 * M * K + 2 * M * N
            gbs = nbytes / (us * 1e-6) / 1e9
            mt = 8 if M <= 8 else (16 if M <= 16 else 32)      # tokens per launch of the warp-MMA kernel, padded
            fits_mma = M <= mma_max and 256 + ((K + 255) // 256) * 16 * mt * 16 + 2 * 16 * mt * 4 <= 200 * 1024
            kernel = "gemv" if M <= gemv_max else (("mma" if M <= 8 else "mma_preq") if fits_mma else "tcgen05")
            cases.append({"M": M, "K": K, "N": N, "kernel": kernel, "overlap": overlap, "us_per_call": us, "GBps": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"],
                          "algorithmic_bytes": nbytes})
        ops.check_device_status(dev)
        del Ws
    pkg._lib.lib().el_set_decode_gemv_max_tokens(2)
    pkg._lib.lib().el_set_decode_mma_max_tokens(64)
    ops.set_decode_overlap(False)
    # The feed-forward block at decode through the module API: six blocks (203 MB of packed weights) rotated in one graph.
    # Without gradient recording each layer is one small kernel (norm / gate) plus the decode call; with it, the training
    # kernels (fused norm or gate + quantiser, then the tcgen05 GEMM).
    ffns = []
    for i in range(6):
        f = pkg.SwiGLUFFNInt2(4096).to(dev).eval()
        for layer in (f.w1, f.w2, f.w3):
            il = layer.int2_layer
            il.init_from_float(torch.randn(il.out_features, il.in_features, device=dev) * 0.02)
        ffns.append(f)
    module_cases = []
    for M in (1, 8, 32):
        xm = torch.randn(M, 4096, device=dev).to(torch.bfloat16)
        row = {"M": M}
        for name, ctx in (("inference_us", torch.no_grad), ("training_kernels_us", torch.enable_grad)):
            with ctx():
                for f in ffns[:2]:
                    f(xm)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    keep = [f(xm) for f in ffns]
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            reps = max(args.steps, 10)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            row[name] = e0.elapsed_time(e1) * 1e3 / (reps * len(ffns))
            del graph, keep
        module_cases.append(row)
    ops.check_device_status(dev)
    del ffns
    head = next(c for c in cases if c["M"] == 1 and c["K"] == 4096 and c["overlap"])
    line = {
        "metric": "decode linear call (quantise + packed-weight GEMV), GB/s of algorithmic bytes", "value": head["GBps"],
        "unit": "GB/s", "n_gpus": 1, "steps": max(args.steps, 10), "warmup": 3, "ms_per_step": head["us_per_call"] * 1e-3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int2 -> int32 (bf16 in/out)",
        "data": "synthetic",
        "config": {"workload": "config3: decode shapes, M in {1,4,8,16,32,64}, 4096->11008 and 11008->4096; 16 rotating weight "
                               "buffers (> L2) in one CUDA graph; value = M=1, 4096->11008, dependent-launch overlap on"},
        "roofline": {"bound": "hbm", "achieved": head["GBps"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": head["GBps"] / peaks["hbm_gbs"], "traffic": None, "peak_source": f"hbm_gbs ({peak_kind})"},
        "cases": cases, "copy_us_per_call": stream_us,
        "ffn_block_4096_11008_module_api": module_cases, "gpu_launches": 2 * nbuf * max(args.steps, 10),
    }
    print(json.dumps(line))


def run_hbm_kernels(args):
    """The memory-bound kernels that the layer step does not launch in its fused form, each alone at the 4096 x 11008
    layer's size: stand-alone hysteresis update from a float32 gradient, ternarise + pack, unpack, the per-tensor
    quantiser pair of the reference rule, the post-reduction scale pass, the plain dW GEMM's float32 output feeding the
    stand-alone update.  L2 is flushed before every timed launch; GB/s counts the algorithmic bytes."""
    import torch
    pkg = load_package()
    ops = pkg.int2_tc_ops
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks, peak_kind = measured_peaks()
    N, K, M = 11008, 4096, 4096
    gen = torch.Generator().manual_seed(3)
    W = (torch.randn(N, K, generator=gen) * 0.02).to(dev)
    gamma = float(W.abs().mean().item())
    Wp = ops.ternarize_pack(W, gamma)
    Hp = torch.randint(0, 256, (N, K // 2), generator=gen, dtype=torch.uint8).to(dev)
    dW = (torch.randn(N, K, generator=gen) * 1e-3).to(dev)
    x16 = torch.randn(M, K, generator=gen).to(torch.float16).to(dev)
    acc = torch.randint(-100000, 100000, (M, K), generator=gen, dtype=torch.int32).to(dev)
    ax = torch.rand(M, generator=gen).to(dev) + 0.5
    w8 = torch.empty(N, K, dtype=torch.int8, device=dev)
    gmax = torch.zeros(1, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    reps = max(args.steps, 2)

    def timed(fn):
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(reps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / reps

    step = [0]

    def hyst():
        step[0] += 1
        ops.hysteresis_step_v2(dW, Wp, Hp, 1e-2, 5.0, 3, 0.001, step[0])

    q8, sc = ops.quantize_activation_async(x16, gmax)
    # SwiGLU gate in front of the 11008 -> 4096 down projection: gate|up as one [M, 2H] matrix
    Hd = N
    gu = torch.randn(M, 2 * Hd, generator=gen).to(torch.bfloat16).to(dev)
    gyh = (torch.randn(M, Hd, generator=gen) * 1e-2).to(torch.bfloat16).to(dev)
    dgu = torch.empty_like(gu)
    nw = torch.ones(Hd, device=dev)
    norm_mod = pkg.bitnet_int2_optimized._ExtraRMSNorm(Hd).to(dev)
    rstd_h = ops.swiglu_quantize_rows(gu[:, :Hd], gu[:, Hd:], nw)[2]

    def swiglu_unfused():
        with torch.no_grad():
            return ops.quantize_rows(norm_mod(torch.nn.functional.silu(gu[:, :Hd]) * gu[:, Hd:]))

    cases = {
        "swiglu_quantize_rows (silu*up + norm + quantise)": (lambda: ops.swiglu_quantize_rows(gu[:, :Hd], gu[:, Hd:], nw), M * Hd * 5.0),
        "swiglu_backward (norm + gate backward)": (lambda: ops.swiglu_backward(gyh, gu[:, :Hd], gu[:, Hd:], nw, rstd_h, out=dgu), M * Hd * 10.0),
        "same forward as tensor operations + quantiser (bytes of the fused form)": (swiglu_unfused, M * Hd * 5.0),
        "hysteresis_from_dw": (hyst, N * K * 5.5),
        "ternarize_pack": (lambda: ops.ternarize_pack(W, gamma, out=Wp), N * K * 4.25),
        "unpack_int2": (lambda: ops.unpack_int2(Wp, w8, K), N * K * 1.25),
        "quantize_tensor (reference rule, absmax + quantise)": (lambda: ops.quantize_activation_async(x16, gmax), M * K * 5.0),
        "dequantize_tensor": (lambda: ops.dequantize_activation(q8, sc), M * K * 3.0),
        "scale_rows (int32 -> bf16)": (lambda: ops.scale_rows(acc, ax, 0.02, torch.bfloat16), M * K * 6.0),
    }
    out = {}
    for name, (fn, nbytes) in cases.items():
        ms = timed(fn)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "GBps": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"], "algorithmic_bytes": nbytes}
    ops.check_device_status(dev)
    head = out["hysteresis_from_dw"]
    print(json.dumps({
        "metric": "stand-alone memory-bound kernels of the INT2 linear path, GB/s of algorithmic bytes", "value": head["GBps"],
        "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": 3, "ms_per_step": head["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int2/int4 state, f32 gradient", "data": "synthetic",
        "config": {"workload": "hbm: each kernel alone at N=11008, K=4096 (M=4096 for the activation kernels), L2 flushed before "
                               "every launch; value = stand-alone hysteresis update"},
        "roofline": {"bound": "hbm", "achieved": head["GBps"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": head["frac_of_hbm"], "traffic": None, "peak_source": f"hbm_gbs ({peak_kind})"},
        "kernels": out, "gpu_launches": (reps + 3) * len(cases),
    }))


def run_ffn(args):
    """The reference's feed-forward block at the 7B shape through the module API: `w3(silu(w1 x) * w2 x)` with
    d_model 4096 and hidden size 11008 over INT2 layers (SwiGLUFFNInt2), forward + backward + the three weight updates
    per step, M = 4096 tokens.  Timed with the gate fused into the down projection's quantiser and with the gate as tensor
    operations (everything else identical); L2 flushed between steps, inputs resident."""
    import torch
    pkg = load_package()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    peaks, peak_kind = measured_peaks()
    M, D = 4096, 4096
    gen = torch.Generator().manual_seed(11)
    ffn = pkg.SwiGLUFFNInt2(D, threshold=3, hysteresis_order="after_dx").to(dev)
    Hd = ffn.hidden_dim
    for layer in (ffn.w1, ffn.w2, ffn.w3):
        il = layer.int2_layer
        il.init_from_float((torch.randn(il.out_features, il.in_features, generator=gen) * 0.02).to(dev))
        counters = torch.randint(-3, 4, (il.out_features, il.in_features), generator=gen, dtype=torch.int16)
        il.H_packed.copy_(((counters[:, 0::2] & 0xF) | ((counters[:, 1::2] & 0xF) << 4)).to(torch.uint8))
    ffn.train()
    pkg.set_all_int2_lr(ffn, 1e-2)
    x = torch.randn(M, D, generator=gen).to(torch.bfloat16).to(dev).requires_grad_(True)
    dY = (torch.randn(M, D, generator=gen) * 1e-3).to(torch.bfloat16).to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        x.grad = None
        ffn(x).backward(dY)

    def timed(fused):
        ffn.w3.fuse_swiglu = fused
        for _ in range(max(args.warmup, 3)):
            step()
        total = 0.0
        for _ in range(args.steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / args.steps

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    fused_ms = timed(True)
    clocks = sampler.stop()
    unfused_ms = timed(False)
    pkg.int2_tc_ops.check_device_status(dev)
    ops_per_step = 3 * 3 * 2.0 * M * D * Hd
    tops = ops_per_step / (fused_ms * 1e-3) / 1e12
    peak = 2.0 * peaks["bf16_tflops"]
    print(json.dumps({
        "metric": "SwiGLU feed-forward block (3 INT2 layers) fwd+bwd+hysteresis tokens/s at the 7B shape", "value": M / (fused_ms * 1e-3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": fused_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int2 -> int32, bf16 I/O",
        "data": "synthetic",
        "config": {"workload": f"ffn: M={M} tokens, d_model={D}, hidden={Hd}, module API with autograd, L2 flushed between steps",
                   "threshold": 3, "hysteresis_order": "after_dx"},
        "gate_as_tensor_operations": {"ms_per_step": unfused_ms, "tokens_per_s": M / (unfused_ms * 1e-3)},
        "roofline": {"bound": "tensor", "achieved": tops, "peak": peak, "unit": "TOP/s", "frac": tops / peak, "traffic": None,
                     "peak_source": f"2 x bf16_tflops (burst) ({peak_kind}); whole step including quantisers, gate and autograd"},
        "clocks": clocks, "gpu_launches": (args.steps + max(args.warmup, 3)) * 26,
    }))


def run_config1(args):
    env = Env(args)
    res = measure_config1(env, reps=max(args.steps, 10))
    head = res["shapes"][1]
    ceiling = int8_ceiling(env)
    peak = 2.0 * env.peaks["bf16_tflops"]
    print(json.dumps({
        "metric": "forward GEMM TOP/s at M=4096 (BASELINE config 1)", "value": head["tops"], "unit": "TOP/s", "n_gpus": 1,
        "steps": max(args.steps, 10), "warmup": 3, "ms_per_step": head["gemm_ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int2 -> int32 (bf16 out)", "data": "synthetic",
        "config": {"workload": "config1: forward sweep, M=4096, 4096->4096, 4096->11008, 11008->4096, 4096->512; value = 4096->11008"},
        "roofline": {"bound": "tensor", "achieved": head["tops"], "peak": peak, "unit": "TFLOP/s", "frac": head["tops"] / peak,
                     "traffic": None, "peak_source": f"2 x bf16_tflops (burst) ({env.peak_kind})", "int8_ceiling_tops": ceiling},
        "config1": res, "gpu_launches": 4 * 2 * (max(args.steps, 10) + 3),
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config2", choices=sorted(WORKLOADS) + ["config1", "config3", "hbm", "ffn"])
    ap.add_argument("--partition", default="both", choices=["both", "tokens", "features"],
                    help="N > 1: which partition(s) of the step to measure (value = the faster of those measured)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg of the default run")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--e2e-order", default="step", choices=["step", "layer"],
                    help="end-to-end leg: forward through all layers then backward in reverse (a training step), or each "
                         "layer's forward and backward back to back")
    ap.add_argument("--no-config4", action="store_true", help="skip the config-4 sub-record of the default run")
    ap.add_argument("--push-ctas", type=int, default=0,
                    help="token partition: CTAs of the peer-store kernel that pushes tokens and weight rows "
                         "(negative: copy engines; 0: the layer's choice by size)")
    ap.add_argument("--no-graph", action="store_true",
                    help="token partition: queue every launch of the step from the host instead of replaying a recorded CUDA graph")
    ap.add_argument("--brief", action="store_true",
                    help="skip the sub-records measured outside the step (int8 ceiling, configs 1 and 3, reference kernels)")
    ap.add_argument("--inline-kernel-events", action="store_true",
                    help="record the per-kernel event pairs inside the headline region instead of in a second pass")
    args = ap.parse_args()
    if args.workload in ("config1", "config3", "hbm", "ffn"):
        if args.impl == "ours" and int(os.environ.get("RANK", "0")) == 0:
            {"config1": run_config1, "config3": run_decode, "hbm": run_hbm_kernels, "ffn": run_ffn}[args.workload](args)
        return
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
