"""Benchmark of the INT2 linear layer step on B200: forward + dX + dW/hysteresis tokens per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload config2|config4|config3|hbm|ffn]

One "step" is one pass of the hot path over one batch of synthetic tokens: for every layer of the workload,
per-token int8 quantisation of the activations, the forward GEMM, per-token quantisation of the output gradient,
the dX GEMM, and the weight-gradient GEMM fused with the hysteresis update of the packed weights and counters.

  config2 (default)  M = 4096 tokens through the two 7B MLP projections 4096->11008 and 11008->4096,
                     counters seeded uniformly in [-3, 3], threshold 3, dY ~ N(0, 1e-3)
  config4            M = 65536 tokens through one 4096->16384 projection

With N > 1 (launched by torch.distributed.run, one rank per GPU) the weights are sharded along N; the output is
all-gathered and the dX partial sums are all-reduced with NCCL (strong scaling: the problem is fixed).

Rank 0 prints one JSON line.  `value` is timed with CUDA events, inputs resident in HBM, L2 flushed between
steps; `e2e` goes through the module API with pinned host buffers copied in every step; `--impl reference`
times the CPU port of the reference layer (oracle/cpu_baseline.py) instead.
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

def cpu_baseline_sample(wl, steps: int, warmup: int, sample_tokens: int):
    import torch
    from oracle import cpu_baseline as cb
    from oracle import native
    native.build_oracle_lib()
    layers = [cb.CpuLayer(K, N, torch.bfloat16, seed=i, counters=wl["counters"]) for i, (K, N) in enumerate(wl["layers"])]
    times, spent = [], 0.0
    for i in range(warmup + steps):
        full, cpu_s = cb.time_step(layers, wl["M"], sample_tokens, torch.bfloat16, lr=LR, threshold=wl["threshold"], seed=i)
        spent += cpu_s
        if i >= warmup:
            times.append(full)
    sec = sum(times) / len(times)
    return {
        "value": wl["M"] / sec, "unit": "tokens/s", "cores": cb.cores_used(), "kind": "port",
        "sample": (f"{steps} steps after {warmup} warm-up; forward+dX+dW (torch, bf16) on {sample_tokens} of "
                   f"{wl['M']} tokens per step scaled to {wl['M']}, plus the hysteresis update of every weight"),
        "ms_per_step": sec * 1e3, "cpu_seconds_spent": spent,
    }


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # one CPU step takes about 1.7 s on 16 cores: K steps as asked, bounded so that the run stays within a few minutes
    steps, warmup = max(1, min(args.steps, 60)), max(1, min(args.warmup, 3))
    base = cpu_baseline_sample(wl, steps, warmup, sample_tokens=min(512, wl["M"]))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (CPU torch) + int (hysteresis)", "data": "synthetic",
        "config": {"workload": wl["desc"], "M": wl["M"], "layers": wl["layers"]},
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


def run_ours(args, wl):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = load_package()
    ops = pkg.int2_tc_ops
    if not os.path.exists(pkg.LIB_PATH):
        raise SystemExit("libelleci_int2.so is not built; there is no fallback path")

    M, thr = wl["M"], wl["threshold"]
    gen = torch.Generator().manual_seed(1234)

    # ---- state: one (sharded) layer per projection ------------------------------------------------------------
    class L:
        pass

    layers = []
    for li, (K, N) in enumerate(wl["layers"]):
        lay = L()
        lay.K, lay.N = K, N
        lay.n0, lay.n1 = pkg.sharded.shard_rows(N, world, rank)
        lay.Nl = lay.n1 - lay.n0
        Wl = torch.randn(lay.Nl, K, generator=torch.Generator().manual_seed(100 + li * 16 + rank)) * 0.02
        lay.gamma = 0.0160
        lay.Wp = ops.ternarize_pack(Wl.to(dev), lay.gamma)
        h = torch.randint(-wl["counters"], wl["counters"] + 1, (lay.Nl, K), generator=gen, dtype=torch.int8)
        hb = (h & 0xF).to(torch.uint8).view(lay.Nl, K // 2, 2)
        lay.Hp = (hb[:, :, 0] | (hb[:, :, 1] << 4)).to(dev).contiguous()
        lay.W0, lay.H0 = lay.Wp.clone(), lay.Hp.clone()
        lay.x = torch.randn(M, K, generator=gen).to(torch.bfloat16).to(dev)
        lay.dY = (torch.randn(M, N, generator=gen) * wl["dy_std"]).to(torch.bfloat16).to(dev)
        lay.step = 0
        lay.symm = None
        if world > 1 and not args.no_fused_gather:
            import torch.distributed._symmetric_memory as symm_mem
            # two sets of buffers alternate between steps, which removes the barriers that would otherwise guard reuse
            lay.flags = symm_mem.empty((8,), dtype=torch.int32, device=dev)
            lay.flags.zero_()
            lay.flags_hdl = symm_mem.rendezvous(lay.flags, dist.group.WORLD)
            lay.flags_hdl.barrier(channel=0)
            lay.epoch = 0
            lay.symm, lay.symm_dx = [], []
            for _ in range(2):
                ybuf = symm_mem.empty((M, N), dtype=torch.bfloat16, device=dev)
                lay.symm.append((ybuf, symm_mem.rendezvous(ybuf, dist.group.WORLD)))
                parts = symm_mem.empty((world, M // world, K), dtype=torch.int32, device=dev)
                dxbuf = symm_mem.empty((M, K), dtype=torch.bfloat16, device=dev)
                lay.symm_dx.append((parts, symm_mem.rendezvous(parts, dist.group.WORLD), dxbuf,
                                    symm_mem.rendezvous(dxbuf, dist.group.WORLD)))
        layers.append(lay)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the 126 MB L2
    timer = Timer(torch)

    def peer_barrier(lay, hdl, channel):
        if not args.own_barrier:
            hdl.barrier(channel=channel)
        else:
            lay.epoch += 1
            ops.peer_barrier(lay.flags_hdl.buffer_ptrs, rank, lay.epoch, dev)

    overlap_dx = world > 1 and not args.no_overlap_dx
    side = torch.cuda.Stream(device=dev) if overlap_dx else None

    def layer_step(lay):
        """One layer: forward, then the weight update and dX (update first, as the reference's hook does; with several
        GPUs dX first, so that its exchange can run under the update)."""
        K, Nl = lay.K, lay.Nl
        Xq, ax = timer.run("quantize_rows", ops.quantize_rows, lay.x)
        if lay.symm is not None:
            # forward GEMM fused with the all-gather: the epilogue stores into every rank's Y over NVLink
            ybuf, hdl = lay.symm[lay.step & 1]
            timer.run("gemm_fwd", ops.matmul_rows_gather, Xq, lay.Wp, ax, lay.gamma, hdl.buffer_ptrs, lay.N, lay.n0, torch.bfloat16)
            timer.run("barrier_post", peer_barrier, lay, hdl, 1)
            y = ybuf
        else:
            y = timer.run("gemm_fwd", ops.matmul_rows, Xq, lay.Wp, ax, lay.gamma, torch.bfloat16)
        if world > 1 and lay.symm is None:
            gathered = torch.empty(world * M, Nl, dtype=torch.bfloat16, device=dev)
            timer.run("all_gather_y", dist.all_gather_into_tensor, gathered, y)
            y = timer.run("permute_y", lambda t: t.view(world, M, Nl).permute(1, 0, 2).reshape(M, world * Nl), gathered)
        window = lay.dY[:, lay.n0:lay.n1] if world > 1 else lay.dY
        if world > 1 and lay.dY.numel() * 2 <= (256 << 20):
            raw = timer.run("absmax_rows", ops.absmax_rows, lay.dY)      # replicated dY: scan all of it, no collective
            dYq, ady, gmax = timer.run("quantize_rows_dy", ops.quantize_rows, window, ops.GRAD_EPS, ax, raw)
        elif world > 1:
            raw = timer.run("absmax_rows", ops.absmax_rows, window)
            timer.run("all_reduce_absmax", dist.all_reduce, raw, op=dist.ReduceOp.MAX)
            dYq, ady, gmax = timer.run("quantize_rows_dy", ops.quantize_rows, window, ops.GRAD_EPS, ax, raw)
        else:
            dYq, ady, gmax = timer.run("quantize_rows_dy", ops.quantize_rows, window, ops.GRAD_EPS, ax)
        lay.step += 1

        def update():
            Gq = timer.run("quantize_grad", ops.quantize_grad, window, ax, gmax)
            timer.run("gemm_dw_hysteresis", ops.dw_hysteresis, Gq, Xq, gmax, lay.Wp, lay.Hp, LR, LR_SCALE, thr, DECAY, lay.step,
                      lay.n0 * K)

        if lay.symm is not None and overlap_dx:
            # Order "forward, dX, weight update": the dX GEMM scatters its int32 partial sums to the owners (epilogue TMA
            # stores); after the barrier the owner's sum + scale + gather pass and its barrier run on a side stream, under
            # the local dW + hysteresis kernel of the main stream.
            parts, hp, dxbuf, hd = lay.symm_dx[lay.step & 1]
            timer.run("gemm_dx", ops.backward_input_scatter, dYq, lay.Wp, K, hp.buffer_ptrs, rank)
            timer.run("barrier_dx1", peer_barrier, lay, hp, 3)
            main = torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                timer.run("reduce_scale_gather", ops.reduce_scale_gather, parts, hd.buffer_ptrs, rank, ady, lay.gamma, M, K, torch.bfloat16)
                timer.run("barrier_dx2", peer_barrier, lay, hd, 4)
            update()
            main.wait_stream(side)
            dX = dxbuf
        elif lay.symm is not None:
            # reference order: the weight update first, then dX with the scatter / sum / gather in sequence
            update()
            parts, hp, dxbuf, hd = lay.symm_dx[lay.step & 1]
            timer.run("gemm_dx", ops.backward_input_scatter, dYq, lay.Wp, K, hp.buffer_ptrs, rank)
            timer.run("barrier_dx1", peer_barrier, lay, hp, 3)
            timer.run("reduce_scale_gather", ops.reduce_scale_gather, parts, hd.buffer_ptrs, rank, ady, lay.gamma, M, K, torch.bfloat16)
            timer.run("barrier_dx2", peer_barrier, lay, hd, 4)
            dX = dxbuf
        elif world > 1:
            update()
            acc = timer.run("gemm_dx", ops.backward_input_rows, dYq, lay.Wp, ady, lay.gamma, K, torch.int32)
            timer.run("all_reduce_dx", dist.all_reduce, acc)
            dX = timer.run("scale_rows", ops.scale_rows, acc, ady, lay.gamma, torch.bfloat16)
        else:
            update()
            dX = timer.run("gemm_dx", ops.backward_input_rows, dYq, lay.Wp, ady, lay.gamma, K, torch.bfloat16)
        return y, dX

    def device_step():
        for lay in layers:
            layer_step(lay)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up ---------------------------------------------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        device_step()
    barrier()
    ops.check_device_status(dev)

    # ---- timed region: K steps, one event pair per step, L2 flushed (untimed) between steps -------------------------
    sampler = ClockSampler(local_rank)
    timer.enabled = args.inline_kernel_events
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    sampler.start()
    for i in range(args.steps):
        flush.zero_()
        ev[i][0].record()
        device_step()
        ev[i][1].record()
    barrier()
    clocks = sampler.stop()
    timer.enabled = False
    total_ms = sum(a.elapsed_time(b) for a, b in ev)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ops.check_device_status(dev)
    ms_per_step = total_ms / args.steps
    value = M / (ms_per_step * 1e-3)
    if not args.inline_kernel_events:
        # The per-kernel event pairs (roofline, breakdown) come from a second pass of the same K steps: inside the
        # headline region the 24 extra event records per step cost about 5 % of it.
        timer.enabled = True
        for i in range(args.steps):
            flush.zero_()
            device_step()
        barrier()
        timer.enabled = False
    kernel_totals = timer.totals()

    # flips actually realised by the first timed update (workload sanity, reported in config)
    lay0 = layers[0]
    w_now = torch.empty(lay0.Nl, lay0.K, dtype=torch.int8, device=dev)
    w_was = torch.empty_like(w_now)
    ops.unpack_int2(lay0.Wp, w_now, lay0.K)
    ops.unpack_int2(lay0.W0, w_was, lay0.K)
    changed_frac = float((w_now != w_was).float().mean().item())

    # ---- end to end through the module API, inputs in pinned host memory ------------------------------------------
    e2e = None
    if world == 1 and not args.no_e2e:
        mods = []
        for lay in layers:
            m = pkg.Int2LinearTCWithGradHook(lay.K, lay.N, threshold=thr, lr_scale=LR_SCALE, decay_rate=DECAY).to(dev)
            m.W_packed.copy_(lay.W0)
            m.H_packed.copy_(lay.H0)
            m.gamma.data.fill_(lay.gamma)
            m._gamma_cached = lay.gamma
            m._initialized = True
            m.set_lr(LR)
            m.train()
            mods.append((m, lay.x.cpu().pin_memory(), lay.dY.cpu().pin_memory()))
        out_host = torch.empty(layers[-1].K, dtype=torch.bfloat16).pin_memory()
        h2d = sum(x.numel() * 2 + dy.numel() * 2 for _, x, dy in mods)
        d2h = out_host.numel() * 2

        copy_stream = torch.cuda.Stream(device=dev)

        def e2e_step():
            # the host->device copies of both layers go out on a copy stream at the start of the step, so the second
            # layer's inputs cross PCIe while the first layer computes; each layer waits for its own inputs only
            main = torch.cuda.current_stream()
            copy_stream.wait_stream(main)                  # copies start inside the timed region
            staged = []
            with torch.cuda.stream(copy_stream):
                for m, xh, dyh in mods:
                    x = xh.to(dev, non_blocking=True)
                    dy = dyh.to(dev, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(copy_stream)
                    staged.append((m, x, dy, ev))
            dx = None
            for m, x, dy, ev in staged:
                main.wait_event(ev)
                x.record_stream(main)
                dy.record_stream(main)
                x.requires_grad_(True)
                y = m(x)
                y.backward(dy)
                dx = x.grad
            out_host.copy_(dx[0], non_blocking=True)

        e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        ee = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(e_steps)]
        for i in range(e_steps):
            flush.zero_()
            ee[i][0].record()
            e2e_step()
            ee[i][1].record()
        torch.cuda.synchronize()
        e_ms = sum(a.elapsed_time(b) for a, b in ee) / e_steps
        e2e = {"value": M / (e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e_ms, "steps": e_steps}
        ops.check_device_status(dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel (the tcgen05 GEMM in its three modes) ---------------------------------------
    peaks, peak_kind = measured_peaks()
    gemm_ops = sum(2.0 * M * (lay.Nl) * lay.K for lay in layers)           # per GEMM mode per step, this rank
    gemm_ms = sum(kernel_totals[n][0] for n in ("gemm_fwd", "gemm_dx", "gemm_dw_hysteresis"))
    gemm_launches = sum(kernel_totals[n][1] for n in ("gemm_fwd", "gemm_dx", "gemm_dw_hysteresis"))
    achieved = 3.0 * gemm_ops * args.steps / (gemm_ms * 1e-3) / 1e12
    int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    # DRAM bytes per GEMM launch from the ncu capture summarised in profiles/gemm_tc2_fwd_dx_config2_ncu_full.md
    # (mean of the forward, dX and dW+hysteresis launches of the 4096->11008 layer at M=4096)
    traffic = 91.3e6 if args.workload == "config2" and world == 1 else None
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s", "frac": achieved / int8_peak,
        "traffic": traffic, "kernel": "gemm_tc_kernel (tcgen05 kind::i8; forward, dX and dW+hysteresis launches)",
        "launches": gemm_launches, "avg_launch_ms": gemm_ms / max(gemm_launches, 1),
        "timing": ("CUDA event pair around every launch, " + ("inside the headline region" if args.inline_kernel_events else
                   "second pass of the same K steps right after the headline region (the headline has one pair per step)")),
        "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_kind}); nominal dense INT8 is 4500",
        "frac_of_nominal_int8": achieved / 4500.0,
    }
    per_mode = {}
    for n in ("gemm_fwd", "gemm_dx", "gemm_dw_hysteresis"):
        ms, cnt = kernel_totals[n]
        per_mode[n] = {"ms_per_launch": ms / cnt, "tops": gemm_ops * args.steps / (ms * 1e-3) / 1e12}
    hbm = {}
    bytes_per_step = {
        "quantize_rows": sum(M * lay.K * 3 + 4 * M for lay in layers),
        "quantize_rows_dy": sum(M * lay.Nl * 3 + 8 * M for lay in layers),
        "quantize_grad": sum(M * lay.Nl * 3 + 4 * M for lay in layers),
    }
    for n, b in bytes_per_step.items():
        if n in kernel_totals:
            ms, cnt = kernel_totals[n]
            gbs = b * args.steps / (ms * 1e-3) / 1e9
            hbm[n] = {"ms_per_launch": ms / cnt, "GBps": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"]}
    comm = {n: {"ms_per_step": kernel_totals[n][0] / args.steps} for n in kernel_totals
            if n.startswith("all_") or n.startswith("barrier_") or n in ("permute_y", "scale_rows", "absmax_rows", "reduce_scale_gather")}

    pre_norm = measure_pre_norm(torch, pkg, M, layers[0].K, dev, flush, peaks) if world == 1 else None
    cpu = cpu_baseline_sample(wl, steps=2, warmup=1, sample_tokens=min(512, M)) if world == 1 and not args.no_cpu else None

    own_launches = sum(cnt for n, (ms, cnt) in kernel_totals.items()
                       if not n.startswith("all_") and not n.startswith("barrier_") and n != "permute_y")
    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 x int2 -> int32 (bf16 in/out)", "data": "synthetic",
        "config": {"workload": wl["desc"], "M": M, "layers": wl["layers"], "threshold": thr,
                   "parallelism": (f"N-sharded x{world}, " + ("Y all-gathered and dX all-reduced by NCCL" if args.no_fused_gather else
                                                              "Y gathered and dX partial sums reduce-scattered by TMA stores from "
                                                              "the GEMM epilogues, dX rows summed and re-gathered by peer stores"
                                                              + ("" if args.no_overlap_dx else " on a side stream under the local dW + hysteresis"))
                                   ) if world > 1 else "single GPU",
                   "l2": "256 MiB written between timed steps (untimed)", "weights_changed_after_run": changed_frac},
        "clocks": clocks, "e2e": e2e, "gpu_launches": own_launches,
        "roofline": roofline, "gemm_modes": per_mode, "hbm_kernels": hbm,
    }
    if comm:
        line["collectives"] = comm
    if pre_norm is not None:
        line["pre_norm"] = pre_norm
    if cpu is not None:
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


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
        for M, gemv_max, mma_max, overlap in ((1, 1, 32, False), (1, 1, 32, True), (1, 0, 32, True), (2, 2, 32, True),
                                              (2, 1, 32, True), (4, 4, 32, True), (4, 1, 32, False), (4, 1, 32, True),
                                              (8, 8, 32, True), (8, 1, 32, False), (8, 1, 32, True), (8, 0, 0, False),
                                              (16, 1, 32, True), (32, 1, 32, True), (32, 1, 0, False), (64, 1, 32, False)):
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
            fits_mma = M <= mma_max and M * K <= 190 * 1024 * (M / (8 if M <= 8 else 16 if M <= 16 else 32))
            kernel = "gemv" if M <= gemv_max else ("mma" if fits_mma else "tcgen05")
            cases.append({"M": M, "K": K, "N": N, "kernel": kernel, "overlap": overlap, "us_per_call": us, "GBps": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"],
                          "algorithmic_bytes": nbytes})
        ops.check_device_status(dev)
        del Ws
    pkg._lib.lib().el_set_decode_gemv_max_tokens(2)
    pkg._lib.lib().el_set_decode_mma_max_tokens(32)
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
    peak = 2.0 * peaks["bf16_tflops_sustained"]
    print(json.dumps({
        "metric": "SwiGLU feed-forward block (3 INT2 layers) fwd+bwd+hysteresis tokens/s at the 7B shape", "value": M / (fused_ms * 1e-3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": fused_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int2 -> int32, bf16 I/O",
        "data": "synthetic",
        "config": {"workload": f"ffn: M={M} tokens, d_model={D}, hidden={Hd}, module API with autograd, L2 flushed between steps",
                   "threshold": 3, "hysteresis_order": "after_dx"},
        "gate_as_tensor_operations": {"ms_per_step": unfused_ms, "tokens_per_s": M / (unfused_ms * 1e-3)},
        "roofline": {"bound": "tensor", "achieved": tops, "peak": peak, "unit": "TOP/s", "frac": tops / peak, "traffic": None,
                     "peak_source": f"2 x bf16_tflops_sustained ({peak_kind}); whole step including quantisers, gate and autograd"},
        "clocks": clocks, "gpu_launches": (args.steps + max(args.warmup, 3)) * 26,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config2", choices=sorted(WORKLOADS) + ["config3", "hbm", "ffn"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg of the default run")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--inline-kernel-events", action="store_true",
                    help="record the per-kernel event pairs inside the headline region instead of in a second pass")
    ap.add_argument("--no-overlap-dx", action="store_true",
                    help="N > 1: keep the reference order (update, then dX) with the dX exchange in sequence")
    ap.add_argument("--own-barrier", action="store_true",
                    help="N > 1: use el_peer_barrier instead of the symmetric-memory handle's barrier (same speed)")
    ap.add_argument("--no-fused-gather", action="store_true",
                    help="N > 1: all-gather the output with NCCL instead of TMA stores from the GEMM epilogue")
    args = ap.parse_args()
    if args.workload in ("config3", "hbm", "ffn"):
        if args.impl == "ours" and int(os.environ.get("RANK", "0")) == 0:
            {"config3": run_decode, "hbm": run_hbm_kernels, "ffn": run_ffn}[args.workload](args)
        return
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
