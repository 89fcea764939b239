"""INT2 linear layer run token-parallel over the GPUs of one node.

Every rank keeps a full replica of `W_packed` and runs the forward and dX GEMMs on ITS OWN tokens: the layer's input,
output and input gradient are token-sharded and need no communication at all.  The weight update is split by rows, as in
the N-sharded layer (sharded.py): rank r owns rows [r*N/g, (r+1)*N/g) of `W_packed` / `H_packed`, forms their weight
gradient over ALL tokens and runs their hysteresis update.  For that it receives int8 operands only:

  Xq      the other ranks' quantised tokens            all-gather, int8 [M, K]            (pushed during the forward GEMM)
  gmax    one float per rank (partial maximum)        all-gather of g floats, max taken by the consumer
  Gq      its column window of every rank's folded,   all-to-all, int8 [M, N/g]
          quantised output gradient
  W rows  the updated rows of every other rank        all-gather, uint8 [N, K/4]          (before the next forward)

Against N-sharding (replicated activations, bf16 Y all-gathered, int32 dX partial sums reduced) this moves about a fifth
of the bytes, and the per-token quantisers run on M/g tokens per rank instead of on all of them.  The integers are those
of the single-GPU layer: a token's scales depend on its own row only, the per-tensor gradient maximum is a maximum of
maxima, the weight gradient is an exact int32 sum over all tokens, and the per-weight random numbers use the global row
index.  The reference has no multi-GPU code (README.md:58); the single-GPU contract kept here is
Int2LinearTCFunction's (core/bitnet/int2_linear_tc.py:255-305) with the hook's update
(core/bitnet/int2_linear_tc_offload.py:210-285).

Two data paths.  `fused=False`: torch.distributed collectives (NCCL on GPUs; gloo in the CPU tests, where a stand-in for
the operator module is injected).  `fused=True` (CUDA): no collective kernel moves data; all buffers that peers write
live in symmetric memory and the library's own kernels store into them over NVLink (el_peer_put, el_quantize_grad_scatter),
ordered by el_peer_barrier; pushes of 8 MiB and more per destination go through the copy engines instead
(el_peer_put_dma), so that the GEMM beside them keeps every SM.  Only stores and copies cross NVLink; no kernel loads
from a peer.  `train_step` issues the fused step from a prepared plan and, with `graph_steps=True`, replays it from a
recorded CUDA graph (what changes per step - barrier numbers, the hysteresis step - then lives in device memory).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.autograd import Function

from .int2_tc_ops import ACT_EPS, GRAD_EPS
from .sharded import shard_rows

_FLOAT_IO = (torch.float16, torch.bfloat16, torch.float32)
PUSH_DMA_MIN_BYTES = 8 << 20      # pushes of at least this many bytes per destination go through the copy engines
PUSH_STREAMS = 4                  # side streams a copy-engine push spreads its destinations over
MAX_RECORDED_STEPS = 8            # recorded CUDA graphs kept per (layer, token count): one per distinct (x, dY, settings)


class PeerGroup:
    """The barrier of the fused path, shared by all token-parallel layers of one process group on one device: a flag
    array per rank in symmetric memory and a common epoch counter.  Because the epochs are shared, a barrier that one
    layer queues also serves every other layer that was waiting for "a barrier after my last push"."""

    _cache: dict = {}

    def __init__(self, group, device: torch.device, ops):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.ops, self.device = ops, device
        self.rank = dist.get_rank(self.group)
        self.flags = symm_mem.empty((8,), dtype=torch.int32, device=device)
        self.flags.zero_()
        self.handle = symm_mem.rendezvous(self.flags, self.group)
        self.handle.barrier(channel=0)              # every rank's flags are zero before anybody signals
        self.epoch = 0
        # Side streams for the pushes.  A peer-store kernel runs on the first; copy-engine pushes spread their
        # destinations over all of them, so that several copy engines work at once instead of one copy after the other.
        self.sides = [torch.cuda.Stream(device=device) for _ in range(PUSH_STREAMS)]
        self.side = self.sides[0]
        self.pending = []               # events of the pushes queued on side streams and not yet joined

    @classmethod
    def get(cls, group, device: torch.device, ops) -> "PeerGroup":
        key = (id(group) if group is not None else None, device.index)
        if key not in cls._cache:
            cls._cache[key] = cls(group, device, ops)
        return cls._cache[key]

    def join_side(self) -> None:
        """Pushes queued on the side stream are ordered before whatever the main stream does next (a barrier)."""
        if self.pending:
            main = torch.cuda.current_stream()
            for ev in self.pending:
                main.wait_event(ev)
            self.pending = []

    def barrier(self, word: Optional[torch.Tensor] = None, dst_ptrs=None, dst_offset: int = 0) -> None:
        """All ranks have finished the work queued on their main streams so far - and on the side stream before this
        call - peer stores included.  With `word` (4 bytes) the barrier also delivers it to `dst_offset` of every rank's
        buffer in `dst_ptrs`."""
        self.join_side()
        self.epoch += 1
        if word is None:
            self.ops.peer_barrier(self.handle.buffer_ptrs, self.rank, self.epoch, self.device)
        else:
            self.ops.peer_barrier_put(self.handle.buffer_ptrs, self.rank, self.epoch, self.device, word, dst_ptrs, dst_offset)


def _forward_impl(layer: "TokenParallelInt2Linear", x: torch.Tensor):
    """Quantise this rank's tokens (into its row block of the gathered-token buffer when an update will follow), start
    their all-gather, run the forward GEMM.  Returns (y [Ml, N], saved state for the backward pass or None, I/O dtype)."""
    ops, K = layer.ops, layer.in_features
    io = x.dtype if x.dtype in _FLOAT_IO else torch.bfloat16
    x2 = x.reshape(-1, K)
    if x2.dtype not in _FLOAT_IO:
        x2 = x2.to(io)
    Ml = x2.shape[0]
    will_update = layer.training and layer.hysteresis_enabled
    run = layer._run
    if will_update:
        bufs = layer._exchange_buffers(Ml)
        own = bufs["xq_all"][layer.rank * Ml:(layer.rank + 1) * Ml]         # this rank's rows of the gathered tokens
        Xq, ax = run("quantize_rows", ops.quantize_rows, x2, ACT_EPS, out=own)
    else:
        bufs = None
        Xq, ax = run("quantize_rows", ops.quantize_rows, x2, ACT_EPS)
    layer._weights_ready()                  # the other ranks' updated rows of W_packed have landed
    # The GEMM is queued before the push that runs beside it: queued the other way round, the push kernel took the SMs
    # first and the persistent GEMM's CTA pairs waited for them (the forward launch took three times its own time at
    # eight ranks).  The push only has to start after the quantiser, which the event marks.
    share = will_update and layer.world > 1
    ready = None
    if share and layer._use_fused():
        ready = torch.cuda.Event()
        ready.record()
    y = run("gemm_fwd", ops.matmul_rows, Xq, layer.W_packed, ax, layer.gamma_value(), io, layer._gemm_flags(Ml))
    if share:
        layer._share_tokens(bufs, own, Ml, ready)
    return y, ((bufs, ax) if will_update else None), io


def _backward_impl(layer: "TokenParallelInt2Linear", saved, dY: torch.Tensor, io: torch.dtype, need_dx: bool):
    """Quantise this rank's gradient rows, run the dX GEMM on them and the weight update of this rank's rows, in the
    layer's order.  Returns dX [Ml, K] or None."""
    ops, K, N = layer.ops, layer.in_features, layer.out_features
    run = layer._run
    dY2 = dY.reshape(-1, N)
    if dY2.dtype not in _FLOAT_IO:
        dY2 = dY2.to(io)
    if not dY2.is_contiguous():
        dY2 = dY2.contiguous()
    do_update = saved is not None and layer.training and layer.hysteresis_enabled
    if do_update:
        bufs, ax = saved
        dYq, ady, gloc = run("quantize_rows_dy", ops.quantize_rows, dY2, GRAD_EPS, fold_absmax=ax)
    else:
        dYq, ady = run("quantize_rows_dy", ops.quantize_rows, dY2, GRAD_EPS)

    def input_grad():
        if not need_dx:
            return None
        return run("gemm_dx", ops.backward_input_rows, dYq, layer.W_packed, ady, layer.gamma_value(), K, io, layer._gemm_flags(dYq.shape[0]))

    if do_update and layer.hysteresis_order == "reference":
        layer._update(bufs, dY2, ax, gloc)             # as the reference's hook: before dX ...
        layer._weights_ready()                         # ... which then reads every rank's updated rows
        return input_grad()
    dX = input_grad()
    if do_update:
        layer._update(bufs, dY2, ax, gloc)
    return dX


class _TokenParallelFn(Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, gamma: torch.Tensor, layer: "TokenParallelInt2Linear") -> torch.Tensor:
        y, ctx.saved, ctx.io = _forward_impl(layer, x)
        ctx.layer, ctx.x_shape = layer, x.shape
        return y.view(*x.shape[:-1], layer.out_features)

    @staticmethod
    def backward(ctx, dY: torch.Tensor):
        dX = _backward_impl(ctx.layer, ctx.saved, dY, ctx.io, ctx.needs_input_grad[0])
        return (None if dX is None else dX.view(ctx.x_shape)), None, None


class TokenParallelInt2Linear(nn.Module):
    """One rank of a token-parallel INT2 linear layer.  `W_packed` is the full [N, ceil(K/4)] matrix (a replica per
    rank); `H_packed` holds the counters of the rows this rank updates; `gamma`, `_step` as in Int2LinearTC.  Call it
    with this rank's tokens; every rank must pass the same number of tokens per call."""

    def __init__(self, in_features: int, out_features: int, group: Optional[dist.ProcessGroup] = None, threshold: int = 7,
                 lr_scale: float = 5.0, decay_rate: float = 0.001, hysteresis_order: str = "after_dx", ops=None,
                 fused: bool = False, push_ctas: int = 0, graph_steps: bool = False):
        super().__init__()
        if ops is None:
            from . import int2_tc_ops as ops_mod
            ops = ops_mod
        if hysteresis_order not in ("reference", "after_dx"):
            raise ValueError("hysteresis_order must be 'reference' or 'after_dx'")
        self.ops, self.group = ops, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features, self.out_features = in_features, out_features
        self.row_start, self.row_stop = shard_rows(out_features, self.world, self.rank)
        self.local_out_features = self.row_stop - self.row_start
        self.threshold, self.lr_scale, self.decay_rate = threshold, lr_scale, decay_rate
        self.hysteresis_order = hysteresis_order
        self.hysteresis_enabled = True
        self.fused = fused
        # How the pushes that run on a side stream beside the GEMMs move their bytes.  push_ctas > 0: a peer-store kernel of
        # that many CTAs.  It holds no shared memory, so it sits on the SMs next to the GEMM's CTAs; NVLink needs a few
        # megabytes of stores in flight to run at rate (32 CTAs moved 140-310 GB/s, a fifth of the link), and one CTA per
        # SM is the most that fits: the register-lean GEMM leaves 16 K registers per SM, a push CTA takes 12 K, and with
        # two per SM a GEMM CTA that arrives second finds no room and waits for the whole push.  push_ctas < 0: the copy
        # engines, one copy per destination (el_peer_put_dma): no SM takes part and the GEMM beside it keeps its faster
        # form, but the copies run one after the other at about 10 us each plus their bytes.  0 (default): by size -
        # copy engines from PUSH_DMA_MIN_BYTES per destination on, the kernel with one CTA per SM below.  Measured at
        # eight ranks: 33 MB per destination (65536 tokens): step 1.92 -> 1.64 ms with the copy engines; 2-6 MB per
        # destination (4096 tokens): 0.436 ms with the kernel, 0.463 ms with the copy engines.
        self.push_ctas = push_ctas
        # From four ranks on, the pushes are a large enough share of the step that they must overlap with the GEMMs: next
        # to a push kernel the forward and dX GEMMs run in their register-lean form (EL_FLAG_LEAN), which leaves room on
        # the SMs for it.  With two ranks the faster form wins (measured).
        self._lean = getattr(ops, "EL_FLAG_LEAN", 0) if (fused and self.world >= 4) else 0
        # train_step on the fused path replays a recorded CUDA graph per (input buffers, settings) instead of queueing its
        # launches one by one; for callers that pass the same x and dY buffers every step (see _replayed_step).
        self.graph_steps = graph_steps
        self._lr = 0.001
        self._step_py = 0
        self._gamma_cached: Optional[float] = None
        self._peer: Optional[PeerGroup] = None
        self._w_handle = None
        self._w_ready_epoch = 0                 # fused path: W_packed is complete once the group's epoch has reached this
        self._bufs: dict = {}
        self._plans: dict = {}
        self._step_dirty = False                # the `_step` buffer lags the Python counter (synced when the state is saved)
        self._run = lambda name, fn, *a, **k: fn(*a, **k)       # a benchmark replaces this to time the calls by name
        self.register_buffer("W_packed", torch.zeros(out_features, (in_features + 3) // 4, dtype=torch.uint8))
        self.register_buffer("H_packed", torch.zeros(self.local_out_features, (in_features + 1) // 2, dtype=torch.uint8))
        self.gamma = nn.Parameter(torch.ones(1))
        self.register_buffer("_step", torch.tensor(0, dtype=torch.int64))

    # ---- state -------------------------------------------------------------------------------------------------------
    def set_lr(self, lr: float):
        self._lr = lr

    def gamma_value(self) -> float:
        if self._gamma_cached is None:
            self._gamma_cached = self.gamma.detach().item()
        return self._gamma_cached

    def sync_step_buffer(self):
        self._step.fill_(self._step_py)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        if prefix + "_step" in state_dict:
            self._step_py = int(self._step.item())
        self._gamma_cached = None

    def init_from_float(self, weight_full: torch.Tensor, scale: Optional[float] = None):
        """Ternarises the full [N,K] weight (every rank holds all of it); counters start at zero."""
        assert weight_full.shape == (self.out_features, self.in_features)
        if scale is None:
            scale = max(weight_full.abs().mean().item(), 1e-5)
        self.W_packed.copy_(self.ops.ternarize_pack(weight_full.to(self.W_packed.device), scale))
        self.gamma.data.fill_(scale)
        self._gamma_cached = scale
        self.H_packed.zero_()

    def load_full(self, W_packed_full: torch.Tensor, H_packed_full: torch.Tensor, gamma: float):
        """Takes the state of an unsharded layer: all of its weights, and the counters of this rank's rows."""
        self.W_packed.copy_(W_packed_full)
        self.H_packed.copy_(H_packed_full[self.row_start:self.row_stop])
        self.gamma.data.fill_(gamma)
        self._gamma_cached = float(gamma)

    def owned_rows(self) -> torch.Tensor:
        """The rows of the replica this rank updates (a view)."""
        return self.W_packed[self.row_start:self.row_stop]

    # ---- exchange plumbing ---------------------------------------------------------------------------------------------
    def _push_mode(self, bytes_per_destination: int) -> int:
        """The max_ctas argument of ops.peer_put for a push of that size: negative = copy engines."""
        if self.push_ctas != 0:
            return self.push_ctas
        return -1 if bytes_per_destination >= PUSH_DMA_MIN_BYTES else 148

    def _gemm_flags(self, Ml: int) -> int:
        """Path flags of the forward and dX GEMMs for Ml local tokens: register-lean only beside a push kernel."""
        return self._lean if self._push_mode(Ml * self.in_features) > 0 else 0

    def _queue_push(self, name: str, src: torch.Tensor, dst_ptrs, dst_offset: int, after: Optional[torch.cuda.Event]):
        """Queues the push of the contiguous tensor `src` to `dst_offset` of every buffer in `dst_ptrs` (peers, from the
        successor on) on the side stream(s), after `after` (an event of the main stream; None: after everything queued
        on the main stream so far), and notes the events a later barrier has to wait for."""
        peer, main = self._peer, torch.cuda.current_stream()
        mode = self._push_mode(src.numel() * src.element_size())
        if mode < 0:            # copy engines: destination j goes to side stream j mod PUSH_STREAMS
            groups = [(peer.sides[j], dst_ptrs[j::PUSH_STREAMS]) for j in range(min(PUSH_STREAMS, len(dst_ptrs)))]
        else:
            groups = [(peer.side, list(dst_ptrs))]
        for stream, ptrs in groups:
            if after is not None:
                stream.wait_event(after)
            else:
                stream.wait_stream(main)
            with torch.cuda.stream(stream):
                self._run(name if mode >= 0 else name + "_dma", self.ops.peer_put, src, ptrs, dst_offset, mode)
                ev = torch.cuda.Event()
                ev.record(stream)
            peer.pending.append(ev)

    def _successors(self, ptrs):
        """The peers' entries of `ptrs`, starting with this rank's successor: when every rank pushes in this order, each
        GPU receives from one sender at a time (copy-engine pushes run one destination after the other)."""
        return [ptrs[(self.rank + j) % self.world] for j in range(1, self.world)]

    def _use_fused(self) -> bool:
        return self.fused and self.world > 1 and self.W_packed.is_cuda

    def _symm(self, shape, dtype):
        import torch.distributed._symmetric_memory as symm_mem
        t = symm_mem.empty(shape, dtype=dtype, device=self.W_packed.device)
        return t, symm_mem.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)

    def _fused_setup(self):
        """First use of the fused path (collective: every rank gets here in its first forward): the barrier group, and
        the weight replica moved into symmetric memory so that peers can store their updated rows into it."""
        if self._peer is None:
            self._peer = PeerGroup.get(self.group, self.W_packed.device, self.ops)
            w, self._w_handle = self._symm(tuple(self.W_packed.shape), torch.uint8)
            w.copy_(self.W_packed)
            self._buffers["W_packed"] = w
            self._peer.barrier()

    def _exchange_buffers(self, Ml: int) -> dict:
        """Receive buffers for a call with Ml tokens per rank: the gathered int8 tokens [g*Ml, K], this rank's column
        window of every rank's quantised gradient [g*Ml, N/g], the partial maxima [g] and the reduced maximum [1]."""
        if self._use_fused():
            self._fused_setup()
        if Ml not in self._bufs:
            g, dev = self.world, self.W_packed.device
            if self._use_fused():
                xq_all, hx = self._symm((g * Ml, self.in_features), torch.int8)
                gq_recv, hg = self._symm((g * Ml, self.local_out_features), torch.int8)
                slots, hs = self._symm((8,), torch.float32)
                slots.zero_()
                self._bufs[Ml] = dict(xq_all=xq_all, hx=hx, gq_recv=gq_recv, hg=hg, slots=slots, hs=hs,
                                      gmax=torch.zeros(1, dtype=torch.float32, device=dev))
                self._peer.barrier()            # nobody pushes into buffers that a rank has not created yet
            else:
                self._bufs[Ml] = dict(xq_all=torch.empty(g * Ml, self.in_features, dtype=torch.int8, device=dev))
        return self._bufs[Ml]

    def _weights_ready(self):
        """Before a GEMM reads the replica: the rows the other ranks updated last must have landed.  On the fused path
        that is any barrier queued after this rank's last push; one is queued here only if none has been since."""
        if self._use_fused() and self._peer is not None and self._peer.epoch < self._w_ready_epoch:
            self._run("barrier_weights", self._peer.barrier)

    def _share_tokens(self, bufs: dict, own: torch.Tensor, Ml: int, ready: Optional[torch.cuda.Event] = None):
        """All-gather of the int8 tokens; on the fused path a push to the peers on a side stream, beside the forward GEMM
        (`ready`: recorded on the main stream once the tokens were quantised; without it the push waits for all of the
        main stream's queued work)."""
        if self._use_fused():
            self._queue_push("push_tokens", own, self._successors(bufs["hx"].buffer_ptrs), self.rank * Ml * self.in_features, ready)
        else:
            self._run("all_gather_tokens", dist.all_gather_into_tensor, bufs["xq_all"], own.clone(), group=self.group)

    def _update(self, bufs: dict, dY2: torch.Tensor, ax: torch.Tensor, gloc: torch.Tensor):
        """The weight update of this rank's rows from all ranks' tokens, then the push of the new rows to the replicas."""
        ops, run = self.ops, self._run
        g, r, K, Nl = self.world, self.rank, self.in_features, self.local_out_features
        Ml = dY2.shape[0]
        self._step_py += 1
        self._step.fill_(self._step_py)
        if g == 1:
            gmax = gloc
            gq = run("quantize_grad", ops.quantize_grad, dY2, ax, gmax)
        elif self._use_fused():
            peer = self._peer
            # the barrier carries this rank's partial maximum to slot r of every rank; after it all maxima and (the side
            # stream is joined first) all tokens have landed
            run("barrier_gmax", peer.barrier, gloc, list(bufs["hs"].buffer_ptrs), 4 * r)
            gmax = bufs["gmax"]
            run("quantize_grad", ops.quantize_grad_scatter, dY2, ax, bufs["slots"][:g], list(bufs["hg"].buffer_ptrs), r * Ml, gmax)
            run("barrier_grad", peer.barrier)           # every rank's window of the gradient has landed
            gq = bufs["gq_recv"]
        else:
            gmax = gloc.clone()
            run("all_reduce_gmax", dist.all_reduce, gmax, op=dist.ReduceOp.MAX, group=self.group)
            full = run("quantize_grad", ops.quantize_grad, dY2, ax, gmax)
            send = full.view(Ml, g, Nl).permute(1, 0, 2).contiguous()           # [destination rank, token, window column]
            gq = torch.empty(g * Ml, Nl, dtype=torch.int8, device=full.device)  # [source rank * Ml + token, window column]
            run("all_to_all_grad", dist.all_to_all_single, gq, send, group=self.group)
        own = self.owned_rows()
        idx_base = self.row_start * K
        if ops.dw_hysteresis_supported(Nl, K):
            run("gemm_dw_hysteresis", ops.dw_hysteresis, gq, bufs["xq_all"], gmax, own, self.H_packed, self._lr, self.lr_scale,
                self.threshold, self.decay_rate, self._step_py, idx_base)
        else:
            dW = run("gemm_dw", ops.weight_grad, gq, bufs["xq_all"], gmax)
            run("hysteresis", ops.hysteresis_step_v2, dW, own, self.H_packed, self._lr, self.lr_scale, self.threshold,
                self.decay_rate, self._step_py, idx_base)
        if g == 1:
            return
        if self._use_fused():
            # the updated rows go out on the side stream, under whatever the main stream does until the next barrier
            self._queue_push("push_weights", own, self._successors(self._w_handle.buffer_ptrs),
                             self.row_start * self.W_packed.shape[1], None)
            self._w_ready_epoch = self._peer.epoch + 1          # complete after the next barrier, whoever queues it
        else:
            run("all_gather_weights", dist.all_gather_into_tensor, self.W_packed, own.clone(), group=self.group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _TokenParallelFn.apply(x, self.gamma, self)

    def train_step(self, x: torch.Tensor, dY: torch.Tensor, need_dx: bool = True):
        """Forward, dX and the weight update for this rank's tokens x [Ml, K] with the output gradient dY [Ml, N], without
        the autograd machinery around them (a trainer that schedules the layer itself; the benchmark).  Same kernels, same
        order and same results as `layer(x)` followed by `backward(dY)`.  Returns (y, dX).  On the fused CUDA path the
        step is issued from a prepared plan (buffers allocated once per token count, one library call per kernel), and
        the returned tensors are the plan's own: they are overwritten by the next call with the same token count."""
        if (self._use_fused() and self.training and self.hysteresis_enabled and x.dim() == 2 and dY.dim() == 2
                and x.dtype in _FLOAT_IO and dY.dtype == x.dtype and x.is_contiguous() and dY.is_contiguous()
                and self.ops.dw_hysteresis_supported(self.local_out_features, self.in_features)):
            return self._planned_step(x, dY, need_dx)
        y, saved, io = _forward_impl(self, x)
        dX = _backward_impl(self, saved, dY, io, need_dx)
        return y, dX

    # ---- the fused step from a prepared plan ---------------------------------------------------------------------------
    def _make_plan(self, Ml: int, io: torch.dtype):
        import ctypes
        from types import SimpleNamespace
        ops = self.ops
        lib = ops._lib
        dev = self.W_packed.device
        g, r, K, N, Nl = self.world, self.rank, self.in_features, self.out_features, self.local_out_features
        bufs = self._exchange_buffers(Ml)
        P = SimpleNamespace()
        P.lib, P.bufs, P.dt = lib.lib(), bufs, {torch.float16: lib.EL_F16, torch.bfloat16: lib.EL_BF16, torch.float32: lib.EL_F32}[io]
        P.y = torch.empty(Ml, N, dtype=io, device=dev)
        P.dx = torch.empty(Ml, K, dtype=io, device=dev)
        P.ax = torch.empty(Ml, dtype=torch.float32, device=dev)
        P.ady = torch.empty(Ml, dtype=torch.float32, device=dev)
        P.dyq = torch.empty(Ml, N, dtype=torch.int8, device=dev)
        P.gloc = torch.zeros(1, dtype=torch.float32, device=dev)
        P.step_dev = torch.zeros(1, dtype=torch.int32, device=dev)      # the hysteresis step, for recorded steps
        P.step_dev_value = 0
        P.graphs = {}
        P.warm = False
        P.succ_x, P.succ_w = self._successors(bufs["hx"].buffer_ptrs), self._successors(self._w_handle.buffer_ptrs)
        P.gemm_path = self._gemm_flags(Ml)
        P.own = bufs["xq_all"][r * Ml:(r + 1) * Ml]
        P.status = ops.device_status(dev).data_ptr()
        # scratch for the split reduction of GEMMs with few output tiles (a rank's share of a small batch): see el_gemm_fwd_ws
        need = max(P.lib.el_gemm_workspace_bytes(0, Ml, N, K), P.lib.el_gemm_workspace_bytes(1, Ml, N, K))
        P.ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        P.ws_bytes = need

        def arr(ptrs):
            a = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
            return a, ctypes.cast(a, ctypes.c_void_p)

        P.keep = []
        for name, ptrs in (("all_slots", list(bufs["hs"].buffer_ptrs)), ("all_gq", list(bufs["hg"].buffer_ptrs)),
                           ("flags", list(self._peer.handle.buffer_ptrs))):
            a, c = arr(ptrs)
            P.keep.append(a)
            setattr(P, name, c)
        return P

    def _planned_step(self, x: torch.Tensor, dY: torch.Tensor, need_dx: bool):
        Ml = x.shape[0]
        key = (Ml, x.dtype)
        P = self._plans.get(key)
        if P is None:
            P = self._plans[key] = self._make_plan(Ml, x.dtype)
        if self.graph_steps and P.warm:
            return self._replayed_step(P, x, dY, need_dx)
        P.warm = True        # a plan's first step is always queued launch by launch: first-call set-up cannot be recorded
        return self._issue_step(P, x, dY, need_dx, recorded=False)

    def _replayed_step(self, P, x: torch.Tensor, dY: torch.Tensor, need_dx: bool):
        """The planned step as one CUDA graph per (inputs, settings): recorded on first use, replayed afterwards, so that
        the host queues one launch per step instead of about twenty (at eight ranks and 512 tokens per rank the host
        needed as long to queue a step as the GPU to run it).  What changes from step to step lives in device memory: the
        barriers take their number from the flag array (el_peer_barrier_next), the weight update reads its step from a
        counter that a one-thread kernel advances.  The host mirrors both so that unrecorded calls can be mixed in."""
        peer = self._peer
        need_wbar = peer.epoch < self._w_ready_epoch
        key = (x.data_ptr(), dY.data_ptr(), need_dx, need_wbar, self.gamma_value(), float(self._lr), float(self.lr_scale),
               int(self.threshold), float(self.decay_rate), self.hysteresis_order)
        G = P.graphs.get(key)
        if G is None:
            if len(P.graphs) >= MAX_RECORDED_STEPS:
                # The caller's buffers keep changing (every step a new x or dY address): recording a graph per address
                # would only pile graphs up, so such steps are queued launch by launch.
                return self._issue_step(P, x, dY, need_dx, recorded=False)
            from types import SimpleNamespace
            peer.join_side()                # nothing recorded waits on work queued before the recording
            saved = (peer.epoch, self._step_py, self._w_ready_epoch, self._step_dirty)
            graph = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    y, dx = self._issue_step(P, x, dY, need_dx, recorded=True)
                    peer.join_side()        # the side stream's pushes end inside the recording
                G = SimpleNamespace(graph=graph, y=y, dx=dx, barriers=peer.epoch - saved[0],
                                    w_ready=self._w_ready_epoch - saved[0])
            finally:                        # recording ran nothing: the host's mirrors go back to where they were
                peer.epoch, self._step_py, self._w_ready_epoch, self._step_dirty = saved
                peer.pending = []
            P.graphs[key] = G
        if P.step_dev_value != self._step_py:
            P.step_dev.fill_(self._step_py)
            P.step_dev_value = self._step_py
        peer.join_side()
        G.graph.replay()
        self._step_py += 1
        P.step_dev_value += 1
        self._step_dirty = True
        self._w_ready_epoch = peer.epoch + G.w_ready
        peer.epoch += G.barriers
        return G.y, G.dx

    def _issue_step(self, P, x: torch.Tensor, dY: torch.Tensor, need_dx: bool, recorded: bool):
        Ml = x.shape[0]
        lib, run, peer, bufs = P.lib, self._run, self._peer, P.bufs
        g, r, K, N, Nl = self.world, self.rank, self.in_features, self.out_features, self.local_out_features
        gam = self.gamma_value()
        main = torch.cuda.current_stream()
        st = main.cuda_stream
        W, own_w = self.W_packed.data_ptr(), self.W_packed.data_ptr() + self.row_start * self.W_packed.shape[1]

        def call(name, fn, *a):
            rc = run(name, fn, *a)
            if rc != 0:
                self.ops._lib.check(name, rc)

        def barrier(name, with_gmax=False):
            peer.join_side()
            peer.epoch += 1
            if recorded:        # the barrier's number comes from the flag array: nothing in the launch changes per step
                if with_gmax:
                    call(name, lib.el_peer_barrier_next, P.flags, g, r, P.status, P.gloc.data_ptr(), P.all_slots, 4 * r, st)
                else:
                    call(name, lib.el_peer_barrier_next, P.flags, g, r, P.status, None, None, 0, st)
            elif with_gmax:     # the barrier carries this rank's partial maximum to slot r of every rank
                call(name, lib.el_peer_barrier_put, P.flags, g, r, peer.epoch & 0xFFFFFFFF, P.status, P.gloc.data_ptr(),
                     P.all_slots, 4 * r, st)
            else:
                call(name, lib.el_peer_barrier, P.flags, g, r, peer.epoch & 0xFFFFFFFF, P.status, st)

        # forward: quantise into this rank's rows of the gathered tokens, push them to the peers beside the GEMM
        call("quantize_rows", lib.el_quantize_rows, x.data_ptr(), P.dt, K, P.own.data_ptr(), P.ax.data_ptr(), Ml, K, ACT_EPS, 0,
             None, None, st)
        if peer.epoch < self._w_ready_epoch:
            barrier("barrier_weights")
        ready = torch.cuda.Event()
        ready.record(main)                  # tokens quantised, replica complete: the push may start here ...
        call("gemm_fwd", lib.el_gemm_fwd_ws, P.own.data_ptr(), W, P.y.data_ptr(), P.dt, P.ax.data_ptr(), 1, gam, Ml, N, K,
             P.gemm_path, P.ws.data_ptr(), P.ws_bytes, P.status, st)
        # ... but is queued after the GEMM, so that the GEMM's CTA pairs get their SMs first
        self._queue_push("push_tokens", P.own, P.succ_x, r * Ml * K, ready)
        # backward: quantise the gradient rows (with the fold that yields this rank's partial maximum)
        P.gloc.zero_()
        call("quantize_rows_dy", lib.el_quantize_rows, dY.data_ptr(), P.dt, N, P.dyq.data_ptr(), P.ady.data_ptr(), Ml, N, GRAD_EPS, 0,
             P.ax.data_ptr(), P.gloc.data_ptr(), st)

        def input_grad():
            if need_dx:
                call("gemm_dx", lib.el_gemm_dx_ws, P.dyq.data_ptr(), W, P.dx.data_ptr(), P.dt, P.ady.data_ptr(), 1, gam, Ml, N, K,
                     P.gemm_path, P.ws.data_ptr(), P.ws_bytes, P.status, st)

        def update():
            self._step_py += 1
            self._step_dirty = True
            barrier("barrier_gmax", with_gmax=True)
            call("quantize_grad", lib.el_quantize_grad_scatter, dY.data_ptr(), P.dt, N, P.ax.data_ptr(), bufs["slots"].data_ptr(), g,
                 bufs["gmax"].data_ptr(), P.all_gq, g, r * Ml, Ml, N, st)
            barrier("barrier_grad")
            step32 = self._step_py & 0xFFFFFFFF
            if recorded:
                call("step_counter", lib.el_counter_add, P.step_dev.data_ptr(), 1, st)
                call("gemm_dw_hysteresis", lib.el_dw_hysteresis_step_ptr, bufs["gq_recv"].data_ptr(), bufs["xq_all"].data_ptr(),
                     bufs["gmax"].data_ptr(), own_w, self.H_packed.data_ptr(), float(self._lr), float(self.lr_scale),
                     int(self.threshold), float(self.decay_rate), P.step_dev.data_ptr(), (self.row_start * K) & 0xFFFFFFFF,
                     g * Ml, Nl, K, P.status, st)
            else:
                call("gemm_dw_hysteresis", lib.el_dw_hysteresis, bufs["gq_recv"].data_ptr(), bufs["xq_all"].data_ptr(),
                     bufs["gmax"].data_ptr(), own_w, self.H_packed.data_ptr(), float(self._lr), float(self.lr_scale),
                     int(self.threshold), float(self.decay_rate), step32 - (1 << 32) if step32 >= (1 << 31) else step32,
                     (self.row_start * K) & 0xFFFFFFFF, g * Ml, Nl, K, P.status, st)
            # the updated rows go out on the side stream(s), under the main stream's next work
            self._queue_push("push_weights", self.owned_rows(), P.succ_w, self.row_start * self.W_packed.shape[1], None)
            self._w_ready_epoch = peer.epoch + 1

        if self.hysteresis_order == "reference":
            update()
            barrier("barrier_weights")
            input_grad()
        else:
            input_grad()
            update()
        return P.y, (P.dx if need_dx else None)

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        if self._step_dirty:
            self._step.fill_(self._step_py)
            self._step_dirty = False
        super()._save_to_state_dict(destination, prefix, keep_vars)
