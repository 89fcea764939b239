"""INT2 linear layer sharded along N (output features) over the GPUs of one node.

Rank r of g owns rows [r*N/g, (r+1)*N/g) of `W_packed` / `H_packed`; activations are replicated (every rank
sees all M tokens).  The reference has no multi-GPU code; this is the sharding its layer admits:

  forward   local Y_r[M, N/g] = Q(X) . W_r^T, then one all-gather -> Y[M, N]
  dX        local int32 partial sums dYq[:, shard] . W_r, summed over ranks (exact: integer addition is
            associative, so the result is bit-identical to one GPU), then scaled once
  dW        local to the shard: no communication; the per-weight random-number counter uses the global
            row index, so the flips equal those of the unsharded layer
  scales    a token's absmax of dY spans all N columns: each rank reduces its column window and a max
            all-reduce of M floats completes it

Collectives go through torch.distributed (NCCL over NVLink on GPUs; gloo in the CPU tests, where a stand-in
for the operator module is injected).  With `fused_gather=True` (CUDA only) the forward all-gather is not a collective
at all: the output of every rank lives in symmetric memory and each rank's GEMM epilogue writes its columns straight
into all ranks' buffers with TMA stores over NVLink (`el_gemm_fwd_gather`), followed by one device-side barrier.  The
dX reduction is fused the same way: the dX epilogue scatters its int32 partial rows to the rank that owns them
(`el_gemm_dx_scatter`), the owner sums, scales and writes its rows of dX into every rank (`el_reduce_scale_gather`).
Every symmetric buffer exists twice and calls alternate between the two, so no barrier guards the reuse of a buffer.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.autograd import Function

from .int2_tc_ops import ACT_EPS, GRAD_EPS

_FLOAT_IO = (torch.float16, torch.bfloat16, torch.float32)


def shard_rows(n_total: int, world: int, rank: int):
    """[start, stop) of the rows rank `rank` owns; N must divide evenly (and by 16 per shard for the
    tensor-core kernels to take the shard)."""
    if n_total % world != 0:
        raise ValueError(f"out_features={n_total} is not divisible by the group size {world}")
    per = n_total // world
    return rank * per, (rank + 1) * per


class _ShardedLinearFn(Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, gamma: torch.Tensor, layer: "ShardedInt2Linear") -> torch.Tensor:
        ops, grp = layer.ops, layer.group
        K, Nl, g, r_ = layer.in_features, layer.local_out_features, layer.world, layer.rank
        io = x.dtype if x.dtype in _FLOAT_IO else torch.bfloat16
        x2 = x.reshape(-1, K)
        Xq, ax = ops.quantize_rows(x2 if x2.dtype in _FLOAT_IO else x2.to(io), ACT_EPS)
        M = x2.shape[0]
        if g > 1 and layer.fused_gather and layer.fused_forward_ok():
            # Two output buffers alternate between calls.  A rank can only start call i+1 after the barrier of call i,
            # by which time every rank has issued (in stream order) its reads of the buffer of call i-1: no barrier is
            # needed before overwriting that buffer.
            buf, hdl = layer._symmetric_output(M, io)
            ops.matmul_rows_gather(Xq, layer.W_packed, ax, layer.gamma_value(), hdl.buffer_ptrs, g * Nl, r_ * Nl, io)
            layer._barrier(hdl, 1)          # every rank's stores into this rank's buffer have landed
            y = buf.clone() if layer.copy_output else buf
            ctx.layer, ctx.io, ctx.x_shape = layer, io, x.shape
            ctx.saved = (Xq, ax) if layer.training else None
            return y.view(*x.shape[:-1], g * Nl)
        y_local = ops.matmul_rows(Xq, layer.W_packed, ax, layer.gamma_value(), io)
        if g > 1:
            gathered = torch.empty(g * M, Nl, dtype=io, device=x.device)     # rank-major concatenation
            dist.all_gather_into_tensor(gathered, y_local.contiguous(), group=grp)
            y = gathered.view(g, M, Nl).permute(1, 0, 2).reshape(M, g * Nl)
        else:
            y = y_local
        ctx.layer, ctx.io, ctx.x_shape = layer, io, x.shape
        ctx.saved = (Xq, ax) if layer.training else None
        return y.view(*x.shape[:-1], g * Nl)

    @staticmethod
    def backward(ctx, dY: torch.Tensor):
        layer = ctx.layer
        ops, grp = layer.ops, layer.group
        K, Nl, g, r = layer.in_features, layer.local_out_features, layer.world, layer.rank
        dY2 = dY.reshape(-1, g * Nl)
        if dY2.dtype not in _FLOAT_IO:
            dY2 = dY2.to(ctx.io)
        window = dY2[:, r * Nl:(r + 1) * Nl]                # this rank's columns, read in place
        if g > 1 and dY2.numel() * dY2.element_size() <= layer.local_absmax_bytes:
            raw = ops.absmax_rows(dY2)      # dY is replicated: for small gradients reading all of it beats a collective
        else:
            raw = ops.absmax_rows(window)
            if g > 1:
                dist.all_reduce(raw, op=dist.ReduceOp.MAX, group=grp)
        do_update = layer.training and layer.hysteresis_enabled and ctx.saved is not None
        if do_update:
            Xq, ax = ctx.saved
            dYq, ady, gmax = ops.quantize_rows(window, GRAD_EPS, fold_absmax=ax, raw_absmax=raw)
        else:
            dYq, ady = ops.quantize_rows(window, GRAD_EPS, raw_absmax=raw)

        def update():
            layer._step_py += 1
            layer._step.fill_(layer._step_py)       # the buffer follows the counter, so a plain state_dict() resumes exactly
            Gq = ops.quantize_grad(window, ax, gmax)
            idx_base = layer.row_start * K
            if ops.dw_hysteresis_supported(Nl, K):
                ops.dw_hysteresis(Gq, Xq, gmax, layer.W_packed, layer.H_packed, layer._lr, layer.lr_scale, layer.threshold,
                                  layer.decay_rate, layer._step_py, idx_base)
            else:
                dW = ops.weight_grad(Gq, Xq, gmax)
                ops.hysteresis_step_v2(dW, layer.W_packed, layer.H_packed, layer._lr, layer.lr_scale, layer.threshold,
                                       layer.decay_rate, layer._step_py, idx_base)

        if do_update and layer.hysteresis_order == "reference":
            update()                                        # as the reference's hook: before dX
        dX = None
        if ctx.needs_input_grad[0]:
            gam = layer.gamma_value()
            M_tok = dY2.shape[0]
            if g > 1 and layer.fused_gather and M_tok % (32 * g) == 0:
                # reduce-scatter of the int32 partial sums as TMA stores from the dX epilogue, then each rank sums
                # and scales the rows it owns and writes them into every rank's dX: no collective kernel
                parts, hp, dxbuf, hd = layer._symmetric_dx(M_tok, ctx.io)     # alternating buffers, as in the forward
                ops.backward_input_scatter(dYq, layer.W_packed, K, hp.buffer_ptrs, r)
                layer._barrier(hp, 3)       # all partial sums of my rows have landed
                if do_update and layer.hysteresis_order != "reference" and layer.overlap_dx:
                    # the owner's sum + scale + gather pass and its barrier run on a side stream, under the local
                    # dW + hysteresis kernel of the main stream
                    main, side = torch.cuda.current_stream(), layer._side_stream()
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        ops.reduce_scale_gather(parts, hd.buffer_ptrs, r, ady, gam, M_tok, K, ctx.io)
                        layer._barrier(hd, 4)
                    update()
                    do_update = False
                    main.wait_stream(side)
                else:
                    ops.reduce_scale_gather(parts, hd.buffer_ptrs, r, ady, gam, M_tok, K, ctx.io)
                    layer._barrier(hd, 4)       # all rows of my dX have landed
                dX = dxbuf.clone() if layer.copy_output else dxbuf
            elif g > 1:
                acc = ops.backward_input_rows(dYq, layer.W_packed, ady, gam, K, torch.int32)
                dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=grp)
                dX = ops.scale_rows(acc, ady, gam, ctx.io)
            else:
                dX = ops.backward_input_rows(dYq, layer.W_packed, ady, gam, K, ctx.io)
            dX = dX.view(ctx.x_shape)
        if do_update and layer.hysteresis_order != "reference":
            update()
        return dX, None, None


class ShardedInt2Linear(nn.Module):
    """One N-shard of an INT2 linear layer.  State names follow Int2LinearTC (`W_packed`, `H_packed`, `gamma`,
    `_step`) with the shard's row count; `ops` is the operator module (the CUDA one by default)."""

    def __init__(self, in_features: int, out_features: int, group: Optional[dist.ProcessGroup] = None, threshold: int = 7,
                 lr_scale: float = 5.0, decay_rate: float = 0.001, hysteresis_order: str = "reference", ops=None,
                 fused_gather: bool = False, copy_output: bool = True, own_barrier: bool = False):
        super().__init__()
        if ops is None:
            from . import int2_tc_ops as ops_mod
            ops = ops_mod
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.in_features = in_features
        self.out_features = out_features
        self.row_start, self.row_stop = shard_rows(out_features, self.world, self.rank)
        self.local_out_features = self.row_stop - self.row_start
        self.threshold, self.lr_scale, self.decay_rate = threshold, lr_scale, decay_rate
        self.hysteresis_order = hysteresis_order
        self.hysteresis_enabled = True
        # fused_gather: forward all-gather as TMA stores from the GEMM epilogue into symmetric memory (CUDA only).
        # copy_output=False hands out the symmetric buffer itself: valid until this layer's forward (backward) after next.
        self.fused_gather = fused_gather
        self.copy_output = copy_output
        # own_barrier: the barriers of the fused path are el_peer_barrier (one small kernel over peer-mapped flags, bounded
        # wait of a few seconds reported through the device status word) instead of the symmetric-memory handle's own
        # barrier.  Measured equal in time (a barrier's time is the wait for the slowest rank); off by default because its
        # bound would turn a rank that is merely seconds late into an error.
        self.own_barrier = own_barrier
        # overlap_dx (fused path, hysteresis_order="after_dx"): the second half of the dX exchange runs on a side stream
        # while the main stream runs the local dW + hysteresis kernel
        self.overlap_dx = True
        self._side = None
        self._flags = None
        self._epoch = 0
        self._symm = {}
        self.local_absmax_bytes = 256 << 20     # below this size every rank scans the whole replicated dY itself
        self._lr = 0.001
        self._step_py = 0
        self._gamma_cached: Optional[float] = None
        self.register_buffer("W_packed", torch.zeros(self.local_out_features, (in_features + 3) // 4, dtype=torch.uint8))
        self.register_buffer("H_packed", torch.zeros(self.local_out_features, (in_features + 1) // 2, dtype=torch.uint8))
        self.gamma = nn.Parameter(torch.ones(1))
        self.register_buffer("_step", torch.tensor(0, dtype=torch.int64))

    def set_lr(self, lr: float):
        self._lr = lr

    def fused_forward_ok(self) -> bool:
        """The epilogue-store all-gather needs the tensor-core kernel (K % 64 == 0) and a shard whose 32-column store
        boxes stay inside its own column window; other shapes take the NCCL all-gather."""
        return self.in_features % 64 == 0 and self.local_out_features % 32 == 0

    def sync_step_buffer(self):
        """Writes the Python step counter into the `_step` buffer (done after every update as well)."""
        self._step.fill_(self._step_py)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        # the random numbers of the next update continue from the restored counter; gamma's cache follows the parameter
        if prefix + "_step" in state_dict:
            self._step_py = int(self._step.item())
        self._gamma_cached = None

    def _side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.W_packed.device)
        return self._side

    def _barrier(self, hdl, channel: int):
        """All ranks have finished the work queued so far (their stores into this rank's buffers have landed)."""
        if not self.own_barrier:
            hdl.barrier(channel=channel)
            return
        if self._flags is None:
            import torch.distributed._symmetric_memory as symm_mem
            flags = symm_mem.empty((max(self.world, 8),), dtype=torch.int32, device=self.W_packed.device)
            flags.zero_()
            fh = symm_mem.rendezvous(flags, self.group if self.group is not None else dist.group.WORLD)
            fh.barrier(channel=0)           # every rank's flags are zero before anybody signals
            self._flags = (flags, fh)
        self._epoch += 1
        self.ops.peer_barrier(self._flags[1].buffer_ptrs, self.rank, self._epoch, self.W_packed.device)

    def _symmetric_output(self, M: int, dtype: torch.dtype):
        """The [M, N] output buffer in symmetric memory and its rendezvous handle (allocated once per shape)."""
        key = (M, dtype)
        if key not in self._symm:
            import torch.distributed._symmetric_memory as symm_mem
            pair = []
            for _ in range(2):
                buf = symm_mem.empty((M, self.out_features), dtype=dtype, device=self.W_packed.device)
                pair.append((buf, symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)))
            self._symm[key] = [pair, 0]
        entry = self._symm[key]
        entry[1] ^= 1
        return entry[0][entry[1]]

    def _symmetric_dx(self, M: int, dtype: torch.dtype):
        """Staging buffer [g, M/g, K] int32 for incoming partial sums, the dX buffer [M, K], and their handles."""
        key = ("dx", M, dtype)
        if key not in self._symm:
            import torch.distributed._symmetric_memory as symm_mem
            grp = self.group if self.group is not None else dist.group.WORLD
            pair = []
            for _ in range(2):
                parts = symm_mem.empty((self.world, M // self.world, self.in_features), dtype=torch.int32, device=self.W_packed.device)
                hp = symm_mem.rendezvous(parts, grp)
                dx = symm_mem.empty((M, self.in_features), dtype=dtype, device=self.W_packed.device)
                hd = symm_mem.rendezvous(dx, grp)
                pair.append((parts, hp, dx, hd))
            self._symm[key] = [pair, 0]
        entry = self._symm[key]
        entry[1] ^= 1
        return entry[0][entry[1]]

    def gamma_value(self) -> float:
        if self._gamma_cached is None:
            self._gamma_cached = self.gamma.detach().item()
        return self._gamma_cached

    def init_from_float(self, weight_full: torch.Tensor, scale: Optional[float] = None):
        """Ternarises this rank's rows of the full [N,K] weight with the scale of the WHOLE matrix."""
        assert weight_full.shape == (self.out_features, self.in_features)
        if scale is None:
            scale = max(weight_full.abs().mean().item(), 1e-5)
        rows = weight_full[self.row_start:self.row_stop].to(self.W_packed.device)
        self.W_packed.copy_(self.ops.ternarize_pack(rows, scale))
        self.gamma.data.fill_(scale)
        self._gamma_cached = scale
        self.H_packed.zero_()

    def load_shard(self, W_packed_full: torch.Tensor, H_packed_full: torch.Tensor, gamma: float):
        """Takes this rank's rows out of an unsharded layer's state."""
        self.W_packed.copy_(W_packed_full[self.row_start:self.row_stop])
        self.H_packed.copy_(H_packed_full[self.row_start:self.row_stop])
        self.gamma.data.fill_(gamma)
        self._gamma_cached = float(gamma)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _ShardedLinearFn.apply(x, self.gamma, self)
