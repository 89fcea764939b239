"""Model-level drop-in: a miniature of the reference model's block, converted and trained the way the reference's
trainer does it (train.py:1050-1068 conversion, :577-600 accumulation switch, :699-728 per-step learning rate, threshold
and gamma refresh, :784-849 checkpoint), including the awkward projection shapes the model really has (reduction length
16, 48 and 16 output features, a 64-wide latent) and the fused SwiGLU call.  Checks that every INT2 layer steps exactly
once per optimiser step, and that a run resumed from a checkpoint continues bit for bit."""
import io

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint

pytestmark = pytest.mark.gpu
DEV = "cuda"
D, INNER, HID = 256, 512, 768


class _MlaLike(nn.Module):
    """Projections of the reference's latent attention (model/common/mla.py:38-45,177-179), without the attention."""

    def __init__(self):
        super().__init__()
        self.w_q = nn.Linear(D, D, bias=False)
        self.w_kv_down = nn.Linear(D, 64, bias=False)
        self.w_kv_up = nn.Linear(64, 2 * D, bias=False)
        self.embed_gate = nn.Linear(D, 16, bias=False)          # 16 output features
        self.w_out = nn.Linear(D, D, bias=False)

    def forward(self, x):
        kv = self.w_kv_up(self.w_kv_down(x))
        k, v = kv[..., :D], kv[..., D:]
        a = torch.sigmoid((self.w_q(x) * k).mean(-1, keepdim=True)) * v
        g = torch.sigmoid(self.embed_gate(x)).mean(-1, keepdim=True)
        return self.w_out(a * g)


class _MambaLike(nn.Module):
    """Projections of the reference's Mamba block (core/mamba/mamba2.py:136,149-156,171), without the scan."""

    def __init__(self):
        super().__init__()
        self.in_proj = nn.Linear(D, 2 * INNER, bias=False)
        self.x_proj = nn.Linear(INNER, 48, bias=False)           # 48 output features
        self.dt_proj = nn.Linear(16, INNER, bias=True)           # reduction length 16
        self.out_proj = nn.Linear(INNER, D, bias=False)

    def forward(self, x):
        xz = self.in_proj(x)
        h, z = xz[..., :INNER], xz[..., INNER:]
        dt = F.softplus(self.dt_proj(self.x_proj(h)[..., :16].contiguous()))
        return self.out_proj(h * dt * F.silu(z))


class _Ffn(nn.Module):
    """model/model.py:86-108; `fused_gate` is the one-line change that hands the gate to the down projection."""

    def __init__(self, fused_gate):
        super().__init__()
        self.w1, self.w2, self.w3 = nn.Linear(D, HID, bias=False), nn.Linear(D, HID, bias=False), nn.Linear(HID, D, bias=False)
        self.fused_gate = fused_gate

    def forward(self, x):
        if self.fused_gate:
            return self.w3(self.w1(x), up=self.w2(x))
        return self.w3(F.silu(self.w1(x)) * self.w2(x))


class _Mini(nn.Module):
    # None: plain blocks; True / False: every block under torch.utils.checkpoint with that `use_reentrant`
    # (the reference's model wraps its blocks with use_reentrant=False, model/model.py:422-424)
    checkpoint_blocks = None

    def _block(self, block, x):
        if self.checkpoint_blocks is None or not self.training:
            return block(x)
        return torch.utils.checkpoint.checkpoint(block, x, use_reentrant=self.checkpoint_blocks)

    def __init__(self, fused_gate):
        super().__init__()
        self.in_norm = nn.LayerNorm(D)
        self.mla, self.mamba, self.ffn = _MlaLike(), _MambaLike(), _Ffn(fused_gate)
        self.lm_head = nn.Linear(D, 64, bias=False)              # excluded from the conversion by its name

    def forward(self, x):
        x = self.in_norm(x.float()).to(torch.bfloat16)          # the INT2 layers see bfloat16, as under the trainer's autocast
        x = x + self._block(self.mla, x)
        x = x + self._block(self.mamba, x)
        x = x + self._block(self.ffn, x)
        return self.lm_head(x.float())


def _build(pkg, fused_gate):
    torch.manual_seed(1234)
    model = pkg.convert_all_linear_to_int2(_Mini(fused_gate), threshold=2, lr_scale=5.0, decay_rate=0.001, min_size=16,
                                           inplace=True, verbose=False, enable_offload=False).to(DEV)
    assert not model._int2_conversion_stats["errors"]
    return model


class _Trainer:
    """The reference trainer's handling of the INT2 layers, reduced to what touches them."""

    def __init__(self, pkg, model, accum=2):
        self.pkg, self.model, self.accum = pkg, model, accum
        self.int2_layers = pkg.get_int2_layers(model)
        self.opt = torch.optim.AdamW(pkg.get_non_int2_params(model), lr=1e-3)
        self.global_step = 0

    def optimizer_step(self, batches):
        assert len(batches) == self.accum
        self.model.train()
        lr = 0.5 / (1 + self.global_step)
        for layer in self.int2_layers:                       # train.py:699-728
            layer.int2_layer.set_lr(lr)
            layer.int2_layer.threshold = 2 if self.global_step < 2 else 3
            layer.int2_layer._gamma_cached = layer.int2_layer.gamma.detach().item()
        losses = []
        for i, (x, y) in enumerate(batches):                 # train.py:577-600
            (self.pkg.enable_hysteresis if i + 1 >= self.accum else self.pkg.disable_hysteresis)()
            loss = F.cross_entropy(self.model(x).float().view(-1, 64), y.view(-1)) / self.accum
            loss.backward()
            losses.append(float(loss))
        self.pkg.enable_hysteresis()
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        self.global_step += 1
        return losses

    def save(self):                                          # train.py:784-824
        buf = io.BytesIO()
        torch.save({"global_step": self.global_step, "model_state_dict": self.model.state_dict(),
                    "int2_state": self.pkg.checkpoint.collect_int2_state(self.int2_layers),
                    "optimizer_state_dict": self.opt.state_dict()}, buf)
        buf.seek(0)
        return buf

    def load(self, buf):                                     # train.py:826-849
        ck = torch.load(buf, map_location=DEV)
        self.global_step = ck["global_step"]
        self.model.load_state_dict(ck["model_state_dict"])
        self.opt.load_state_dict(ck["optimizer_state_dict"])
        self.pkg.checkpoint.sync_after_load(self.int2_layers)
        return ck


def _batches(seed, n):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(4, 32, D, generator=g).to(torch.bfloat16).to(DEV), torch.randint(0, 64, (4, 32), generator=g).to(DEV))
            for _ in range(n)]


@pytest.mark.parametrize("fused_gate", [True, False])
def test_converted_block_trains_and_resumes_bit_for_bit(pkg, fused_gate):
    model = _build(pkg, fused_gate)
    tr = _Trainer(pkg, model)
    names = {n for n, m in model.named_modules() if isinstance(m, pkg.BitLinearInt2)}
    assert names == {"mla.w_q", "mla.w_kv_down", "mla.w_kv_up", "mla.embed_gate", "mla.w_out", "mamba.in_proj", "mamba.x_proj",
                     "mamba.dt_proj", "mamba.out_proj", "ffn.w1", "ffn.w2", "ffn.w3"}
    assert isinstance(model.lm_head, nn.Linear)
    before = [(l.int2_layer.W_packed.clone(), l.int2_layer.H_packed.clone()) for l in tr.int2_layers]
    for s in range(2):
        losses = tr.optimizer_step(_batches(10 + s, 2))
        assert all(l == l and abs(l) < 1e4 for l in losses)
    torch.cuda.synchronize()
    pkg.int2_tc_ops.check_device_status(torch.device(DEV))
    # one update per optimiser step and layer: the accumulation micro-batch left the weights alone
    assert all(l.int2_layer._step_py == 2 for l in tr.int2_layers)
    flipped = [not torch.equal(b[0], l.int2_layer.W_packed) for b, l in zip(before, tr.int2_layers)]
    counted = [not torch.equal(b[1], l.int2_layer.H_packed) for b, l in zip(before, tr.int2_layers)]
    assert sum(counted) >= 10 and sum(flipped) >= 3, (counted, flipped)

    # checkpoint, restore into a freshly built model, continue both: identical from then on
    buf = tr.save()
    model2 = _build(pkg, fused_gate)
    tr2 = _Trainer(pkg, model2)
    ck = tr2.load(buf)
    assert set(ck["int2_state"]) == {f"layer_{i}" for i in range(12)}
    for a, b in zip(tr.int2_layers, tr2.int2_layers):
        assert b.int2_layer._step_py == 2 and torch.equal(a.int2_layer.W_packed, b.int2_layer.W_packed)
        assert torch.equal(a.int2_layer.H_packed, b.int2_layer.H_packed)
    nxt = _batches(99, 2)
    l1, l2 = tr.optimizer_step(nxt), tr2.optimizer_step(nxt)
    torch.cuda.synchronize()
    assert l1 == l2
    for a, b in zip(tr.int2_layers, tr2.int2_layers):
        assert a.int2_layer._step_py == 3 and b.int2_layer._step_py == 3
        assert torch.equal(a.int2_layer.W_packed, b.int2_layer.W_packed) and torch.equal(a.int2_layer.H_packed, b.int2_layer.H_packed)
    for (n, p), (_, q) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(p, q), n

    # the int2_state route restores the same layers as the state dict
    model3 = _build(pkg, fused_gate)
    layers3 = pkg.get_int2_layers(model3)
    buf.seek(0)
    pkg.checkpoint.load_int2_state(layers3, torch.load(buf, map_location="cpu")["int2_state"])
    ref_state = torch.load(io.BytesIO(buf.getvalue()), map_location="cpu")["int2_state"]
    for i, l in enumerate(layers3):
        assert torch.equal(l.int2_layer.W_packed.cpu(), ref_state[f"layer_{i}"]["W_packed"]) and l.int2_layer._step_py == 2


@pytest.mark.parametrize("tokens", [(2, 16), (4, 32)])          # 32 tokens per call (decode-sized) and 128
@pytest.mark.parametrize("use_reentrant", [False, True])
def test_blocks_under_activation_checkpointing_train_like_plain_blocks(pkg, use_reentrant, tokens):
    """Per-block activation checkpointing runs every layer's forward twice.  With use_reentrant=False (what the
    reference's model uses) both passes record gradients and the recompute starts inside the backward pass, after the
    last layer's update hook has already fired; with use_reentrant=True the first pass runs without gradient recording
    (calls of at most 64 tokens then take the decode kernels and save nothing) and the hook exists only on the recompute
    pass (core/bitnet/int2_linear_tc_offload.py:338-344).  With use_reentrant=False two optimiser steps with accumulation
    must leave the same losses, packed weights, counters, step counters and other parameters as the same model without
    checkpointing, bit for bit; with use_reentrant=True the first step's losses are identical and the state agrees up
    to the reordering of bfloat16 gradient sums that this form of checkpointing brings."""
    B, T = tokens

    def batches(seed):
        g = torch.Generator().manual_seed(seed)
        return [(torch.randn(B, T, D, generator=g).to(torch.bfloat16).to(DEV), torch.randint(0, 64, (B, T), generator=g).to(DEV))
                for _ in range(2)]

    plain, ckpt = _build(pkg, True), _build(pkg, True)
    ckpt.checkpoint_blocks = use_reentrant
    tp, tc = _Trainer(pkg, plain), _Trainer(pkg, ckpt)
    for s in range(2):
        lp, lc = tp.optimizer_step(batches(40 + s)), tc.optimizer_step(batches(40 + s))
        if not use_reentrant or s == 0:
            assert lp == lc, (s, lp, lc)            # same forward, same kernels (decode kernels included): same losses
        else:
            assert all(abs(a - b) <= 5e-3 * abs(a) for a, b in zip(lp, lc)), (s, lp, lc)
    torch.cuda.synchronize()
    pkg.int2_tc_ops.check_device_status(torch.device(DEV))
    changed = 0
    for a, b in zip(tp.int2_layers, tc.int2_layers):
        assert a.int2_layer._step_py == 2 and b.int2_layer._step_py == 2
        if not use_reentrant:
            assert torch.equal(a.int2_layer.W_packed, b.int2_layer.W_packed) and torch.equal(a.int2_layer.H_packed, b.int2_layer.H_packed)
        else:
            # The re-entrant form hands a block's input gradient back as one tensor, so the bfloat16 sums of the gradients
            # that meet at a block input are taken in another order than in the plain graph: the gradients reaching the
            # earlier blocks differ in their last bit here and there, and with them a few counters.
            assert float((a.int2_layer.H_packed != b.int2_layer.H_packed).float().mean()) < 0.01
            assert float((a.int2_layer.W_packed != b.int2_layer.W_packed).float().mean()) < 0.01
        changed += int(bool((a.int2_layer.H_packed != 0).any()))
    assert changed >= 10
    if use_reentrant:
        return
    for (n, p), (_, q) in zip(plain.named_parameters(), ckpt.named_parameters()):
        assert torch.equal(p, q), n
