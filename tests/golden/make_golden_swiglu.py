"""Generates tests/golden/swiglu.npz from the reference's own feed-forward expression.

Run where the reference checkout is available (its path in the environment variable REFERENCE_ROOT):

    python tests/golden/make_golden_swiglu.py

What is imported from the reference (nothing is copied into this repository):
  * model/model.py                  SwiGLUFFN.forward: `w3(F.silu(w1(x)) * w2(x))` (:107-108).  The object is made
                                    without its constructor; w1 / w2 are stand-ins that hand out the two halves of a
                                    given [M, 2H] tensor (the outputs of the gate and up projections), w3 is the
                                    normalisation the INT2 layer applies to its input first
  * model/common/bitnet_legacy.py   _RMSNorm (the same expression as _ExtraRMSNorm of
                                    core/bitnet/bitnet_int2_optimized.py:72-86) and BitLinear.activation_quant

For bf16, fp16 and fp32 the file holds gate|up, the norm weight, the upstream gradient, and the reference's
normalised product, its int8-valued tokens, and the autograd gradients of gate|up and of the norm weight; one case
has no norm (w3 = identity).
"""
import importlib.util
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
if not REF:
    raise SystemExit("usage: %s REFERENCE_ROOT   (the checkout of the reference project; or set REFERENCE_ROOT)" % sys.argv[0])


class _Half(nn.Module):
    def __init__(self, which: int):
        super().__init__()
        self.which = which

    def forward(self, x):
        H = x.shape[-1] // 2
        return x[..., self.which * H:(self.which + 1) * H]


def main():
    spec = importlib.util.spec_from_file_location("ref_bitnet_legacy", os.path.join(REF, "model/common/bitnet_legacy.py"))
    legacy = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(legacy)
    sys.path.insert(0, REF)
    from model.model import SwiGLUFFN

    out = {}
    cases = [(16, 64, torch.bfloat16, 1e-6, True), (12, 1024, torch.bfloat16, 1e-6, True), (8, 256, torch.float32, 1e-5, True),
             (12, 512, torch.float16, 1e-6, True), (10, 128, torch.bfloat16, 1e-6, False)]
    for i, (M, H, dt, eps, has_norm) in enumerate(cases):
        g = torch.Generator().manual_seed(300 + i)
        gu = (torch.randn(M, 2 * H, generator=g) * (1.0 + i)).to(dt)
        if i == 1:
            gu[0] = 0.0                                  # an all-zero token
            gu[1, :H] = -30.0                            # a saturated gate: silu -> about -3e-12
            gu[2, :H] = 30.0
        ffn = SwiGLUFFN.__new__(SwiGLUFFN)
        nn.Module.__init__(ffn)
        ffn.w1, ffn.w2 = _Half(0), _Half(1)
        if has_norm:
            ffn.w3 = legacy._RMSNorm(H, eps=eps)
            with torch.no_grad():
                ffn.w3.weight.copy_(1.0 + 0.2 * torch.randn(H, generator=g))
        else:
            ffn.w3 = nn.Identity()
        gy = (torch.randn(M, H, generator=g) * 1e-2).to(dt)
        xin = gu.clone().requires_grad_(True)
        y = ffn(xin)
        y.backward(gy)
        layer = legacy.BitLinear(H, 8, bias=False)
        xq = layer.activation_quant(y.detach())
        a = y.detach().float().abs().max(dim=-1).values.clamp(min=layer.eps)
        q = torch.round(xq.float() * (127.0 / a)[:, None])
        out.update({f"gu{i}": gu.float().numpy(), f"gy{i}": gy.float().numpy(), f"y{i}": y.detach().float().numpy(),
                    f"dgu{i}": xin.grad.float().numpy(), f"q{i}": q.numpy().astype(np.int16), f"absmax{i}": a.numpy(),
                    f"eps{i}": np.float32(eps), f"norm{i}": np.array(has_norm),
                    f"io{i}": np.array({torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dt])})
        if has_norm:
            out.update({f"w{i}": ffn.w3.weight.detach().numpy(), f"dw{i}": ffn.w3.weight.grad.numpy()})
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "swiglu.npz"), **out)
    print("written", os.path.join(HERE, "swiglu.npz"))


if __name__ == "__main__":
    main()
