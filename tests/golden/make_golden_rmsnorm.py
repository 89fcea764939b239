"""Generates tests/golden/rmsnorm.npz from the reference's own pre-linear RMSNorm.

Run where the reference checkout is available (its path as the argument, or in REFERENCE_ROOT):

    python tests/golden/make_golden_rmsnorm.py REFERENCE_ROOT

What is imported from the reference (nothing is copied into this repository):
  * model/common/bitnet_legacy.py   _RMSNorm (the same expression as _ExtraRMSNorm of
                                    core/bitnet/bitnet_int2_optimized.py:72-86, which cannot be imported
                                    without its CUDA extension) and BitLinear.activation_quant

For bf16, fp16 and fp32 inputs the file holds x, the norm weight, the upstream gradient, and the reference's
output, input gradient and weight gradient (autograd), plus the int8-valued tokens that the reference's
activation_quant makes of the normalised output.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
if not REF:
    raise SystemExit("usage: %s REFERENCE_ROOT   (the checkout of the reference project; or set REFERENCE_ROOT)" % sys.argv[0])


def main():
    spec = importlib.util.spec_from_file_location("ref_bitnet_legacy", os.path.join(REF, "model/common/bitnet_legacy.py"))
    legacy = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(legacy)
    out = {}
    cases = [(16, 64, torch.bfloat16, 1e-6), (24, 1024, torch.bfloat16, 1e-6), (8, 256, torch.float32, 1e-5),
             (12, 512, torch.float16, 1e-6)]
    for i, (M, K, dt, eps) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        x = (torch.randn(M, K, generator=g) * (0.5 + i)).to(dt)
        if i == 1:
            x[0] = 0.0                                  # an all-zero token: rstd = 1/sqrt(eps)
            x[1] = x[1] * 1e-3
        norm = legacy._RMSNorm(K, eps=eps)
        with torch.no_grad():
            norm.weight.copy_(1.0 + 0.2 * torch.randn(K, generator=g))
        gy = (torch.randn(M, K, generator=g) * 1e-2).to(dt)
        xin = x.clone().requires_grad_(True)
        y = norm(xin)
        y.backward(gy)
        layer = legacy.BitLinear(K, 8, bias=False)
        xq = layer.activation_quant(y.detach())
        a = y.detach().float().abs().max(dim=-1).values.clamp(min=layer.eps)
        q = torch.round(xq.float() * (127.0 / a)[:, None])
        out.update({f"x{i}": x.float().numpy(), f"w{i}": norm.weight.detach().numpy(), f"gy{i}": gy.float().numpy(),
                    f"y{i}": y.detach().float().numpy(), f"dx{i}": xin.grad.float().numpy(),
                    f"dw{i}": norm.weight.grad.numpy(), f"q{i}": q.numpy().astype(np.int16),
                    f"absmax{i}": a.numpy(), f"eps{i}": np.float32(eps),
                    f"io{i}": np.array({torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32"}[dt])})
    np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), **out)
    print("written", os.path.join(HERE, "rmsnorm.npz"))


if __name__ == "__main__":
    main()
