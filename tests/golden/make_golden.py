"""Generates tests/golden/*.npz from the reference itself (run in a container that has the
reference tree; the fixtures are committed, this script documents how they were made).

    python tests/golden/make_golden.py [REFERENCE_ROOT]     (path of the reference checkout)

Sources of the expected values:
  * kernels/tests/kernel_build.py            pack_int2 / unpack_int2 (pure torch, imported)
  * core/bitnet/int2_linear_tc.py            Int2LinearTC.init_from_float / _pack_int2_cpu (imported with
                                             the JIT extension loader stubbed out: no kernel is built)
  * model/common/bitnet_legacy.py            BitLinear.activation_quant / weight_quant / F.linear (imported)
  * kernels/int2/int2_hysteresis_v2.cu,
    kernels/int2/int2_activation_quant.cu    compiled for the host by oracle/build_ref.sh and called
                                             through oracle/native.py (flush-to-zero on, as the
                                             reference's fast-math build behaves)
All inputs are seeded; nothing here is copied from the reference, only its outputs are recorded.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
if not REF:
    raise SystemExit("usage: %s REFERENCE_ROOT   (the checkout of the reference project; or set REFERENCE_ROOT)" % sys.argv[0])
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import native  # noqa: E402


def _import(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    torch.manual_seed(0)
    rng = np.random.default_rng(0)

    # the reference modules JIT-build a CUDA extension at import; make that a no-op failure
    import torch.utils.cpp_extension as cpp_ext
    real_load = cpp_ext.load

    def _no_load(*a, **k):
        raise RuntimeError("extension loading disabled while generating golden vectors")

    cpp_ext.load = _no_load
    try:
        kb = _import(os.path.join(REF, "kernels/tests/kernel_build.py"), "ref_kernel_build")
        tc = _import(os.path.join(REF, "core/bitnet/int2_linear_tc.py"), "ref_int2_linear_tc")
        legacy = _import(os.path.join(REF, "model/common/bitnet_legacy.py"), "ref_bitnet_legacy")
    finally:
        cpp_ext.load = real_load

    # ---- 1. packing (test helper pads with code 1, module packer with code 0) ----------------
    pack = {}
    for i, (N, K) in enumerate([(8, 8), (5, 7), (16, 130), (3, 1), (33, 64)]):
        w = torch.randint(-1, 2, (N, K), generator=torch.Generator().manual_seed(10 + i), dtype=torch.int8)
        pack[f"w{i}"] = w.numpy()
        pack[f"helper_packed{i}"] = kb.pack_int2(w.float()).numpy()
        pack[f"helper_unpacked{i}"] = kb.unpack_int2(kb.pack_int2(w.float()), K).numpy()
        fake = types.SimpleNamespace(W_packed=torch.zeros(N, (K + 3) // 4, dtype=torch.uint8))
        tc.Int2LinearTC._pack_int2_cpu(fake, w)
        pack[f"module_packed{i}"] = fake.W_packed.numpy()
    # every byte value, to pin the decode of code 3
    allb = torch.arange(256, dtype=torch.uint8).view(1, 256)
    pack["all_bytes_unpacked"] = kb.unpack_int2(allb, 1024).numpy()
    np.savez_compressed(os.path.join(HERE, "pack.npz"), **pack)

    # ---- 2. ternarisation through Int2LinearTC.init_from_float ------------------------------
    tern = {}
    for i, (N, K, std) in enumerate([(48, 100, 0.02), (64, 256, 0.02), (7, 5, 1.0)]):
        W = torch.randn(N, K, generator=torch.Generator().manual_seed(20 + i)) * std
        fake = types.SimpleNamespace(
            out_features=N, in_features=K, use_24_sparsity=False,
            W_packed=torch.zeros(N, (K + 3) // 4, dtype=torch.uint8),
            H_packed=torch.ones(N, (K + 1) // 2, dtype=torch.uint8),
            gamma=torch.nn.Parameter(torch.ones(1)), _gamma_cached=None, _initialized=False)
        fake._pack_int2_cpu = types.MethodType(tc.Int2LinearTC._pack_int2_cpu, fake)
        tc.Int2LinearTC.init_from_float(fake, W)
        layer = legacy.BitLinear(K, N, bias=False)
        with torch.no_grad():
            wq = layer.weight_quant(W)
        tern[f"W{i}"] = W.numpy()
        tern[f"W_packed{i}"] = fake.W_packed.numpy()
        tern[f"gamma{i}"] = np.float64(fake._gamma_cached)
        tern[f"legacy_wq{i}"] = wq.numpy()
        tern[f"legacy_gamma{i}"] = np.float32(W.abs().mean().clamp(min=layer.eps).item())
    np.savez_compressed(os.path.join(HERE, "ternarize.npz"), **tern)

    # ---- 3. per-token activation quantisation and the legacy layer maths --------------------
    act = {}
    for i, (M, K, N, dt) in enumerate([(16, 64, 32, torch.float32), (32, 256, 48, torch.bfloat16),
                                       (5, 100, 7, torch.float32)]):
        g = torch.Generator().manual_seed(30 + i)
        x = torch.randn(M, K, generator=g).to(dt)
        if i == 2:
            x[0] = 0.0            # an all-zero token exercises the eps clamp
            x[1] = x[1] * 1e-7
        W = torch.randn(N, K, generator=g) * 0.02
        dY = (torch.randn(M, N, generator=g) * 1e-2).to(dt)
        layer = legacy.BitLinear(K, N, bias=False)
        with torch.no_grad():
            layer.weight.copy_(W)
        xin = x.clone().requires_grad_(True)
        xq = layer.activation_quant(xin)
        wq = layer.weight_quant(layer.weight)
        y = torch.nn.functional.linear(xq, wq.to(dt))
        y.backward(dY)
        act[f"x{i}"] = x.float().numpy()
        act[f"W{i}"] = W.numpy()
        act[f"dY{i}"] = dY.float().numpy()
        act[f"xq{i}"] = xq.detach().float().numpy()
        act[f"y{i}"] = y.detach().float().numpy()
        act[f"dx{i}"] = xin.grad.float().numpy()
        act[f"dw{i}"] = layer.weight.grad.float().numpy()
        act[f"is_bf16_{i}"] = np.bool_(dt == torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "legacy_layer.npz"), **act)

    # ---- 4. hysteresis: the reference kernel source run on the host --------------------------
    hyst = {}
    cases = [(48, 100, 2, 1e-2, 1e-3, 5.0, 0.001, 1), (16, 130, 3, 1e-3, 2e-2, 5.0, 0.25, 7),
             (5, 7, 7, 1.0, 1e-3, 5.0, 0.001, 3), (64, 64, 1, 1e-2, 1e-3, 5.0, 0.5, 123456),
             (9, 20, 9, 5e-2, 1e-3, 2.5, 0.01, 2), (8, 33, 0, 5e-2, 1e-2, 5.0, 0.9, 4000000000)]
    for i, (N, K, thr, gstd, lr, ls, dec, step) in enumerate(cases):
        w = rng.integers(-1, 2, (N, K)).astype(np.int8)
        enc = (w + 1).astype(np.uint8)
        enc[rng.random((N, K)) < 0.05] = 3                      # some fields carry the reserved code
        pk = (K + 3) // 4
        full = np.full((N, pk * 4), 3 if i % 2 else 0, dtype=np.uint8)  # padding fields: code 3 or 0
        full[:, :K] = enc
        full = full.reshape(N, pk, 4)
        Wp = (full[:, :, 0] | (full[:, :, 1] << 2) | (full[:, :, 2] << 4) | (full[:, :, 3] << 6)).astype(np.uint8)
        h = rng.integers(-7, 8, (N, K)).astype(np.int8)
        ph = (K + 1) // 2
        hb = np.full((N, ph * 2), 0xA, dtype=np.uint8)
        hb[:, :K] = (h & 0xF).astype(np.uint8)
        hb = hb.reshape(N, ph, 2)
        Hp = (hb[:, :, 0] | (hb[:, :, 1] << 4)).astype(np.uint8)
        dW = (rng.standard_normal((N, K)) * gstd).astype(np.float32)
        dW.flat[::17] *= 300.0
        dW.flat[5::29] = 1e-41
        step_i = step if step < 2 ** 31 else step - 2 ** 32
        W1, H1 = native.ref_hysteresis_step(dW, Wp, Hp, lr, ls, thr, dec, step_i, K, ftz=True)
        W2, H2 = native.ref_hysteresis_step(dW, W1, H1, lr, ls, thr, dec, step_i + 1, K, ftz=True)
        hyst.update({f"dW{i}": dW, f"W0_{i}": Wp, f"H0_{i}": Hp, f"W1_{i}": W1, f"H1_{i}": H1,
                     f"W2_{i}": W2, f"H2_{i}": H2,
                     f"params{i}": np.array([N, K, thr, lr, ls, dec, step], dtype=np.float64)})
    np.savez_compressed(os.path.join(HERE, "hysteresis.npz"), **hyst)

    # ---- 5. per-tensor quantisation: the reference kernel source run on the host -------------
    qt = {}
    lib = native.ref_cpu_lib()
    for i, (size, mul) in enumerate([(256 * 256, 3.0), (255, 3.0), (1, 1.0), (1000, 1e-9), (777, 50.0)]):
        x = (torch.randn(size, generator=torch.Generator().manual_seed(40 + i)) * mul).half()
        if i == 4:
            x[3] = float("inf"); x[4] = float("nan"); x[5] = -float("inf")
        bits = x.view(torch.int16).numpy().view(np.uint16).copy()
        q = np.zeros(size, dtype=np.int8)
        am = np.zeros(1, dtype=np.float32)
        lib.ref_quantize_tensor_cpu(bits, q, am, size, 0)
        deq = np.zeros(size, dtype=np.uint16)
        lib.ref_dequantize_tensor_cpu(q, deq, am, size)
        qt.update({f"x_bits{i}": bits, f"q{i}": q, f"absmax{i}": am, f"deq_bits{i}": deq})
    np.savez_compressed(os.path.join(HERE, "quant_tensor.npz"), **qt)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
