"""Seeded inputs with the shapes and distributions of the benchmark configurations, and torch<->numpy glue."""
import numpy as np
import torch

from oracle import int2_oracle as O


def t2n(t: torch.Tensor) -> np.ndarray:
    """Tensor -> numpy (bf16/fp16 are widened to float32, exactly)."""
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    return t.numpy()


def make_layer_inputs(M, K, N, seed=0, dtype=torch.bfloat16, dy_std=1e-2, w_std=0.02, counters=None):
    """x ~ N(0,1) in `dtype`, W ~ N(0, w_std) float32, dY ~ N(0, dy_std) in `dtype`, counters zero or uniform in
    [-c, c]: the distributions of the benchmark configurations.  Everything is generated on the CPU from `seed`."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype)
    W = torch.randn(N, K, generator=g) * w_std
    dY = (torch.randn(M, N, generator=g) * dy_std).to(dtype)
    gamma = float(max(W.abs().mean().item(), 1e-5))
    Wq = O.ternarize(W.numpy(), gamma)
    Wp = O.pack_ternary(Wq, pad_code=0)
    if counters:
        h = torch.randint(-counters, counters + 1, (N, K), generator=g, dtype=torch.int8).numpy()
    else:
        h = np.zeros((N, K), dtype=np.int8)
    Hp = O.pack_counters(h)
    return dict(x=x, W=W, dY=dY, gamma=gamma, Wp=Wp, Hp=Hp)


def random_packed(N, K, seed, third_zero=True):
    """Packed ternary weights with about one third zeros (torch.randint(-1, 2), as the reference's
    make_packed_weights, kernels/tests/kernel_build.py:93-97)."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randint(-1, 2, (N, K), generator=g, dtype=torch.int8).numpy()
    return O.pack_ternary(w, pad_code=1), w
