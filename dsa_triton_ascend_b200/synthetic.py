"""Seeded synthetic workloads of the benchmark configurations.

The reference has no dataset; its tests and perf scripts draw `np.random` data
(test_li_triton.py:30-36, test_sfa_triton.py:47-85, perf_sfa_triton.py:35-62).  The two
full-size configurations are defined here once, so that the GPU tests and the benchmark work on
the same tensors:

  configuration 3: `RandomState(2)`; q [1,S,64,128], k [1,S,1,128], w [1,S,64] / 8, in that order
  configuration 4: `RandomState(3)`; q [T,128,512], k [T,1,512], v (drawn, unused), q_rope
                   [T,128,64], k_rope [T,1,64] - the order of test_sfa_triton.py:54-58 - followed by
                   the indexer inputs that produce its sparse indices: q_i [T,64,128], k_i [T,1,128],
                   w_i [T,64] / 8 (TND, same cumulative lengths)

Values are fp32 normal draws rounded to bf16 (round to nearest even).  Tensors are produced in
row chunks (a normal stream drawn in pieces equals the stream drawn at once), so the fp32
staging never exceeds a few hundred MB; `device=None` keeps them on the host.
"""
import numpy as np
import torch

CONFIG3 = dict(seed=2, S=8192, heads=64, dim=128, sparse_count=2048)
CONFIG4 = dict(seed=3, lens=(8192, 4096, 2048, 1024), heads=128, dim=512, rope=64, topk=2048,
               li_heads=64, li_dim=128)


def _draw(rng, shape, device, dtype, scale=None, chunk_elems=1 << 25):
    """randn(*shape) from `rng`, cast to `dtype` on `device`, drawn in chunks along dim 0."""
    out = torch.empty(shape, dtype=dtype, device=device if device is not None else "cpu")
    inner = int(np.prod(shape[1:])) if len(shape) > 1 else 1
    step = max(1, chunk_elems // max(inner, 1))
    for i in range(0, shape[0], step):
        n = min(step, shape[0] - i)
        a = rng.randn(n, *shape[1:]).astype(np.float32)
        if scale is not None:
            a *= np.float32(scale)
        out[i:i + n] = torch.from_numpy(a).to(device=out.device).to(dtype)
    return out


def config3(device=None, scale=1):
    """Indexer at the prefill shape.  `scale` > 1 divides the sequence length (quick runs)."""
    c = CONFIG3
    S = c["S"] // scale
    rng = np.random.RandomState(c["seed"])
    q = _draw(rng, (1, S, c["heads"], c["dim"]), device, torch.bfloat16)
    k = _draw(rng, (1, S, 1, c["dim"]), device, torch.bfloat16)
    w = _draw(rng, (1, S, c["heads"]), device, torch.float32, scale=0.125)
    return dict(q=q, k=k, w=w, S=S, sparse_count=c["sparse_count"] // scale, sparse_mode=3)


def config4(device=None, scale=1, lens=None):
    """Attention at the prefill shape (TND) plus the indexer inputs its indices come from.
    `lens` overrides the sequence lengths (profiling captures on a part of the batch)."""
    c = CONFIG4
    lens = [L // scale for L in (lens or c["lens"])]
    T = sum(lens)
    rng = np.random.RandomState(c["seed"])
    bf = torch.bfloat16
    q = _draw(rng, (T, c["heads"], c["dim"]), device, bf)
    k = _draw(rng, (T, 1, c["dim"]), device, bf)
    rng.randn(T, 1, c["dim"])                       # value: drawn to keep the stream aligned, unused
    qr = _draw(rng, (T, c["heads"], c["rope"]), device, bf)
    kr = _draw(rng, (T, 1, c["rope"]), device, bf)
    qi = _draw(rng, (T, c["li_heads"], c["li_dim"]), device, bf)
    ki = _draw(rng, (T, 1, c["li_dim"]), device, bf)
    wi = _draw(rng, (T, c["li_heads"]), device, torch.float32, scale=0.125)
    cum = np.cumsum(lens).tolist()
    return dict(q=q, k=k, qr=qr, kr=kr, qi=qi, ki=ki, wi=wi, lens=lens, cum=cum, T=T,
                topk=c["topk"] // scale, scale=1.0 / float(np.sqrt(c["dim"] + c["rope"])), sparse_mode=3)


def valid_pairs(lens, topk):
    """(token, key) pairs configuration 4 touches: sum over tokens of min(topk, position + 1)."""
    return int(sum(min(topk, s + 1) for L in lens for s in range(L)))
