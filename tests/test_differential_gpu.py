"""Randomised differential tests: the tcgen05 paths against the portable CUDA-core kernels over
randomly drawn shapes, layouts, lengths and index patterns (seeded).  The portable kernels are the
ones pinned to the reference goldens case by case; these tests carry that parity across the corners
of the operator surface that the tensor-core paths serve (split-KV, paged caches with holes,
block-wise indices, -1 entries, duplicates, ragged and empty sequences, both sparse modes)."""
import numpy as np
import pytest
import torch

from oracle.compare import sfa_acceptance_rule
from tests.util import host

pytestmark = pytest.mark.gpu


def _rand_bf16(rng, *shape, dtype=torch.bfloat16):
    return torch.from_numpy(rng.randn(*shape).astype(np.float32)).cuda().to(dtype)


def _paged(rng, B, lens_k, bs, width, dtype, holes):
    need = [-(-int(L) // bs) for L in lens_k]
    max_blocks = max(need) + int(rng.randint(0, 3))
    nblk = sum(need) + 4
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
        if holes and need[b] > 2:
            bt[b, int(rng.randint(0, need[b]))] = -1
    caches = [_rand_bf16(rng, nblk, bs, 1, w, dtype=dtype) for w in width]
    return caches, torch.from_numpy(bt).cuda(), max_blocks


@pytest.mark.parametrize("seed", range(12))
def test_sfa_tensor_path_equals_portable_on_random_problems(seed):
    import dsa_triton_ascend_b200.sparse_flash_attention as sfa
    rng = np.random.RandomState(9000 + seed)
    dtype = torch.bfloat16 if seed % 4 else torch.float16
    layout = ("BSND", "TND", "PA_BSND")[seed % 3]
    mode = 0 if seed % 5 == 4 else 3
    B = int(rng.randint(1, 5))
    N1 = int(rng.choice([128, 128, 64, 40, 16]))      # fewer than 128 heads: a tensor-parallel shard
    blk = int(rng.choice([1, 1, 2, 8]))
    count = int(rng.choice([24, 96, 300, 1024 // blk]))
    S1 = int(rng.choice([1, 2, 5, 40]))
    S2 = int(rng.choice([130, 700, 2600]))
    lens_q = [int(rng.randint(0 if B > 1 else 1, S1 + 1)) for _ in range(B)]
    lens_k = [int(rng.randint(1, S2 + 1)) for _ in range(B)]
    if max(lens_q) == 0:
        lens_q[0] = S1
    # indices: ascending distinct block ids inside the window, then -1 entries, a duplicate, an
    # out-of-window id and a hole sprinkled in
    nblocks = -(-S2 // blk)
    idx = np.full((B, S1, 1, count), -1, np.int32)
    for b in range(B):
        for s in range(S1):
            n = int(rng.randint(0, min(count, nblocks) + 1))
            idx[b, s, 0, :n] = np.sort(rng.permutation(nblocks)[:n])
            if n > 4:
                idx[b, s, 0, n // 2] = -1
                idx[b, s, 0, n // 3] = idx[b, s, 0, n // 3 + 1]
                idx[b, s, 0, n - 1] = nblocks + 5
    scale = 1.0 / 24.0
    kw = dict(scale_value=scale, sparse_block_size=blk, sparse_mode=mode, return_softmax_lse=bool(seed % 2 == 0))
    if layout == "BSND":
        q, qr = _rand_bf16(rng, B, S1, N1, 512, dtype=dtype), _rand_bf16(rng, B, S1, N1, 64, dtype=dtype)
        k, kr = _rand_bf16(rng, B, S2, 1, 512, dtype=dtype), _rand_bf16(rng, B, S2, 1, 64, dtype=dtype)
        args = (q, k, k, torch.from_numpy(idx).cuda())
        kw.update(query_rope=qr, key_rope=kr, actual_seq_lengths_query=lens_q, actual_seq_lengths_kv=lens_k)
    elif layout == "TND":
        lens_q = [max(1, v) for v in lens_q]
        lens_k = [max(lens_k[b], 1) for b in range(B)]
        T1, T2 = sum(lens_q), sum(lens_k)
        q, qr = _rand_bf16(rng, T1, N1, 512, dtype=dtype), _rand_bf16(rng, T1, N1, 64, dtype=dtype)
        k, kr = _rand_bf16(rng, T2, 1, 512, dtype=dtype), _rand_bf16(rng, T2, 1, 64, dtype=dtype)
        flat = np.concatenate([idx[b, :lens_q[b]] for b in range(B)], axis=0)
        args = (q, k, k, torch.from_numpy(np.ascontiguousarray(flat)).cuda())
        kw.update(query_rope=qr, key_rope=kr, layout_query="TND", layout_kv="TND",
                  actual_seq_lengths_query=list(np.cumsum(lens_q)), actual_seq_lengths_kv=list(np.cumsum(lens_k)))
    else:
        bs = int(rng.choice([16, 128]))
        (kc, krc), table, _ = _paged(rng, B, lens_k, bs, (512, 64), dtype, holes=bool(seed % 2))
        q, qr = _rand_bf16(rng, B, S1, N1, 512, dtype=dtype), _rand_bf16(rng, B, S1, N1, 64, dtype=dtype)
        args = (q, kc, kc, torch.from_numpy(idx).cuda())
        kw.update(query_rope=qr, key_rope=krc, layout_kv="PA_BSND", block_table=table, block_size=bs,
                  actual_seq_lengths_query=lens_q, actual_seq_lengths_kv=lens_k)
    out = {}
    for kind in ("tensor", "portable"):
        sfa.set_kernel(kind)
        try:
            out[kind] = [host(t) for t in sfa.sparse_flash_attention_triton(*args, **kw)]
        finally:
            sfa.set_kernel("auto")
    # (odd seeds with a paged cache have absent blocks inside the valid length: both paths read such
    # a slot as a zero row that takes part, like the reference's un-paging)
    sfa_acceptance_rule(*out["tensor"], *out["portable"])


@pytest.mark.parametrize("seed", range(10))
def test_li_tensor_path_equals_portable_on_random_problems(seed):
    import dsa_triton_ascend_b200.lightning_indexer as li
    rng = np.random.RandomState(9100 + seed)
    dtype = torch.bfloat16 if seed % 3 else torch.float16
    layout = ("BSND", "TND", "PA_BSND")[seed % 3]
    mode = 0 if seed % 4 == 3 else 3
    B = int(rng.randint(1, 5))
    H = int(rng.choice([64, 64, 48, 32, 16]))         # fewer than 64 heads: a tensor-parallel shard
    S1 = int(rng.choice([1, 2, 7, 33, 130]))
    S2 = int(rng.choice([100, 900, 3000]))
    count = int(rng.choice([16, 200, 1024]))
    lens_q = [int(rng.randint(1, S1 + 1)) for _ in range(B)]
    lens_k = [int(rng.randint(1, S2 + 1)) for _ in range(B)]
    wdt = (torch.float32, torch.bfloat16, torch.float16)[seed % 3] if dtype == torch.bfloat16 else torch.float32
    kw = dict(sparse_count=count, sparse_mode=mode, return_value=True)
    if layout == "BSND":
        q, k = _rand_bf16(rng, B, S1, H, 128, dtype=dtype), _rand_bf16(rng, B, S2, 1, 128, dtype=dtype)
        w = (torch.from_numpy(rng.randn(B, S1, H).astype(np.float32)).cuda() / 8).to(wdt)
        kw.update(actual_seq_lengths_query=lens_q, actual_seq_lengths_key=lens_k)
    elif layout == "TND":
        T1, T2 = sum(lens_q), sum(lens_k)
        q, k = _rand_bf16(rng, T1, H, 128, dtype=dtype), _rand_bf16(rng, T2, 1, 128, dtype=dtype)
        w = (torch.from_numpy(rng.randn(T1, H).astype(np.float32)).cuda() / 8).to(wdt)
        kw.update(layout_query="TND", layout_key="TND", actual_seq_lengths_query=list(np.cumsum(lens_q)),
                  actual_seq_lengths_key=list(np.cumsum(lens_k)))
    else:
        bs = int(rng.choice([16, 32, 64, 128, 256]))
        (k,), table, _ = _paged(rng, B, lens_k, bs, (128,), dtype, holes=bool(seed % 2))
        q = _rand_bf16(rng, B, S1, H, 128, dtype=dtype)
        w = (torch.from_numpy(rng.randn(B, S1, H).astype(np.float32)).cuda() / 8).to(wdt)
        kw.update(layout_key="PA_BSND", block_table=table, actual_seq_lengths_query=lens_q,
                  actual_seq_lengths_key=lens_k)
    out = {}
    for kind in ("tensor", "portable"):
        li.set_kernel(kind)
        try:
            i_, v_ = li.lightning_indexer_triton(q, k, w, **kw)
            out[kind] = (host(i_), host(v_))
        finally:
            li.set_kernel("auto")
    ti, tv = out["tensor"]
    pi, pv = out["portable"]
    # same number of valid slots everywhere; values agree to a rounding step of the io dtype (the two
    # kernels add 64 products in different orders); the index sets agree except at such boundaries
    assert ((ti >= 0) == (pi >= 0)).all()
    step = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    assert np.allclose(tv, pv, rtol=2 * step, atol=1e-3)
    assert (ti == pi).mean() >= 0.97
