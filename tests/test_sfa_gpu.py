"""GPU parity of sparse_flash_attention forward against the reference goldens and the oracle.

Tolerances: attention_out atol = rtol = 2e-2 (bf16 and fp16), softmax_max / softmax_sum 1e-3
relative; the reference's own percentage rule (test_sfa_triton.py:88-123) is checked as well.
"""
import os

import numpy as np
import pytest
import torch

from oracle import sparse_flash_attention_oracle
from oracle import layouts
from oracle.compare import sfa_acceptance_rule, sfa_reference_rule
from oracle.inputs import round_io, sparse_indices
from tests.golden.cases import SFA_CASES, sfa_case_inputs
from tests.util import dev, host, tdtype

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _sfa():
    import dsa_triton_ascend_b200.sparse_flash_attention as sfa
    return sfa


def _compare(out, smax, ssum, ref_out, ref_smax, ref_ssum, dtype):
    sfa_acceptance_rule(out, smax, ssum, ref_out, ref_smax, ref_ssum)
    assert sfa_reference_rule(out, ref_out, dtype, pct_thd=99.0 if dtype == "bf16" else 99.5)
    assert sfa_reference_rule(smax, ref_smax, dtype)
    assert sfa_reference_rule(ssum, ref_ssum, dtype)


@pytest.mark.parametrize("name", sorted(SFA_CASES))
def test_sfa_matches_reference_golden(name):
    sfa = _sfa()
    q, k, qr, kr, idx, act_q, act_k, scale, c = sfa_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = tdtype(c["dtype"])
    full = "act_q" not in c and "act_k" not in c
    out, smax, ssum = sfa.sparse_flash_attention_triton(
        dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(idx).cuda(), scale_value=scale,
        actual_seq_lengths_query=None if full else act_q.tolist(),
        actual_seq_lengths_kv=None if full else act_k.tolist(),
        query_rope=dev(qr, dt), key_rope=dev(kr, dt), sparse_block_size=c["block"],
        sparse_mode=c["mode"], return_softmax_lse=True)
    assert out.shape == (c["B"], c["S1"], c["N1"], c["D"]) and out.dtype == dt
    assert smax.shape == (c["B"], 1, c["S1"], c["N1"]) and smax.dtype == torch.float32
    out, smax, ssum = host(out), host(smax), host(ssum)
    sel = g["rows"]
    _compare(out[sel[:, 0], sel[:, 1]], smax[sel[:, 0], 0, sel[:, 1]], ssum[sel[:, 0], 0, sel[:, 1]],
             g["out"].astype(np.float32), g["smax"], g["ssum"], c["dtype"])
    # rows the golden leaves untouched stay zero in all three outputs
    for b in range(c["B"]):
        aq, ak = int(act_q[b]), int(act_k[b])
        dead = [s for s in range(c["S1"]) if s >= aq or (c["mode"] == 3 and ak - aq + s + 1 <= 0)]
        if dead:
            assert (out[b, dead] == 0).all() and (smax[b, 0, dead] == 0).all() and (ssum[b, 0, dead] == 0).all()


def test_sfa_without_lse_returns_zero_stats():
    sfa = _sfa()
    q, k, qr, kr, idx, act_q, act_k, scale, c = sfa_case_inputs("sfa_tiny")
    dt = torch.bfloat16
    args = (dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(idx).cuda())
    kw = dict(scale_value=scale, query_rope=dev(qr, dt), key_rope=dev(kr, dt), sparse_mode=3)
    o1, m1, s1 = sfa.sparse_flash_attention_triton(*args, return_softmax_lse=False, **kw)
    o2, m2, s2 = sfa.sparse_flash_attention_triton(*args, return_softmax_lse=True, **kw)
    assert torch.equal(o1, o2) and not m1.any() and not s1.any() and m2.any()


def _random_case(seed, lens_q, lens_k, N1, D, K, block=1, mode=3):
    rng = np.random.RandomState(seed)
    B = len(lens_q)
    S1, S2 = max(lens_q), max(lens_k)
    q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), "bf16")
    k = round_io(rng.randn(B, S2, 1, D).astype(np.float32), "bf16")
    qr = round_io(rng.randn(B, S1, N1, 64).astype(np.float32), "bf16")
    kr = round_io(rng.randn(B, S2, 1, 64).astype(np.float32), "bf16")
    idx = sparse_indices(seed + 1, B, S1, S2, K, block, mode, lens_q, lens_k)
    return q, k, qr, kr, idx


def test_sfa_tnd_matches_oracle():
    sfa = _sfa()
    lens_q, lens_k = [20, 3, 33], [64, 40, 33]
    N1, D, K = 16, 512, 48
    q, k, qr, kr, idx = _random_case(41, lens_q, lens_k, N1, D, K)
    scale = 1.0 / np.sqrt(D + 64.0)
    ref = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, lens_q, lens_k, sparse_mode=3, dtype="bf16")
    tq = layouts.bsnd_to_tnd(q, lens_q)
    tk = layouts.bsnd_to_tnd(k, lens_k)
    tqr = layouts.bsnd_to_tnd(qr, lens_q)
    tkr = layouts.bsnd_to_tnd(kr, lens_k)
    tidx = layouts.bsnd_to_tnd(idx, lens_q)
    dt = torch.bfloat16
    out, smax, ssum = sfa.sparse_flash_attention_triton(
        dev(tq, dt), dev(tk, dt), dev(tk, dt), torch.from_numpy(tidx).cuda(), scale_value=scale,
        actual_seq_lengths_query=np.cumsum(lens_q).tolist(), actual_seq_lengths_kv=np.cumsum(lens_k).tolist(),
        query_rope=dev(tqr, dt), key_rope=dev(tkr, dt), layout_query="TND", layout_kv="TND",
        sparse_mode=3, return_softmax_lse=True)
    assert out.shape == (sum(lens_q), N1, D) and smax.shape == (1, sum(lens_q), N1)
    _compare(host(out), host(smax), host(ssum), layouts.bsnd_to_tnd(ref[0], lens_q),
             layouts.stats_bsnd_to_tnd(ref[1], lens_q), layouts.stats_bsnd_to_tnd(ref[2], lens_q), "bf16")


def test_sfa_paged_cache_matches_oracle():
    sfa = _sfa()
    lens_q, lens_k = [2, 2, 2], [100, 17, 64]
    B, N1, D, K, bs = 3, 16, 512, 32, 16
    q, k, qr, kr, idx = _random_case(43, lens_q, lens_k, N1, D, K)
    scale = 1.0 / np.sqrt(D + 64.0)
    ref = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, lens_q, lens_k, sparse_mode=3, dtype="bf16")
    rng = np.random.RandomState(44)
    max_blocks, nblk = 8, 40
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, dtype=np.int32)
    cache = np.zeros((nblk, bs, 1, D), np.float32)
    cache_r = np.zeros((nblk, bs, 1, 64), np.float32)
    used = 0
    for b in range(B):
        need = -(-lens_k[b] // bs)
        for i in range(need):
            blk = perm[used]
            used += 1
            bt[b, i] = blk
            n = min(bs, lens_k[b] - i * bs)
            cache[blk, :n] = k[b, i * bs:i * bs + n]
            cache_r[blk, :n] = kr[b, i * bs:i * bs + n]
    dt = torch.bfloat16
    out, smax, ssum = sfa.sparse_flash_attention_triton(
        dev(q, dt), dev(cache, dt), dev(cache, dt), torch.from_numpy(idx).cuda(), scale_value=scale,
        block_table=torch.from_numpy(bt).cuda(), actual_seq_lengths_query=lens_q, actual_seq_lengths_kv=lens_k,
        query_rope=dev(qr, dt), key_rope=dev(cache_r, dt), layout_kv="PA_BSND", sparse_mode=3,
        return_softmax_lse=True, block_size=bs)
    _compare(host(out), host(smax), host(ssum), *ref, "bf16")


def test_sfa_skips_interior_minus_one_and_counts_duplicates():
    """-1 entries are skipped wherever they sit and a repeated index counts twice
    (sparse_flash_attention_triton.py:465): equal to the oracle on the compacted list."""
    sfa = _sfa()
    q, k, qr, kr, idx = _random_case(45, [8], [128], 16, 512, 32)
    scale = 1.0 / np.sqrt(576.0)
    holes = idx.copy()
    holes[0, :, 0, 3] = -1
    holes[0, :, 0, 10] = -1
    compact = np.full_like(holes, -1)
    for s in range(8):
        v = holes[0, s, 0][holes[0, s, 0] >= 0]
        compact[0, s, 0, :len(v)] = v
    ref = sparse_flash_attention_oracle(q, k, compact, qr, kr, scale, [8], [128], sparse_mode=3, dtype="bf16")
    dt = torch.bfloat16
    got = sfa.sparse_flash_attention_triton(
        dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(holes).cuda(), scale_value=scale,
        query_rope=dev(qr, dt), key_rope=dev(kr, dt), sparse_mode=3, return_softmax_lse=True)
    _compare(*(host(t) for t in got), *ref, "bf16")


def test_sfa_is_bitwise_repeatable():
    sfa = _sfa()
    q, k, qr, kr, idx, act_q, act_k, scale, c = sfa_case_inputs("sfa_multi_batch")
    dt = torch.bfloat16
    args = (dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(idx).cuda())
    kw = dict(scale_value=scale, query_rope=dev(qr, dt), key_rope=dev(kr, dt), sparse_mode=3,
              return_softmax_lse=True)
    a = sfa.sparse_flash_attention_triton(*args, **kw)
    b = sfa.sparse_flash_attention_triton(*args, **kw)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_sfa_full_size_tnd_sampled_rows():
    """Configuration 4 shape (TND, lengths 8192/4096/2048/1024 scaled by 1/4 to keep the CUDA-core
    path quick, 128 heads, k=2048 -> 512): sampled tokens against the oracle, plus softmax
    invariants on every token (sum >= 1, finite, zero rows only where nothing is visible)."""
    sfa = _sfa()
    lens = [2048, 1024, 512, 256]
    T, N1, D, K = sum(lens), 128, 512, 512
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(T, N1, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(T, 1, D, generator=g, device="cuda").bfloat16()
    qr = torch.randn(T, N1, 64, generator=g, device="cuda").bfloat16()
    kr = torch.randn(T, 1, 64, generator=g, device="cuda").bfloat16()
    cu = np.cumsum(lens)
    idx = np.full((T, 1, K), -1, np.int32)
    rng = np.random.RandomState(3)
    start = 0
    for L in lens:
        for s in range(L):
            n = min(K, s + 1)
            idx[start + s, 0, :n] = np.sort(rng.choice(s + 1, n, replace=False))
        start += L
    scale = 1.0 / np.sqrt(576.0)
    out, smax, ssum = sfa.sparse_flash_attention_triton(
        q, k, k, torch.from_numpy(idx).cuda(), scale_value=scale, actual_seq_lengths_query=cu.tolist(),
        actual_seq_lengths_kv=cu.tolist(), query_rope=qr, key_rope=kr, layout_query="TND", layout_kv="TND",
        sparse_mode=3, return_softmax_lse=True)
    assert bool(torch.isfinite(out.float()).all()) and bool((ssum >= 1.0 - 1e-6).all())
    toks = [0, 1, 700, 2047, 2048, 2048 + 1023, 3072 + 17, T - 1]
    qn, kn, qrn, krn = host(q), host(k), host(qr), host(kr)
    for t in toks:
        b = int(np.searchsorted(cu, t, side="right"))
        s0 = 0 if b == 0 else int(cu[b - 1])
        s = t - s0
        L = lens[b]
        # the oracle takes the row position from its index: feed the single row at position s
        qq = np.zeros((1, L, N1, D), np.float32)
        qq[0, s] = qn[t]
        qqr = np.zeros((1, L, N1, 64), np.float32)
        qqr[0, s] = qrn[t]
        ii = np.full((1, L, 1, K), -1, np.int32)
        ii[0, s] = idx[t]
        ref = sparse_flash_attention_oracle(qq, kn[None, s0:s0 + L], ii, qqr, krn[None, s0:s0 + L], scale,
                                            [L], [L], sparse_mode=3, dtype="bf16", rows=[(0, s)])
        _compare(host(out[t]), host(smax[0, t]), host(ssum[0, t]), ref[0][0, s], ref[1][0, 0, s],
                 ref[2][0, 0, s], "bf16")


def test_sfa_tensor_path_agrees_with_portable_path_and_reports_clean_status():
    """128 heads x D=512 runs on the tcgen05 kernel: block-wise indices, ragged lengths, fp16 and a
    paged cache must agree with the portable CUDA-core kernel, and the status word must stay 0."""
    import ctypes
    from dsa_triton_ascend_b200 import _cabi
    sfa = _sfa()
    held = []
    orig = sfa.workspace

    def keep_ws(n, dev):
        t = orig(n, dev)
        held.append(t)
        return t

    rng = np.random.RandomState(77)
    B, S1, S2, N1, D, K, bs = 2, 24, 640, 128, 512, 40, 4
    lens_q, lens_k = [24, 9], [640, 333]
    for dtype, tdt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), dtype)
        k = round_io(rng.randn(B, S2, 1, D).astype(np.float32), dtype)
        qr = round_io(rng.randn(B, S1, N1, 64).astype(np.float32), dtype)
        kr = round_io(rng.randn(B, S2, 1, 64).astype(np.float32), dtype)
        idx = sparse_indices(78, B, S1, S2, K, bs, 3, lens_q, lens_k)
        idx[0, 5, 0, 3] = -1          # a hole in the middle of a row
        args = (dev(q, tdt), dev(k, tdt), dev(k, tdt), torch.from_numpy(idx).cuda())
        kw = dict(scale_value=1.0 / 24.0, actual_seq_lengths_query=lens_q, actual_seq_lengths_kv=lens_k,
                  query_rope=dev(qr, tdt), key_rope=dev(kr, tdt), sparse_block_size=bs, sparse_mode=3,
                  return_softmax_lse=True)
        sfa.workspace = keep_ws
        try:
            sfa.set_kernel("tensor")
            got = sfa.sparse_flash_attention_triton(*args, **kw)
            stream = torch.cuda.current_stream().cuda_stream
            assert _cabi.lib.dsa_read_device_status(held[-1].data_ptr(), stream) == 0
            sfa.set_kernel("portable")
            ref = sfa.sparse_flash_attention_triton(*args, **kw)
        finally:
            sfa.set_kernel("auto")
            sfa.workspace = orig
        sfa_acceptance_rule(*(host(t) for t in got), *(host(t) for t in ref))


def test_sfa_portable_kernel_request_is_honoured_for_other_shapes():
    """Shapes outside the tensor path (fewer than 16 heads, other head dims) refuse kernel='tensor'
    with a clear error."""
    sfa = _sfa()
    q, k, qr, kr, idx, act_q, act_k, scale, c = sfa_case_inputs("sfa_tiny")
    dt = torch.bfloat16
    sfa.set_kernel("tensor")
    try:
        with pytest.raises(RuntimeError):
            sfa.sparse_flash_attention_triton(dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(idx).cuda(),
                                              scale_value=scale, query_rope=dev(qr, dt), key_rope=dev(kr, dt),
                                              sparse_mode=3)
    finally:
        sfa.set_kernel("auto")


def test_sfa_full_mode_on_the_tensor_core_path():
    """sparse_mode=0 with 128 heads: every index below act_k takes part, whatever the row."""
    sfa = _sfa()
    rng = np.random.RandomState(91)
    B, S1, S2, N1, D, K = 1, 6, 400, 128, 512, 200
    q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), "bf16")
    k = round_io(rng.randn(B, S2, 1, D).astype(np.float32), "bf16")
    qr = round_io(rng.randn(B, S1, N1, 64).astype(np.float32), "bf16")
    kr = round_io(rng.randn(B, S2, 1, 64).astype(np.float32), "bf16")
    idx = sparse_indices(92, B, S1, S2, K, 1, 0, [S1], [350])
    scale = 1.0 / 24.0
    ref = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, [S1], [350], sparse_mode=0, dtype="bf16")
    dt = torch.bfloat16
    got = sfa.sparse_flash_attention_triton(
        dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(idx).cuda(), scale_value=scale,
        actual_seq_lengths_kv=[350], query_rope=dev(qr, dt), key_rope=dev(kr, dt), sparse_mode=0,
        return_softmax_lse=True)
    _compare(*(host(t) for t in got), *ref, "bf16")


@pytest.mark.parametrize("B,S1,S2,K", [(1, 2, 5000, 2048), (4, 2, 3000, 1024), (1, 6, 700, 512), (2, 1, 9000, 2048)])
def test_sfa_split_kv_for_few_rows_matches_oracle(B, S1, S2, K):
    """Decode at small batch: with fewer query rows than CTA pairs a row's selected keys are cut into
    parts that run on different pairs and are merged afterwards.  Covers rows whose last parts are
    empty (short sequences), a -1 hole, and the statistics of the merged result."""
    sfa = _sfa()
    rng = np.random.RandomState(300 + B * 10 + S1)
    N1, D = 128, 512
    q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), "bf16")
    k = round_io(rng.randn(B, S2, 1, D).astype(np.float32), "bf16")
    qr = round_io(rng.randn(B, S1, N1, 64).astype(np.float32), "bf16")
    kr = round_io(rng.randn(B, S2, 1, 64).astype(np.float32), "bf16")
    act_k = [S2 - 37 * b for b in range(B)]
    if B > 1:
        act_k[-1] = 300                  # a short sequence: most of its parts are empty
    idx = sparse_indices(301, B, S1, S2, K, 1, 3, [S1] * B, act_k)
    scale = 1.0 / 24.0
    ref = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, [S1] * B, act_k, sparse_mode=3, dtype="bf16")
    dt = torch.bfloat16
    args = (dev(q, dt), dev(k, dt), dev(k, dt), torch.from_numpy(idx).cuda())
    kw = dict(scale_value=scale, actual_seq_lengths_kv=act_k, query_rope=dev(qr, dt), key_rope=dev(kr, dt),
              sparse_mode=3, return_softmax_lse=True)
    sfa.set_kernel("tensor")
    try:
        got = sfa.sparse_flash_attention_triton(*args, **kw)
        again = sfa.sparse_flash_attention_triton(*args, **kw)
    finally:
        sfa.set_kernel("auto")
    _compare(*(host(t) for t in got), *ref, "bf16")
    assert all(torch.equal(x, y) for x, y in zip(got, again))
    # the skipping semantics survive the split: punch a hole into the middle of every row
    idx2 = idx.copy()
    idx2[:, :, :, K // 3] = -1
    sfa.set_kernel("tensor")
    try:
        got2 = sfa.sparse_flash_attention_triton(args[0], args[1], args[2], torch.from_numpy(idx2).cuda(), **kw)
    finally:
        sfa.set_kernel("auto")
    sfa.set_kernel("portable")
    try:
        want2 = sfa.sparse_flash_attention_triton(args[0], args[1], args[2], torch.from_numpy(idx2).cuda(), **kw)
    finally:
        sfa.set_kernel("auto")
    sfa_acceptance_rule(*(host(t) for t in got2), *(host(t) for t in want2))


@pytest.mark.parametrize("dtype,boost,K", [("bf16", 160.0, 256), ("fp16", 40.0, 256), ("bf16", 160.0, 2048)])
def test_sfa_rows_whose_scores_outgrow_the_first_tile_are_exact(dtype, boost, K):
    """The tensor-core kernel scales a row's probabilities by the maximum of the row's FIRST 64 keys
    and hands rows whose later scores exceed it by more than the guard (2^60 in bf16, 2^12 in fp16) to
    the portable kernel.  Rows built to do that - scores that climb by tens of natural units after
    the first tile - and rows that climb by less (handled in place) must both match the oracle; rows
    whose first tile holds the maximum are the ordinary case."""
    sfa = _sfa()
    rng = np.random.RandomState(17)
    B, S1, S2, N1, D = 1, 6, K + 64, 64, 512
    q = rng.randn(B, S1, N1, D).astype(np.float32) * 0.05
    k = rng.randn(B, S2, 1, D).astype(np.float32) * 0.05
    qr = rng.randn(B, S1, N1, 64).astype(np.float32) * 0.05
    kr = rng.randn(B, S2, 1, 64).astype(np.float32) * 0.05
    q[..., 0] = 8.0                                   # score = 8 * k[..., 0] / 24 + small terms
    climb = np.zeros(S2, np.float32)
    climb[64:] = np.linspace(boost * 0.25, boost, S2 - 64)       # natural units x 3: up to boost / 3
    k[0, :, 0, 0] = climb
    q, k, qr, kr = (round_io(x, dtype) for x in (q, k, qr, kr))
    idx = np.full((B, S1, 1, K), -1, np.int32)
    idx[0, 0, 0] = np.arange(K)                        # first tile low, then climbing: outgrows the guard
    idx[0, 1, 0] = np.arange(K)[::-1] + 64             # first tile already holds the maximum
    idx[0, 2, 0] = np.arange(K) // 4                   # climbs slowly (duplicates): stays inside the guard in bf16
    idx[0, 3, 0, :100] = np.arange(100) + 30           # short row crossing the step
    idx[0, 4, 0, :64] = np.arange(64)                  # a single tile
    idx[0, 5, 0] = np.arange(K) + 32
    scale = 1.0 / 24.0
    dt = tdtype(dtype)
    ref = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, [S1], [S2], sparse_mode=0, dtype=dtype)
    sfa.set_kernel("tensor")
    try:
        got = sfa.sparse_flash_attention_triton(dev(q, dt), dev(k, dt), dev(k, dt), dev(idx), scale_value=scale,
                                                query_rope=dev(qr, dt), key_rope=dev(kr, dt), sparse_mode=0,
                                                return_softmax_lse=True)
    finally:
        sfa.set_kernel("auto")
    _compare(host(got[0]), host(got[1]), host(got[2]), ref[0], ref[1], ref[2], dtype)
