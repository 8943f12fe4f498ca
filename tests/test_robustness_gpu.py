"""Edge cases around the paged cache and the failure path: absent blocks inside the valid length
against the oracle (both kernels), a TND query over a paged key for the indexer, block ids beyond
the cache, and a device-side wait that runs out."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import layouts, lightning_indexer_oracle, sparse_flash_attention_oracle
from oracle.compare import li_reference_rule, sfa_acceptance_rule
from oracle.inputs import round_io
from tests.util import host

pytestmark = pytest.mark.gpu


def _bf(rng, *shape):
    return torch.from_numpy(round_io(rng.randn(*shape).astype(np.float32), "bf16")).cuda().to(torch.bfloat16)


@pytest.mark.parametrize("kernel", ["tensor", "portable"])
def test_sfa_absent_block_inside_the_valid_length_reads_as_zero_rows(kernel):
    """sparse_flash_attention_triton.py:1012-1033 un-pages the cache into zeros and skips -1 block
    ids: positions of an absent block stay zero rows that still take part in the softmax (score 0).
    Both kernels must reproduce that (the oracle un-pages the same way)."""
    import dsa_triton_ascend_b200.sparse_flash_attention as sfa
    rng = np.random.RandomState(515)
    B, S1, N1, bs, K = 2, 3, 128, 16, 160
    lens = [300, 200]
    need = [-(-L // bs) for L in lens]
    max_blocks, nblk = max(need), sum(need) + 2
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
    bt[0, 3] = -1           # holes inside the valid length
    bt[0, 11] = -1
    bt[1, 0] = -1
    kv, kr = _bf(rng, nblk, bs, 1, 512), _bf(rng, nblk, bs, 1, 64)
    q, qr = _bf(rng, B, S1, N1, 512), _bf(rng, B, S1, N1, 64)
    idx = np.full((B, S1, 1, K), -1, np.int32)
    for b in range(B):
        for s in range(S1):
            lim = lens[b] - S1 + s + 1
            idx[b, s, 0] = np.sort(rng.permutation(lim)[:K])
    scale = 1.0 / 24.0
    sfa.set_kernel(kernel)
    try:
        out, smax, ssum = sfa.sparse_flash_attention_triton(
            q, kv, kv, torch.from_numpy(idx).cuda(), scale_value=scale, block_table=torch.from_numpy(bt).cuda(),
            actual_seq_lengths_kv=lens, query_rope=qr, key_rope=kr, layout_kv="PA_BSND", sparse_mode=3,
            return_softmax_lse=True, block_size=bs)
    finally:
        sfa.set_kernel("auto")
    S2 = max_blocks * bs
    ref = sparse_flash_attention_oracle(host(q), layouts.pa_to_bsnd(host(kv), bt, S2), idx, host(qr),
                                        layouts.pa_to_bsnd(host(kr), bt, S2), scale, [S1] * B, lens,
                                        sparse_mode=3, dtype="bf16")
    # some selected positions really fall into the holes
    holes = [(0, 3), (0, 11), (1, 0)]
    assert any(((idx[b] // bs) == i).any() for b, i in holes)
    sfa_acceptance_rule(host(out), host(smax), host(ssum), ref[0], ref[1], ref[2])


def test_li_tnd_query_over_a_paged_key_takes_per_batch_key_lengths():
    """A paged cache carries per-batch key lengths even under a TND query (as in
    sparse_flash_attention_triton.py:1379); the result equals the oracle on the un-paged cache."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton
    rng = np.random.RandomState(616)
    lens_q, lens_k, bs, K = [5, 1, 9], [700, 130, 401], 64, 96
    B, T1 = len(lens_q), sum(lens_q)
    need = [-(-L // bs) for L in lens_k]
    max_blocks, nblk = max(need), sum(need)
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
    kc = _bf(rng, nblk, bs, 1, 128)
    q = _bf(rng, T1, 64, 128)
    w = torch.from_numpy(rng.randn(T1, 64).astype(np.float32) / 8).cuda()
    idx, val = lightning_indexer_triton(q, kc, w, actual_seq_lengths_query=np.cumsum(lens_q).tolist(),
                                        actual_seq_lengths_key=lens_k, block_table=torch.from_numpy(bt).cuda(),
                                        layout_query="TND", layout_key="PA_BSND", sparse_count=K, sparse_mode=3,
                                        return_value=True)
    S2 = max_blocks * bs
    kd = layouts.pa_to_bsnd(host(kc), bt, S2)
    qh, wh = host(q), host(w)
    t0 = 0
    for b in range(B):
        L = lens_q[b]
        ri, rv = lightning_indexer_oracle(qh[None, t0:t0 + L], kd[b:b + 1], wh[None, t0:t0 + L], [L], [lens_k[b]],
                                          sparse_count=K, sparse_mode=3, return_value=True)
        li_reference_rule(host(idx[t0:t0 + L])[None], host(val[t0:t0 + L])[None], ri, rv)
        assert (host(idx[t0:t0 + L])[None] == ri).mean() >= 0.98
        t0 += L


@pytest.mark.parametrize("kernel", ["tensor", "portable"])
def test_block_ids_beyond_the_cache_read_as_zero_rows_not_out_of_bounds(kernel):
    """A stale block-table entry (block id >= number of blocks) must not become an out-of-bounds
    read: both operators treat it like an absent block (zero rows)."""
    import dsa_triton_ascend_b200.lightning_indexer as li
    import dsa_triton_ascend_b200.sparse_flash_attention as sfa
    rng = np.random.RandomState(717)
    B, S1, bs, nblk, max_blocks = 1, 2, 128, 6, 4
    L = 4 * bs
    bt_bad = np.array([[2, 1000000, 0, 5]], np.int32)       # entry 1 points far beyond the cache
    bt_hole = np.array([[2, -1, 0, 5]], np.int32)
    ik = _bf(rng, nblk, bs, 1, 128)
    iq = _bf(rng, B, S1, 64, 128)
    iw = torch.from_numpy(rng.randn(B, S1, 64).astype(np.float32) / 8).cuda()
    kv, kr = _bf(rng, nblk, bs, 1, 512), _bf(rng, nblk, bs, 1, 64)
    q, qr = _bf(rng, B, S1, 128, 512), _bf(rng, B, S1, 128, 64)
    K = 64
    res = {}
    for name, bt in (("bad", bt_bad), ("hole", bt_hole)):
        table = torch.from_numpy(bt).cuda()
        li.set_kernel(kernel)
        sfa.set_kernel(kernel)
        try:
            i_, v_ = li.lightning_indexer_triton(iq, ik, iw, actual_seq_lengths_key=[L], block_table=table,
                                                 layout_key="PA_BSND", sparse_count=K, sparse_mode=3, return_value=True)
            idx = torch.arange(100, 100 + K, dtype=torch.int32, device="cuda").repeat(B, S1, 1, 1)   # positions 100..163: blocks 0 and 1
            o_ = sfa.sparse_flash_attention_triton(q, kv, kv, idx, scale_value=1 / 24., block_table=table,
                                                   actual_seq_lengths_kv=[L], query_rope=qr, key_rope=kr,
                                                   layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
                                                   block_size=bs)
        finally:
            li.set_kernel("auto")
            sfa.set_kernel("auto")
        torch.cuda.synchronize()
        res[name] = (i_, v_) + tuple(o_)
    for a, b in zip(res["bad"], res["hole"]):
        assert torch.equal(a, b)


def test_a_device_wait_that_runs_out_is_reported_and_leaves_the_gpu_usable():
    """Every wait inside the tensor-core kernels is bounded; one that runs out sets the status word
    of the call's workspace.  The library's self-test kernel makes exactly that happen (a barrier
    nothing signals, no copy or MMA in flight): the status reads DSA_ERR_DEVICE_WAIT, check_status()
    raises, and the next ordinary call on the same GPU is correct."""
    import dsa_triton_ascend_b200 as pkg
    from dsa_triton_ascend_b200 import _cabi, _host
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    stream = _host.current_stream(ws.device)
    assert _cabi.lib.dsa_selftest_wait_timeout(ws.data_ptr(), ws.numel(), stream) == 0
    st = _cabi.lib.dsa_read_device_status(ws.data_ptr(), stream)
    assert st != 0 and "wait" in _cabi.status_string(st)
    _host.note_launch("selftest", ws, ws.device)
    with pytest.raises(RuntimeError, match="wait"):
        pkg.check_status()
    _host._last_ws.pop(("selftest", ws.device.index))
    # a status word written by the host surfaces the same way
    ws.zero_()
    assert _cabi.lib.dsa_read_device_status(ws.data_ptr(), stream) == 0
    ws[:4] = torch.tensor([1, 0, 0, 0], dtype=torch.uint8, device="cuda")
    assert _cabi.lib.dsa_read_device_status(ws.data_ptr(), stream) != 0
    # the context is intact: an ordinary call right afterwards matches the oracle
    rng = np.random.RandomState(818)
    q, k = _bf(rng, 1, 64, 64, 128), _bf(rng, 1, 64, 1, 128)
    w = torch.from_numpy(rng.randn(1, 64, 64).astype(np.float32) / 8).cuda()
    idx, val = pkg.lightning_indexer_triton(q, k, w, sparse_count=16, return_value=True)
    ri, rv = lightning_indexer_oracle(host(q), host(k), host(w), [64], [64], sparse_count=16, sparse_mode=3,
                                      return_value=True)
    li_reference_rule(host(idx), host(val), ri, rv)
    pkg.check_status()
