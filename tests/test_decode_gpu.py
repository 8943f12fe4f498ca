"""Decode step of the hot path on paged caches (configuration 5 shape at reduced batch / length):
lightning_indexer over a paged index-K cache feeds sparse_flash_attention over a paged KV cache,
S1 = 2 query tokens per sequence (MTP), block_size 128, block table = random permutation."""
import numpy as np
import pytest
import torch

from oracle import lightning_indexer_oracle, sparse_flash_attention_oracle
from oracle import layouts
from oracle.compare import li_reference_rule, sfa_acceptance_rule
from tests.util import host

pytestmark = pytest.mark.gpu


def test_paged_decode_indexer_then_attention():
    from dsa_triton_ascend_b200 import lightning_indexer_triton, sparse_flash_attention_triton
    B, S1, bs, K = 8, 2, 128, 2048
    rng = np.random.RandomState(4)
    lens = rng.randint(2048, 12288, size=B)
    max_blocks = int(-(-lens.max() // bs))
    need = [int(-(-L // bs)) for L in lens]
    nblk = sum(need) + 3
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
    g = torch.Generator(device="cuda").manual_seed(4)
    bf = torch.bfloat16
    ik_cache = torch.randn(nblk, bs, 1, 128, generator=g, device="cuda").to(bf)      # index-K cache
    kv_cache = torch.randn(nblk, bs, 1, 512, generator=g, device="cuda").to(bf)
    kr_cache = torch.randn(nblk, bs, 1, 64, generator=g, device="cuda").to(bf)
    iq = torch.randn(B, S1, 64, 128, generator=g, device="cuda").to(bf)
    iw = torch.randn(B, S1, 64, generator=g, device="cuda") / 8
    q = torch.randn(B, S1, 128, 512, generator=g, device="cuda").to(bf)
    qr = torch.randn(B, S1, 128, 64, generator=g, device="cuda").to(bf)
    table = torch.from_numpy(bt).cuda()
    lens_l = [int(v) for v in lens]

    idx, val = lightning_indexer_triton(iq, ik_cache, iw, actual_seq_lengths_key=lens_l, block_table=table,
                                        layout_key="PA_BSND", sparse_count=K, sparse_mode=3, return_value=True)
    assert idx.shape == (B, S1, 1, K)
    scale = 1.0 / np.sqrt(576.0)
    out, smax, ssum = sparse_flash_attention_triton(
        q, kv_cache, kv_cache, idx, scale_value=scale, block_table=table, actual_seq_lengths_kv=lens_l,
        query_rope=qr, key_rope=kr_cache, layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
        block_size=bs)

    # oracle on the un-paged caches (what the reference wrapper would feed its BSND kernels)
    S2 = max_blocks * bs
    ik = layouts.pa_to_bsnd(host(ik_cache), bt, S2)
    ref_i, ref_v = lightning_indexer_oracle(host(iq), ik, host(iw), [S1] * B, lens_l, sparse_count=K, sparse_mode=3,
                                            return_value=True)
    li_reference_rule(host(idx), host(val), ref_i, ref_v)
    # long rows: a single rounding-boundary flip moves a few neighbours, so count slots, not rows
    assert (host(idx) == ref_i).mean() >= 0.99
    kv = layouts.pa_to_bsnd(host(kv_cache), bt, S2)
    kr = layouts.pa_to_bsnd(host(kr_cache), bt, S2)
    rows = [(b, s) for b in (0, 3, B - 1) for s in range(S1)]
    ref = sparse_flash_attention_oracle(host(q), kv, host(idx), host(qr), kr, scale, [S1] * B, lens_l,
                                        sparse_mode=3, dtype="bf16", rows=rows)
    sel = np.asarray(rows)
    sfa_acceptance_rule(host(out)[sel[:, 0], sel[:, 1]], host(smax)[sel[:, 0], 0, sel[:, 1]],
                        host(ssum)[sel[:, 0], 0, sel[:, 1]], ref[0][sel[:, 0], sel[:, 1]],
                        ref[1][sel[:, 0], 0, sel[:, 1]], ref[2][sel[:, 0], 0, sel[:, 1]])


def test_config5_full_size_sampled_sequences():
    """Configuration 5 at its full size (B=64, S1=2, KV lengths uniform in [16384, 65536], block 128,
    block table = random permutation): properties on every row, the oracle on three sequences."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton, sparse_flash_attention_triton
    B, S1, bs, K = 64, 2, 128, 2048
    rng = np.random.RandomState(4)
    lens = rng.randint(16384, 65537, size=B)
    need = [int(-(-L // bs)) for L in lens]
    max_blocks = max(need)
    nblk = sum(need)
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
    g = torch.Generator(device="cuda").manual_seed(4)
    bf = torch.bfloat16

    def randn_bf16(*shape):   # in pieces: the fp32 staging of a whole cache would double its footprint
        out = torch.empty(shape, dtype=bf, device="cuda")
        step = max(1, (1 << 26) // int(np.prod(shape[1:])))
        for i in range(0, shape[0], step):
            out[i:i + step] = torch.randn((min(step, shape[0] - i),) + tuple(shape[1:]), generator=g, device="cuda")
        return out

    ik_cache = randn_bf16(nblk, bs, 1, 128)
    kv_cache = randn_bf16(nblk, bs, 1, 512)
    kr_cache = randn_bf16(nblk, bs, 1, 64)
    iq = randn_bf16(B, S1, 64, 128)
    iw = torch.randn(B, S1, 64, generator=g, device="cuda") / 8
    q = randn_bf16(B, S1, 128, 512)
    qr = randn_bf16(B, S1, 128, 64)
    table = torch.from_numpy(bt).cuda()
    lens_l = [int(v) for v in lens]
    scale = 1.0 / np.sqrt(576.0)

    idx, val = lightning_indexer_triton(iq, ik_cache, iw, actual_seq_lengths_key=lens_l, block_table=table,
                                        layout_key="PA_BSND", sparse_count=K, sparse_mode=3, return_value=True)
    out, smax, ssum = sparse_flash_attention_triton(
        q, kv_cache, kv_cache, idx, scale_value=scale, block_table=table, actual_seq_lengths_kv=lens_l,
        query_rope=qr, key_rope=kr_cache, layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
        block_size=bs)
    torch.cuda.synchronize()

    # bitwise repeatable at full size (128 rows x 32 tiles keep every ring of the kernel busy)
    for _ in range(3):
        out2, smax2, ssum2 = sparse_flash_attention_triton(
            q, kv_cache, kv_cache, idx, scale_value=scale, block_table=table, actual_seq_lengths_kv=lens_l,
            query_rope=qr, key_rope=kr_cache, layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
            block_size=bs)
        assert torch.equal(out2, out) and torch.equal(smax2, smax) and torch.equal(ssum2, ssum)

    # every row: 2048 distinct positions inside the causal window, values descending, sum >= 1
    lens_t = torch.tensor(lens_l, device="cuda")
    limit = (lens_t[:, None] - S1 + torch.arange(S1, device="cuda")[None, :] + 1)[:, :, None, None]
    assert bool((idx >= 0).all()) and bool((idx < limit).all())
    srt = torch.sort(idx[:, :, 0], dim=-1).values
    assert bool((srt[..., 1:] != srt[..., :-1]).all())
    v = val[:, :, 0].float()
    assert bool((v[..., 1:] <= v[..., :-1]).all())
    assert bool(torch.isfinite(out.float()).all()) and bool((ssum >= 1.0 - 1e-5).all())

    # three sequences against the oracle on their un-paged caches
    pick = [0, int(np.argmax(lens)), B - 1]
    S2 = max_blocks * bs
    sub_bt = np.full((len(pick), max_blocks), -1, np.int32)
    blocks = []
    for i, b in enumerate(pick):
        sub_bt[i, :need[b]] = np.arange(len(blocks), len(blocks) + need[b])
        blocks.extend(bt[b, :need[b]].tolist())
    sel = torch.tensor(blocks, device="cuda")
    ik = layouts.pa_to_bsnd(host(ik_cache[sel]), sub_bt, S2)
    lens_p = [lens_l[b] for b in pick]
    ref_i, ref_v = lightning_indexer_oracle(host(iq[pick]), ik, host(iw[pick]), [S1] * len(pick), lens_p,
                                            sparse_count=K, sparse_mode=3, return_value=True)
    li_reference_rule(host(idx[pick]), host(val[pick]), ref_i, ref_v)
    assert (host(idx[pick]) == ref_i).mean() >= 0.99
    kv = layouts.pa_to_bsnd(host(kv_cache[sel]), sub_bt, S2)
    kr = layouts.pa_to_bsnd(host(kr_cache[sel]), sub_bt, S2)
    ref = sparse_flash_attention_oracle(host(q[pick]), kv, host(idx[pick]), host(qr[pick]), kr, scale,
                                        [S1] * len(pick), lens_p, sparse_mode=3, dtype="bf16")
    sfa_acceptance_rule(host(out[pick]), host(smax[pick]), host(ssum[pick]), ref[0], ref[1], ref[2])


def test_decode_step_replays_from_a_cuda_graph():
    """The decode step (paged indexer -> paged attention) makes no host synchronisation and no
    allocation the caching allocator cannot serve under capture, so it can be captured once and
    replayed; with the lengths and tables in device tensors a replay follows updated inputs."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton, sparse_flash_attention_triton
    B, S1, bs, K = 4, 2, 128, 1024
    rng = np.random.RandomState(44)
    max_blocks, nblk = 40, 200
    g = torch.Generator(device="cuda").manual_seed(44)
    bf = torch.bfloat16
    ik_cache = torch.randn(nblk, bs, 1, 128, generator=g, device="cuda").to(bf)
    kv_cache = torch.randn(nblk, bs, 1, 512, generator=g, device="cuda").to(bf)
    kr_cache = torch.randn(nblk, bs, 1, 64, generator=g, device="cuda").to(bf)
    iq = torch.randn(B, S1, 64, 128, generator=g, device="cuda").to(bf)
    iw = torch.randn(B, S1, 64, generator=g, device="cuda") / 8
    q = torch.randn(B, S1, 128, 512, generator=g, device="cuda").to(bf)
    qr = torch.randn(B, S1, 128, 64, generator=g, device="cuda").to(bf)
    table = torch.from_numpy(rng.permutation(nblk)[:B * max_blocks].reshape(B, max_blocks).astype(np.int32)).cuda()
    lens = torch.tensor([3000, 4100, 2222, 5000], dtype=torch.int32, device="cuda")
    scale = 1.0 / np.sqrt(576.0)

    def step():
        idx, _ = lightning_indexer_triton(iq, ik_cache, iw, actual_seq_lengths_key=lens, block_table=table,
                                          layout_key="PA_BSND", sparse_count=K, sparse_mode=3)
        out, smax, ssum = sparse_flash_attention_triton(
            q, kv_cache, kv_cache, idx, scale_value=scale, block_table=table, actual_seq_lengths_kv=lens,
            query_rope=qr, key_rope=kr_cache, layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
            block_size=bs)
        return idx, out, smax, ssum

    eager = [t.clone() for t in step()]          # also the warm-up that sets the kernels' attributes
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            captured = step()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, captured):
        assert torch.equal(a, b)
    # new step: one more token per sequence, different queries; same graph
    lens += 1
    q.copy_(torch.randn(q.shape, generator=g, device="cuda").to(bf))
    iq.copy_(torch.randn(iq.shape, generator=g, device="cuda").to(bf))
    graph.replay()
    torch.cuda.synchronize()
    replayed = [t.clone() for t in captured]
    fresh = step()
    torch.cuda.synchronize()
    for a, b in zip(replayed, fresh):
        assert torch.equal(a, b)
