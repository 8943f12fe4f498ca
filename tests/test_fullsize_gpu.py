"""The two benchmarked configurations at their full size, on the benchmark's own seeded inputs
(dsa_triton_ascend_b200.synthetic: numpy RandomState(2) / RandomState(3)), against the oracle on
sampled rows; and row / token slices of the operators against the unsliced calls, bit for bit."""
import numpy as np
import pytest
import torch

from dsa_triton_ascend_b200 import synthetic
from oracle import lightning_indexer_oracle, sparse_flash_attention_oracle
from oracle.compare import li_reference_rule, sfa_acceptance_rule, sfa_reference_rule
from tests.util import host, li_gap_ok

pytestmark = pytest.mark.gpu


def test_config3_full_size_64_rows_against_the_oracle():
    """Indexer, B=1, S=8192, 64 heads, D=128, k=2048, rightDownCausal: 64 rows spread over the
    sequence.  Reference rule on all of them, identical index SETS wherever the fp32 gap between the
    k-th and (k+1)-th score exceeds 1e-3 relative, nearly all rows identical position for position."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton
    c = synthetic.config3("cuda")
    S, K = c["S"], c["sparse_count"]
    idx, val = lightning_indexer_triton(c["q"], c["k"], c["w"], sparse_count=K, sparse_mode=3, return_value=True)
    pos = sorted(set([0, 1, 7, 8, 2046, 2047, 2048, 2049, 4095, 4096, S - 2, S - 1] +
                     np.linspace(100, S - 100, 52).astype(int).tolist()))
    assert len(pos) >= 64
    rows = [(0, int(s)) for s in pos]
    qn, kn, wn = host(c["q"]), host(c["k"]), host(c["w"])
    ref_i, ref_v = lightning_indexer_oracle(qn, kn, wn, [S], [S], sparse_count=K, sparse_mode=3,
                                            return_value=True, rows=rows)
    got_i, got_v = host(idx)[0, pos], host(val)[0, pos]
    exp_i, exp_v = ref_i[0, pos], ref_v[0, pos]
    li_reference_rule(got_i, got_v, exp_i, exp_v)
    gap = li_gap_ok(qn, kn, wn, [S], [S], rows, 1, K, 3).reshape(-1)
    a, b = got_i.reshape(len(pos), K), exp_i.reshape(len(pos), K)
    assert gap.sum() >= len(pos) // 2          # the rule below must bite on most rows
    for r in range(len(pos)):
        if gap[r]:
            assert set(a[r].tolist()) == set(b[r].tolist()), f"row {pos[r]}: index set differs"
    # io-dtype ranking reproduces the golden position for position except where the two fp32
    # accumulation orders round a score to different bf16 values
    assert (a == b).mean() >= 0.99
    assert (a == b).all(axis=1).mean() >= 0.5


def _sfa_row_oracle(t, cum, lens, q, k, qr, kr, idx_row, scale, K):
    b = int(np.searchsorted(cum, t, side="right"))
    s0 = 0 if b == 0 else int(cum[b - 1])
    s, L = t - s0, lens[b]
    N1, D = q.shape[1], q.shape[2]
    qq = np.zeros((1, L, N1, D), np.float32)
    qq[0, s] = host(q[t])
    qqr = np.zeros((1, L, N1, 64), np.float32)
    qqr[0, s] = host(qr[t])
    ii = np.full((1, L, 1, K), -1, np.int32)
    ii[0, s] = idx_row
    ref = sparse_flash_attention_oracle(qq, host(k[s0:s0 + L])[None], ii, qqr, host(kr[s0:s0 + L])[None], scale,
                                        [L], [L], sparse_mode=3, dtype="bf16", rows=[(0, s)])
    return ref[0][0, s], ref[1][0, 0, s], ref[2][0, 0, s]


def test_config4_full_size_with_indexer_indices_against_the_oracle():
    """Attention, TND 8192/4096/2048/1024, 128 heads, D=512+64, top-k 2048, indices produced by the
    indexer on the same seed: >= 32 tokens spread over the four sequences (first and last token of
    each, tokens with fewer than 2048 visible keys, tokens around the 2048 boundary) against the
    oracle, softmax invariants on every token."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton, sparse_flash_attention_triton
    c = synthetic.config4("cuda")
    lens, cum, T, K = c["lens"], c["cum"], c["T"], c["topk"]
    idx, _ = lightning_indexer_triton(c["qi"], c["ki"], c["wi"], actual_seq_lengths_query=cum,
                                      actual_seq_lengths_key=cum, layout_query="TND", layout_key="TND",
                                      sparse_count=K, sparse_mode=3, max_seqlen_key=max(lens))
    out, smax, ssum = sparse_flash_attention_triton(
        c["q"], c["k"], c["k"], idx, scale_value=c["scale"], actual_seq_lengths_query=cum,
        actual_seq_lengths_kv=cum, query_rope=c["qr"], key_rope=c["kr"], layout_query="TND", layout_kv="TND",
        sparse_mode=3, return_softmax_lse=True)
    assert bool(torch.isfinite(out.float()).all()) and bool((ssum >= 1.0 - 1e-6).all())
    toks, s0 = [], 0
    for L in lens:
        local = {0, 1, 63, 64, 100, L // 3, L // 2, L - 2, L - 1}
        if L > 2048:
            local |= {2046, 2047, 2048, 2049, (L + 2048) // 2}
        toks += [s0 + s for s in sorted(local) if 0 <= s < L]
        s0 += L
    assert len(toks) >= 32
    idx_h = host(idx)
    for t in toks:
        ro, rm, rs = _sfa_row_oracle(t, cum, lens, c["q"], c["k"], c["qr"], c["kr"], idx_h[t], c["scale"], K)
        sfa_acceptance_rule(host(out[t]), host(smax[0, t]), host(ssum[0, t]), ro, rm, rs)
        assert sfa_reference_rule(host(out[t]), ro, "bf16", pct_thd=99.0)


def test_row_and_token_slices_equal_the_unsliced_operators_bit_for_bit():
    """What every rank of a multi-GPU run computes: a slice of the query rows with the keys
    replicated.  2, 4 and 8 slices (balanced by causal work) concatenate to exactly the unsliced
    outputs: indices, values, attention output and both statistics."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton, sparse_flash_attention_triton
    from dsa_triton_ascend_b200.sharding import (lightning_indexer_rows, lightning_indexer_tokens, row_slices,
                                                 sparse_flash_attention_rows, sparse_flash_attention_tokens,
                                                 tnd_token_slices)
    g = torch.Generator(device="cuda").manual_seed(71)
    bf = torch.bfloat16
    # ---- indexer, BSND, one sequence
    S, K = 1536, 512
    q = torch.randn(1, S, 64, 128, generator=g, device="cuda").to(bf)
    k = torch.randn(1, S, 1, 128, generator=g, device="cuda").to(bf)
    w = torch.randn(1, S, 64, generator=g, device="cuda") / 8
    full_i, full_v = lightning_indexer_triton(q, k, w, sparse_count=K, sparse_mode=3, return_value=True)
    for world in (2, 4, 8):
        parts = [lightning_indexer_rows(q, k, w, r0, r1, sparse_count=K, sparse_mode=3, return_value=True)
                 for r0, r1 in row_slices(S, S, world)]
        assert torch.equal(torch.cat([p[0] for p in parts], dim=1), full_i)
        assert torch.equal(torch.cat([p[1] for p in parts], dim=1), full_v)
    # ---- attention, BSND, indices from the indexer above
    aq = torch.randn(1, S, 128, 512, generator=g, device="cuda").to(bf)
    aqr = torch.randn(1, S, 128, 64, generator=g, device="cuda").to(bf)
    ak = torch.randn(1, S, 1, 512, generator=g, device="cuda").to(bf)
    akr = torch.randn(1, S, 1, 64, generator=g, device="cuda").to(bf)
    kw = dict(scale_value=1.0 / 24.0, sparse_mode=3, return_softmax_lse=True)
    full = sparse_flash_attention_triton(aq, ak, ak, full_i, query_rope=aqr, key_rope=akr, **kw)
    for world in (2, 4, 8):
        parts = [sparse_flash_attention_rows(aq, ak, full_i, aqr, akr, r0, r1, **kw)
                 for r0, r1 in row_slices(S, S, world, cap=K)]
        assert torch.equal(torch.cat([p[0] for p in parts], dim=1), full[0])
        assert torch.equal(torch.cat([p[1] for p in parts], dim=2), full[1])
        assert torch.equal(torch.cat([p[2] for p in parts], dim=2), full[2])
    # ---- TND batch: token ranges that cut through sequences
    lens = [700, 300, 200, 100]
    cum = np.cumsum(lens).tolist()
    T = cum[-1]
    tq = torch.randn(T, 64, 128, generator=g, device="cuda").to(bf)
    tk = torch.randn(T, 1, 128, generator=g, device="cuda").to(bf)
    tw = torch.randn(T, 64, generator=g, device="cuda") / 8
    K2 = 256
    fi, fv = lightning_indexer_triton(tq, tk, tw, actual_seq_lengths_query=cum, actual_seq_lengths_key=cum,
                                      layout_query="TND", layout_key="TND", sparse_count=K2, return_value=True)
    bq = torch.randn(T, 128, 512, generator=g, device="cuda").to(bf)
    bqr = torch.randn(T, 128, 64, generator=g, device="cuda").to(bf)
    bk = torch.randn(T, 1, 512, generator=g, device="cuda").to(bf)
    bkr = torch.randn(T, 1, 64, generator=g, device="cuda").to(bf)
    fa = sparse_flash_attention_triton(bq, bk, bk, fi, actual_seq_lengths_query=cum, actual_seq_lengths_kv=cum,
                                       query_rope=bqr, key_rope=bkr, layout_query="TND", layout_kv="TND", **kw)
    for world in (2, 4, 8):
        sl = tnd_token_slices(cum, cum, world, cap=K2)
        assert sl[0][0] == 0 and sl[-1][1] == T and all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
        pi = [lightning_indexer_tokens(tq, tk, tw, cum, cum, t0, t1, sparse_count=K2, return_value=True)
              for t0, t1 in sl if t1 > t0]
        assert torch.equal(torch.cat([p[0] for p in pi], dim=0), fi)
        assert torch.equal(torch.cat([p[1] for p in pi], dim=0), fv)
        pa = [sparse_flash_attention_tokens(bq, bk, fi, bqr, bkr, cum, cum, t0, t1, **kw) for t0, t1 in sl if t1 > t0]
        assert torch.equal(torch.cat([p[0] for p in pa], dim=0), fa[0])
        assert torch.equal(torch.cat([p[1] for p in pa], dim=1), fa[1])
        assert torch.equal(torch.cat([p[2] for p in pa], dim=1), fa[2])
