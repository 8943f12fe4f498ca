"""Numpy oracle for lightning_indexer (test infrastructure only, never shipped).

Restates lightning_indexer_numpy.py:38-111 (`lightning_indexer_golden_bsnd`):
per (b, s1, n2) the score of key s2 is
    sum_{g in group n2} relu(Q[b,s1,g,:] . K[b,s2,n2,:]) * W[b,s1,g]
accumulated in fp32 one head at a time (lightning_indexer_numpy.py:78-83), masked by
the rightDownCausal limit and act_k (:85-90), rounded to the io dtype (:92, `_quantize`
:27-35), ranked by (rounded score descending, index ascending) (:94-97), and the first
min(act_k, sparse_count) finite entries are emitted; the rest stay index -1 / value 0
(:66-67, :99-105).

Extensions used by the tests (none changes the default behaviour):
  * `rank_dtype="fp32"` ranks the un-rounded fp32 scores, which is what the reference's
    device path does (lightning_indexer_triton.py:343-361 runs top-k on fp32 scores);
    the emitted values are still rounded to the io dtype (:546).
  * `rows` restricts the computation to a list of (b, s1) pairs so that full-size
    configurations can be spot-checked in seconds.
"""
import numpy as np


def round_bf16(x):
    """fp32 -> bf16 -> fp32, round-to-nearest-even (lightning_indexer_numpy.py:20-24)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((u + bias) & np.uint32(0xFFFF0000)).view(np.float32)


def quantize(x, value_dtype):
    """Round fp32 scores to the io dtype and back (lightning_indexer_numpy.py:27-35)."""
    if value_dtype == "fp16":
        return x.astype(np.float16).astype(np.float32)
    if value_dtype == "fp32":
        return np.asarray(x, dtype=np.float32)
    return round_bf16(x)


def causal_limit(act_q, act_k, s1, s2_len, sparse_mode):
    """Number of visible keys of query row s1 (lightning_indexer_numpy.py:85-90)."""
    if sparse_mode == 3:
        lim = min(max(act_k - act_q + s1 + 1, 0), s2_len)
        return max(min(lim, act_k), 0)
    return max(min(act_k, s2_len), 0)


def row_scores(q_row, k_b, w_row, n2, group):
    """fp32 scores of one (b, s1, n2): head-by-head accumulation, as :78-83."""
    scores = np.zeros(k_b.shape[0], dtype=np.float32)
    k_mat = k_b[:, n2, :]
    for g in range(n2 * group, (n2 + 1) * group):
        dots = k_mat @ q_row[g, :]
        scores += np.maximum(dots, 0.0) * w_row[g]
    return scores


def lightning_indexer_oracle(q, k, w, act_q, act_k, sparse_count=2048, sparse_mode=3,
                             return_value=False, value_dtype="bf16", rank_dtype=None,
                             rows=None):
    """BSND lightning indexer.

    q [B,S1,N1,D], k [B,S2,N2,D], w [B,S1,N1] fp32 arrays (already rounded to the io
    dtype by the caller); act_q/act_k per-batch lengths.  Returns (indices int32
    [B,S1,N2,sparse_count], values fp32 same shape; zeros unless `return_value`).
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    w = np.asarray(w, dtype=np.float32)
    B, S1, N1, _ = q.shape
    S2, N2 = k.shape[1], k.shape[2]
    group = N1 // N2
    rank_dtype = rank_dtype or value_dtype

    idx_out = np.full((B, S1, N2, sparse_count), -1, dtype=np.int32)
    val_out = np.zeros((B, S1, N2, sparse_count), dtype=np.float32)

    if rows is None:
        rows = [(b, s1) for b in range(B) for s1 in range(int(act_q[b]))]
    positions = np.arange(S2, dtype=np.int64)
    for b, s1 in rows:
        aq, ak = int(act_q[b]), int(act_k[b])
        if s1 >= aq:
            continue
        for n2 in range(N2):
            scores = row_scores(q[b, s1], k[b], w[b, s1], n2, group)
            if sparse_mode == 3:
                lim = min(max(ak - aq + s1 + 1, 0), S2)
                scores[lim:] = -np.inf
            scores[ak:] = -np.inf
            emitted = quantize(scores, value_dtype)
            ranked = emitted if rank_dtype == value_dtype else quantize(scores, rank_dtype)
            order = np.lexsort((positions, -ranked))
            take = min(ak, sparse_count, S2)
            # slot i receives order[i] unless that score is -inf (slot keeps -1 / 0.0)
            head = order[:take]
            finite = ranked[head] != -np.inf
            slots = np.nonzero(finite)[0]
            idx_out[b, s1, n2, slots] = head[finite]
            val_out[b, s1, n2, slots] = emitted[head[finite]]
    if not return_value:
        val_out = np.zeros_like(val_out)
    return idx_out, val_out
