"""Query-row sharding of the hot path across the GPUs of one node.

Both operators are row-parallel: one output row (one query token) depends on its own q / weight /
index row and on the keys of its sequence, never on another row.  The path therefore shards by
query rows with the (small) key tensors replicated and needs no collective; `torch.distributed`
is only used by callers for barriers and for gathering results when they want them in one place.

A contiguous slice [r0, r1) of the S1 query rows of a BSND problem is itself a valid BSND problem
for the unchanged operators: with act_q' = r1 - r0 and act_k' = act_k - (act_q - r1) the
rightDownCausal limit of local row s' is act_k' - act_q' + s' + 1 = act_k - act_q + (r0 + s') + 1,
the global row's limit, and keys at or beyond act_k' are hidden from every row of the slice in the
global problem as well.  `row_slices` balances the slices by causal work (the number of visible
keys), not by row count.
"""
from typing import List, Sequence, Tuple


def causal_work(act_q: int, act_k: int, r0: int, r1: int, cap: int = 0) -> int:
    """Visible (query, key) pairs of rows [r0, r1) under the rightDownCausal mask; `cap` > 0 clips each
    row's count (top-k attention only touches min(cap, visible) keys)."""
    total = 0
    for s in range(r0, r1):
        v = min(max(act_k - act_q + s + 1, 0), act_k)
        total += min(v, cap) if cap > 0 else v
    return total


def row_slices(act_q: int, act_k: int, world: int, cap: int = 0, align: int = 8) -> List[Tuple[int, int]]:
    """Split rows [0, act_q) into `world` contiguous slices of nearly equal causal work.

    Boundaries are multiples of `align` (the tensor-core kernels work on groups of 8 rows)."""
    if world < 1:
        raise ValueError("world must be positive")
    per_row = []
    for s in range(act_q):
        v = min(max(act_k - act_q + s + 1, 0), act_k)
        per_row.append(min(v, cap) if cap > 0 else v)
    total = sum(per_row)
    bounds, acc, r = [0], 0, 0
    for i in range(1, world):
        target = total * i / world
        while r < act_q and acc + per_row[r] / 2 < target:
            acc += per_row[r]
            r += 1
        b = min(act_q, (r + align // 2) // align * align)
        b = max(b, bounds[-1])
        bounds.append(b)
        # keep the running sum consistent with the aligned boundary
        acc, r = sum(per_row[:b]), b
    bounds.append(act_q)
    return [(bounds[i], bounds[i + 1]) for i in range(world)]


def sequence_shards(kv_lengths: Sequence[int], world: int) -> List[List[int]]:
    """Decode: whole sequences per rank (each rank holds its own sequences' paged cache).  The
    indexer reads every cached key of a sequence, so sequences are dealt out longest first to the
    rank with the least cached keys so far; each rank's list is returned in ascending order."""
    if world < 1:
        raise ValueError("world must be positive")
    shards: List[List[int]] = [[] for _ in range(world)]
    load = [0] * world
    for b in sorted(range(len(kv_lengths)), key=lambda i: (-int(kv_lengths[i]), i)):
        r = min(range(world), key=lambda i: (load[i], len(shards[i]), i))
        shards[r].append(b)
        load[r] += int(kv_lengths[b])
    return [sorted(x) for x in shards]


def slice_lengths(act_q: int, act_k: int, r0: int, r1: int) -> Tuple[int, int]:
    """(act_q', act_k') that make rows [r0, r1) a stand-alone problem (see module docstring)."""
    if not (0 <= r0 <= r1 <= act_q):
        raise ValueError("slice outside the sequence")
    return r1 - r0, max(act_k - (act_q - r1), 0)


def lightning_indexer_rows(query, key, weights, r0: int, r1: int, act_q: Sequence[int] = None,
                           act_k: Sequence[int] = None, **kw):
    """lightning_indexer_triton on query rows [r0, r1) of every sequence of a BSND batch.

    `query` / `weights` are the FULL tensors (or any tensors whose dim 1 covers [r0, r1)); the key is
    the replicated full key.  Returns what the full call would return for those rows."""
    from .lightning_indexer import lightning_indexer_triton
    B, S1 = query.shape[0], query.shape[1]
    S2 = key.shape[1]
    act_q = [S1] * B if act_q is None else [int(v) for v in act_q]
    act_k = [S2] * B if act_k is None else [int(v) for v in act_k]
    lq, lk = [], []
    for b in range(B):
        e = min(r1, act_q[b])
        s = min(r0, e)
        q_, k_ = slice_lengths(act_q[b], act_k[b], s, e)
        lq.append(q_)
        lk.append(k_)
    return lightning_indexer_triton(query[:, r0:r1], key, weights[:, r0:r1], actual_seq_lengths_query=lq,
                                    actual_seq_lengths_key=lk, **kw)


def sparse_flash_attention_rows(query, key, sparse_indices, query_rope, key_rope, r0: int, r1: int,
                                act_q: Sequence[int] = None, act_k: Sequence[int] = None, **kw):
    """sparse_flash_attention_triton on query rows [r0, r1) of every sequence of a BSND batch."""
    from .sparse_flash_attention import sparse_flash_attention_triton
    B, S1 = query.shape[0], query.shape[1]
    S2 = key.shape[1]
    act_q = [S1] * B if act_q is None else [int(v) for v in act_q]
    act_k = [S2] * B if act_k is None else [int(v) for v in act_k]
    lq, lk = [], []
    for b in range(B):
        e = min(r1, act_q[b])
        s = min(r0, e)
        q_, k_ = slice_lengths(act_q[b], act_k[b], s, e)
        lq.append(q_)
        lk.append(k_)
    return sparse_flash_attention_triton(
        query[:, r0:r1], key, key, sparse_indices[:, r0:r1], actual_seq_lengths_query=lq,
        actual_seq_lengths_kv=lk, query_rope=query_rope[:, r0:r1], key_rope=key_rope, **kw)


# ---- TND batches: contiguous token ranges -----------------------------------------------------------
def tnd_token_slices(cum_q: Sequence[int], cum_k: Sequence[int], world: int, cap: int = 0,
                     align: int = 8) -> List[Tuple[int, int]]:
    """Split the T1 tokens of a TND batch into `world` contiguous ranges of nearly equal causal work
    (visible keys per token, clipped at `cap` for top-k attention).  Boundaries are multiples of
    `align` tokens."""
    if world < 1:
        raise ValueError("world must be positive")
    per_tok = []
    pq = pk = 0
    for cq, ck in zip(cum_q, cum_k):
        aq, ak = int(cq) - pq, int(ck) - pk
        for s in range(aq):
            v = min(max(ak - aq + s + 1, 0), ak)
            per_tok.append(min(v, cap) if cap > 0 else v)
        pq, pk = int(cq), int(ck)
    total_tok, total = len(per_tok), sum(per_tok)
    bounds, acc, r = [0], 0, 0
    for i in range(1, world):
        target = total * i / world
        while r < total_tok and acc + per_tok[r] / 2 < target:
            acc += per_tok[r]
            r += 1
        b = max(min(total_tok, (r + align // 2) // align * align), bounds[-1])
        bounds.append(b)
        acc, r = sum(per_tok[:b]), b
    bounds.append(total_tok)
    return [(bounds[i], bounds[i + 1]) for i in range(world)]


def tnd_slice(cum_q: Sequence[int], cum_k: Sequence[int], t0: int, t1: int):
    """Tokens [t0, t1) of a TND batch as a stand-alone TND problem.

    Returns (cum_q', cum_k', key_ranges): the cumulative lengths of the sequences the range touches
    and, per such sequence, the rows [k0, k1) of the packed key tensor it needs.  A sequence cut at
    its end keeps act_k' = act_k - (act_q - r1) keys (see the module docstring), so the keys of the
    slice are the concatenation of those row ranges rather than a view of the full key tensor."""
    if not (0 <= t0 <= t1 <= (int(cum_q[-1]) if len(cum_q) else 0)):
        raise ValueError("token range outside the batch")
    out_q, out_k, ranges = [], [], []
    pq = pk = 0
    for cq, ck in zip(cum_q, cum_k):
        cq, ck = int(cq), int(ck)
        lo, hi = max(t0, pq), min(t1, cq)
        if hi > lo:
            q_, k_ = slice_lengths(cq - pq, ck - pk, lo - pq, hi - pq)
            out_q.append((out_q[-1] if out_q else 0) + q_)
            out_k.append((out_k[-1] if out_k else 0) + k_)
            ranges.append((pk, pk + k_))
        pq, pk = cq, ck
    return out_q, out_k, ranges


def _cat_rows(t, ranges):
    import torch
    if len(ranges) == 1:
        return t[ranges[0][0]:ranges[0][1]]
    return torch.cat([t[a:b] for a, b in ranges], dim=0)


def lightning_indexer_tokens(query, key, weights, cum_q: Sequence[int], cum_k: Sequence[int], t0: int,
                             t1: int, **kw):
    """lightning_indexer_triton on tokens [t0, t1) of a TND batch (TND query and key).  Returns what
    the full call returns for those tokens (indices are positions inside each token's own sequence)."""
    from .lightning_indexer import lightning_indexer_triton
    cq, ck, ranges = tnd_slice(cum_q, cum_k, t0, t1)
    return lightning_indexer_triton(query[t0:t1], _cat_rows(key, ranges), weights[t0:t1],
                                    actual_seq_lengths_query=cq, actual_seq_lengths_key=ck,
                                    layout_query="TND", layout_key="TND", **kw)


def sparse_flash_attention_tokens(query, key, sparse_indices, query_rope, key_rope, cum_q: Sequence[int],
                                  cum_k: Sequence[int], t0: int, t1: int, **kw):
    """sparse_flash_attention_triton on tokens [t0, t1) of a TND batch (TND query and KV)."""
    from .sparse_flash_attention import sparse_flash_attention_triton
    cq, ck, ranges = tnd_slice(cum_q, cum_k, t0, t1)
    k = _cat_rows(key, ranges)
    return sparse_flash_attention_triton(
        query[t0:t1], k, k, sparse_indices[t0:t1], actual_seq_lengths_query=cq, actual_seq_lengths_kv=ck,
        query_rope=query_rope[t0:t1], key_rope=_cat_rows(key_rope, ranges), layout_query="TND", layout_kv="TND", **kw)
