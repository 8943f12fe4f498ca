"""Layout adapters of the oracle (test infrastructure only).

The reference normalises every layout to dense BSND with host copy loops and then runs
the BSND path; these helpers restate that normalisation in numpy so that the oracle can
judge the kernels' in-kernel offset arithmetic:
  * TND <-> padded BSND: lightning_indexer_triton.py:294-340,
    sparse_flash_attention_triton.py:975-1009 (cumulative lengths -> per batch, rows
    copied sequence by sequence, padding zero);
  * paged cache -> dense: sparse_flash_attention_triton.py:1012-1033 (`_pa_to_bsnd`;
    block id -1 skipped, dense length = max_blocks * block_size);
  * softmax stats (B,1,S1,N1) -> (1,T1,N1): sparse_flash_attention_triton.py:1446-1453.
"""
import numpy as np


def cumulative_to_lengths(cum):
    cum = np.asarray(cum, dtype=np.int64)
    return np.diff(np.concatenate([[0], cum])).astype(np.int64)


def tnd_to_bsnd(x, lengths):
    lengths = [int(v) for v in lengths]
    max_s = max(lengths) if lengths else 0
    out = np.zeros((len(lengths), max_s) + tuple(x.shape[1:]), dtype=x.dtype)
    start = 0
    for b, n in enumerate(lengths):
        out[b, :n] = x[start:start + n]
        start += n
    return out


def bsnd_to_tnd(x, lengths):
    lengths = [int(v) for v in lengths]
    parts = [x[b, :n] for b, n in enumerate(lengths)]
    if not parts:
        return np.zeros((0,) + tuple(x.shape[2:]), dtype=x.dtype)
    return np.concatenate(parts, axis=0)


def pa_to_bsnd(cache, block_table, max_s2):
    """cache [num_blocks, block_size, N, Dx] + block_table [B, max_blocks] -> [B, max_s2, N, Dx]."""
    _, block_size, n, dx = cache.shape
    bt = np.asarray(block_table)
    out = np.zeros((bt.shape[0], max_s2, n, dx), dtype=cache.dtype)
    for b in range(bt.shape[0]):
        for i in range(bt.shape[1]):
            blk = int(bt[b, i])
            if blk == -1:
                continue
            dst = i * block_size
            if dst >= max_s2:
                break
            end = min(dst + block_size, max_s2)
            out[b, dst:end] = cache[blk, :end - dst]
    return out


def stats_bsnd_to_tnd(stats, lengths):
    """(B,1,S1,N1) -> (1,T1,N1)."""
    return bsnd_to_tnd(stats.transpose(0, 2, 1, 3), lengths).transpose(1, 0, 2)


def li_oracle_tnd(q, k, w, cu_q, cu_k, **kw):
    """TND lightning indexer through the BSND oracle (indices are sequence-local)."""
    from .li_oracle import lightning_indexer_oracle
    lq, lk = cumulative_to_lengths(cu_q), cumulative_to_lengths(cu_k)
    idx, val = lightning_indexer_oracle(tnd_to_bsnd(q, lq), tnd_to_bsnd(k, lk),
                                        tnd_to_bsnd(w, lq), lq, lk, **kw)
    return bsnd_to_tnd(idx, lq), bsnd_to_tnd(val, lq)


def sfa_oracle_tnd(q, k, idx, qr, kr, scale, cu_q, cu_k, **kw):
    """TND sparse flash attention through the BSND oracle."""
    from .sfa_oracle import sparse_flash_attention_oracle
    lq, lk = cumulative_to_lengths(cu_q), cumulative_to_lengths(cu_k)
    out, smax, ssum = sparse_flash_attention_oracle(
        tnd_to_bsnd(q, lq), tnd_to_bsnd(k, lk), tnd_to_bsnd(idx, lq),
        tnd_to_bsnd(qr, lq), tnd_to_bsnd(kr, lk), scale, lq, lk, **kw)
    return bsnd_to_tnd(out, lq), stats_bsnd_to_tnd(smax, lq), stats_bsnd_to_tnd(ssum, lq)
