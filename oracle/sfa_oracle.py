"""Numpy oracle for sparse_flash_attention forward (test infrastructure only).

Restates sparse_flash_attention_numpy.py:63-160 (`sparse_flash_attention_golden_bsnd`)
and its position expansion `_gather_positions` (:38-60).  MLA-absorb, one KV head:
    score[h,p] = (q_nope[h].k_nope[p] + q_rope[h].k_rope[p]) * scale
    out[h]     = softmax_p(score[h,:]) @ k_nope[p]          (value == key[..., :D])
The normalised probabilities are rounded to the io dtype before the second product
(:131-137,149) and the output is rounded to the io dtype (:155-159).
softmax_max is the maximum scaled score, softmax_sum = sum exp(score - max) (:145-153).
Rows outside the causal window or without any valid position stay zero (:120-133).

`rows` restricts the work to a list of (b, s1) pairs for spot checks of big shapes.
"""
import math
import numpy as np

from .li_oracle import round_bf16

BF16 = "bfloat16"


def gather_positions(idx_row, sparse_block_size, threshold, act_k):
    """Token positions selected by one sparse-index row (:38-60).

    Only the first min(len, ceil(threshold / block)) entries are scanned and the scan
    stops at the first -1 (front-packed contract); blocks are clipped to
    [0, min(threshold, act_k)).
    """
    scan = min(idx_row.shape[0], math.ceil(threshold / sparse_block_size))
    out = []
    for i in range(scan):
        sid = int(idx_row[i])
        if sid == -1:
            break
        begin = sid * sparse_block_size
        end = min(begin + sparse_block_size, act_k)
        if begin >= threshold:
            continue
        out.extend(range(begin, min(end, threshold)))
    return out


def _round_io(x, dtype):
    if dtype == np.float16 or dtype == "fp16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == BF16 or dtype == "bf16":
        return round_bf16(x)
    return x


def sparse_flash_attention_oracle(q_nope, k_nope, sparse_indices, q_rope, k_rope, scale_value,
                                  act_q, act_k, sparse_block_size=1, sparse_mode=3,
                                  return_softmax_lse=True, dtype=BF16, rows=None):
    """BSND sparse flash attention forward.

    q_nope [B,S1,N1,D], k_nope [B,S2,1,D], sparse_indices [B,S1,1,K] int32,
    q_rope [B,S1,N1,Dr], k_rope [B,S2,1,Dr]; returns (out [B,S1,N1,D] fp32 holding
    io-dtype-rounded values, softmax_max [B,1,S1,N1], softmax_sum [B,1,S1,N1]).
    """
    qn = np.asarray(q_nope, dtype=np.float32)
    kn = np.asarray(k_nope, dtype=np.float32)
    qr = np.asarray(q_rope, dtype=np.float32)
    kr = np.asarray(k_rope, dtype=np.float32)
    B, S1, N1, D = qn.shape

    out = np.zeros((B, S1, N1, D), dtype=np.float32)
    smax = np.zeros((B, 1, S1, N1), dtype=np.float32)
    ssum = np.zeros((B, 1, S1, N1), dtype=np.float32)

    if rows is None:
        rows = [(b, s1) for b in range(B) for s1 in range(int(act_q[b]))]
    for b, s1 in rows:
        aq, ak = int(act_q[b]), int(act_k[b])
        if s1 >= aq:
            continue
        threshold = ak if sparse_mode == 0 else ak - aq + s1 + 1
        if threshold <= 0:
            continue
        pos = gather_positions(sparse_indices[b, s1, 0, :], sparse_block_size, threshold, ak)
        if not pos:
            continue
        pos = np.asarray(pos, dtype=np.int64)
        k_sp = np.concatenate([kn[b, pos, 0, :], kr[b, pos, 0, :]], axis=-1)
        v_sp = kn[b, pos, 0, :]
        for h in range(N1):
            q_full = np.concatenate([qn[b, s1, h], qr[b, s1, h]], axis=-1)
            scores = (k_sp @ q_full) * scale_value
            x_max = scores.max()
            e = np.exp(scores - x_max)
            x_sum = e.sum()
            probs = _round_io(e / x_sum, dtype)
            out[b, s1, h, :] = probs @ v_sp
            if return_softmax_lse:
                smax[b, 0, s1, h] = x_max
                ssum[b, 0, s1, h] = x_sum
    return _round_io(out, dtype), smax, ssum
