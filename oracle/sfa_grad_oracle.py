"""Numpy oracle for sparse_flash_attention backward (test infrastructure only).

Restates sparse_flash_attention_grad_numpy.py:34-143
(`sparse_flash_attention_grad_golden_bsnd`).  MLA-absorb, one KV head; the forward statistics
are reused to rebuild the probabilities (:118-121):
    score[h,p] = (q_nope[h].k_nope[p] + q_rope[h].k_rope[p]) * scale
    P[h,p]     = exp(score[h,p] - softmax_max[h]) / softmax_sum[h]
    dP[h,p]    = dO[h].k_nope[p]                      (value == key[..., :D])
    delta[h]   = dO[h].O[h]
    dS[h,p]    = P[h,p] * (dP[h,p] - delta[h]) * scale
    d_query[h] = sum_p dS[h,p] k_nope[p]      d_query_rope[h] = sum_p dS[h,p] k_rope[p]   (:125-127)
    d_key[u]  += sum_h dS[h,p->u] q_nope[h]   d_key_rope[u] += sum_h dS[h,p->u] q_rope[h] (:130-131)
    d_value[u]+= sum_h P[h,p->u]  dO[h]                                                   (:132)
Everything accumulates in fp32; the five results are rounded to the io dtype at the end
(:134-135).  d_key (QK path) and d_value (PV path) stay separate.  Rows outside the causal
window or without a valid position contribute nothing (:100-115).

The per-row inner products are written as matrix products over all heads at once; the
sums run over the same terms as the golden's per-head loop.
"""
import numpy as np

from .sfa_oracle import BF16, _round_io, gather_positions


def sparse_flash_attention_grad_oracle(q_nope, k_nope, sparse_indices, d_out, out, softmax_max, softmax_sum,
                                       q_rope, k_rope, scale_value, act_q, act_k,
                                       sparse_block_size=1, sparse_mode=3, dtype=BF16):
    """BSND backward.  q_nope/d_out/out [B,S1,N1,D], k_nope [B,S2,1,D], q_rope [B,S1,N1,Dr],
    k_rope [B,S2,1,Dr], sparse_indices [B,S1,1,K] int32, statistics [B,1,S1,N1] fp32.
    Returns (d_query, d_key, d_value, d_query_rope, d_key_rope) as fp32 arrays holding
    io-dtype-rounded values."""
    qn = np.asarray(q_nope, dtype=np.float32)
    kn = np.asarray(k_nope, dtype=np.float32)
    qr = np.asarray(q_rope, dtype=np.float32)
    kr = np.asarray(k_rope, dtype=np.float32)
    do = np.asarray(d_out, dtype=np.float32)
    o = np.asarray(out, dtype=np.float32)
    smax = np.asarray(softmax_max, dtype=np.float32)
    ssum = np.asarray(softmax_sum, dtype=np.float32)
    B, S1, N1, D = qn.shape
    S2, Dr = kn.shape[1], qr.shape[-1]
    scale = np.float32(scale_value)

    d_query = np.zeros((B, S1, N1, D), np.float32)
    d_query_rope = np.zeros((B, S1, N1, Dr), np.float32)
    d_key = np.zeros((B, S2, 1, D), np.float32)
    d_key_rope = np.zeros((B, S2, 1, Dr), np.float32)
    d_value = np.zeros((B, S2, 1, D), np.float32)

    for b in range(B):
        aq, ak = int(act_q[b]), int(act_k[b])
        for s1 in range(aq):
            threshold = ak if sparse_mode == 0 else ak - aq + s1 + 1
            if threshold <= 0:
                continue
            pos = gather_positions(sparse_indices[b, s1, 0, :], sparse_block_size, threshold, ak)
            if not pos:
                continue
            pos = np.asarray(pos, dtype=np.int64)
            kn_sp, kr_sp = kn[b, pos, 0, :], kr[b, pos, 0, :]                  # [P, D], [P, Dr]
            scores = (qn[b, s1] @ kn_sp.T + qr[b, s1] @ kr_sp.T) * scale       # [N1, P]
            with np.errstate(divide="ignore", invalid="ignore"):
                prob = np.exp(scores - smax[b, 0, s1][:, None]) / ssum[b, 0, s1][:, None]
            dp = do[b, s1] @ kn_sp.T                                           # [N1, P]
            delta = np.sum(do[b, s1] * o[b, s1], axis=-1, keepdims=True)       # [N1, 1]
            ds = prob * (dp - delta) * scale
            d_query[b, s1] += ds @ kn_sp
            d_query_rope[b, s1] += ds @ kr_sp
            np.add.at(d_key[b, :, 0, :], pos, ds.T @ qn[b, s1])
            np.add.at(d_key_rope[b, :, 0, :], pos, ds.T @ qr[b, s1])
            np.add.at(d_value[b, :, 0, :], pos, prob.T @ do[b, s1])
    return tuple(_round_io(x, dtype) for x in (d_query, d_key, d_value, d_query_rope, d_key_rope))
