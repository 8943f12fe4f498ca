"""Numpy oracle for sparse_lightning_indexer_grad_kl_loss (test infrastructure only).

Restates sli_grad_kl_loss_numpy.py:16-156 (`numpy_reference`) with the length handling of the
device path (sparse_lightning_indexer_grad_kl_loss_triton.py:64-74: rows at or beyond the valid
query length are skipped, the number of slots a row uses is
min(topK, S2, max(act_k - act_q + s1 + 1, 0))).  Per used row, with idx = the row's first n sparse
indices clipped to [0, S2):
    I[k]   = sum_g w[g] * relu(qi[g] . ki[idx[k]])                                    (:62-74)
    p[k]   = mean_h exp((q[h].k[idx[k]] + qr[h].kr[idx[k]]) * scale - max[h]) / (sum[h] + 1e-8)   (:78-92)
    sI     = exp(I - max I) / (sum + 1e-8)                                            (:95-103)
    dI     = sI - p;   loss += sum_k max(p,1e-8) * (log max(p,1e-8) - log max(sI,1e-8))   (:106-116)
    dW[g]  = sum_k dI[k] * relu[g,k]                                                  (:127)
    dQI[g] = sum_k dI[k] * w[g] * [relu[g,k] > 0] * ki[idx[k]]                         (:129-131)
    dKI[idx[k]] += sum_g dI[k] * w[g] * [relu[g,k] > 0] * qi[g]                        (:139-151)
Inputs are rounded to the io dtype first (the golden hard-codes fp16, :24-30); results stay fp32,
as the golden returns them.
"""
import numpy as np

from .sfa_oracle import _round_io

EPS = 1e-8


def sli_grad_kl_loss_oracle(q, k, qr, kr, qi, ki, w, si, sm_max, sm_sum, scale, act_q=None, act_k=None,
                            dtype="fp16"):
    """q [B,S1,N1,D], k [B,S2,1,D], qr/kr rope parts (or None), qi [B,S1,G,Di], ki [B,S2,1,Di],
    w [B,S1,G], si [B,S1,1,topK] int32, sm_max/sm_sum [B,1,S1,N1] fp32.
    Returns dict(dQueryIndex, dKeyIndex, dW, loss[1]) in fp32."""
    r = lambda x: _round_io(np.asarray(x, np.float32), dtype)   # noqa: E731
    q, k, qi, ki, w = r(q), r(k), r(qi), r(ki), r(w)
    B, S1, N1, _ = q.shape
    S2, topK = k.shape[1], si.shape[3]
    qr = np.zeros((B, S1, N1, 0), np.float32) if qr is None else r(qr)
    kr = np.zeros((B, S2, 1, 0), np.float32) if kr is None else r(kr)
    si = np.asarray(si, np.int32)
    act_q = [S1] * B if act_q is None else act_q
    act_k = [S2] * B if act_k is None else act_k
    scale = np.float32(scale)

    d_qi = np.zeros_like(qi)
    d_ki = np.zeros_like(ki)
    d_w = np.zeros_like(w)
    loss = 0.0
    for b in range(B):
        aq, ak = int(act_q[b]), int(act_k[b])
        for s1 in range(min(aq, S1)):
            n = min(topK, S2, max(ak - aq + s1 + 1, 0))
            if n <= 0:
                continue
            idx = np.clip(si[b, s1, 0, :n], 0, S2 - 1)
            ki_g = ki[b, idx, 0, :]                                          # [n, Di]
            relu = np.maximum(qi[b, s1] @ ki_g.T, 0.0)                       # [G, n]
            i_vec = w[b, s1] @ relu                                          # [n]
            scores = (q[b, s1] @ k[b, idx, 0, :].T + qr[b, s1] @ kr[b, idx, 0, :].T) * scale
            probs = np.exp(scores - sm_max[b, 0, s1][:, None]) / (sm_sum[b, 0, s1][:, None] + EPS)
            p = probs.sum(axis=0) * np.float32(1.0 / N1)
            e = np.exp(i_vec - i_vec.max())
            s_i = e / (e.sum() + EPS)
            d_i = s_i - p
            pc, sc = np.maximum(p, EPS), np.maximum(s_i, EPS)
            loss += float(np.sum(pc * (np.log(pc) - np.log(sc))))
            d_w[b, s1] = relu @ d_i
            ds = (d_i[None, :] * w[b, s1][:, None]) * (relu > 0)             # [G, n]
            d_qi[b, s1] = ds @ ki_g
            np.add.at(d_ki[b, :, 0, :], idx, ds.T @ qi[b, s1])
    return dict(dQueryIndex=d_qi, dKeyIndex=d_ki, dW=d_w, loss=np.array([loss], np.float32))


def softmax_stats(q, k, qr, kr, scale, act_q=None, act_k=None, dtype="fp16"):
    """softmax_max / softmax_sum [B,1,S1,N1] of the dense causal forward over ALL keys, the
    statistics this operator consumes (test_sli_grad_kl_loss_triton.py:140-175)."""
    r = lambda x: _round_io(np.asarray(x, np.float32), dtype)   # noqa: E731
    q, k, qr, kr = r(q), r(k), r(qr), r(kr)
    B, S1, N1, _ = q.shape
    S2 = k.shape[1]
    act_q = [S1] * B if act_q is None else act_q
    act_k = [S2] * B if act_k is None else act_k
    sm_max = np.full((B, 1, S1, N1), -np.inf, np.float32)
    sm_sum = np.zeros((B, 1, S1, N1), np.float32)
    for b in range(B):
        aq, ak = int(act_q[b]), int(act_k[b])
        for s1 in range(min(aq, S1)):
            lim = min(max(ak - aq + s1 + 1, 0), S2)
            if lim <= 0:
                continue
            sc = (q[b, s1] @ k[b, :lim, 0, :].T + qr[b, s1] @ kr[b, :lim, 0, :].T) * np.float32(scale)
            m = sc.max(axis=1)
            sm_max[b, 0, s1] = m
            sm_sum[b, 0, s1] = np.exp(sc - m[:, None]).sum(axis=1)
    return sm_max, sm_sum
