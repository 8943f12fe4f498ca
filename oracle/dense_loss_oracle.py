"""Numpy oracle for the dense lightning-indexer softmax LSE and KL-loss backward (test
infrastructure only).

Restates the two numpy baselines the reference keeps in its test file:
`_dense_indexer_lse_numpy` (test_dense_loss_backward_triton.py:124-159) and
`_dense_loss_backward_numpy` (:230-315).  Same mathematics as the sparse operator
(oracle/sli_grad_oracle.py) over ALL causally visible keys 0..n-1 of a row,
n = min(max(act_k - act_q + s1 + 1, 0), S2), with two differences: the student distribution is
normalised with index statistics handed in from outside,
    student[k] = exp(I[k] - max_index) / max(sum_index, 1e-8)        (rows with sum_index <= 0 are skipped),
and the attention keys may have N2 heads (query head h reads key head h // (N1 / N2); statistics
are [B, N2, S1, N1 / N2]).
"""
import numpy as np

EPS = 1e-8


def _lens(act, default, B):
    return [default] * B if act is None else [int(v) for v in act]


def dense_indexer_lse_oracle(qi, ki, w, act_q=None, act_k=None):
    """max / sum of exp over the visible keys of I[k] = sum_g w[g] relu(qi[g].ki[k]); both [B,1,S1],
    -inf / 0 for rows without visible keys (:141-158)."""
    qi, ki, w = (np.asarray(x, np.float32) for x in (qi, ki, w))
    B, S1 = qi.shape[:2]
    S2 = ki.shape[1]
    aq, ak = _lens(act_q, S1, B), _lens(act_k, S2, B)
    mx = np.full((B, 1, S1), -np.inf, np.float32)
    sm = np.zeros((B, 1, S1), np.float32)
    for b in range(B):
        for s1 in range(min(aq[b], S1)):
            n = min(max(ak[b] - aq[b] + s1 + 1, 0), ak[b], S2)
            if n <= 0:
                continue
            sc = w[b, s1] @ np.maximum(qi[b, s1] @ ki[b, :n, 0].T, 0.0)
            mx[b, 0, s1] = sc.max()
            sm[b, 0, s1] = np.exp(sc - sc.max()).sum()
    return mx, sm


def dense_loss_backward_oracle(q, k, qr, kr, qi, ki, w, sm_max, sm_sum, max_index, sum_index, scale,
                               act_q=None, act_k=None):
    """Returns dict(dQueryIndex, dKeyIndex, dW, loss[1]) in fp32 (:262-315)."""
    q, k, qi, ki, w = (np.asarray(x, np.float32) for x in (q, k, qi, ki, w))
    B, S1, N1, _ = q.shape
    S2, N2 = k.shape[1], k.shape[2]
    G = N1 // N2
    qr = np.zeros((B, S1, N1, 0), np.float32) if qr is None else np.asarray(qr, np.float32)
    kr = np.zeros((B, S2, N2, 0), np.float32) if kr is None else np.asarray(kr, np.float32)
    max_index = np.asarray(max_index, np.float32).reshape(B, S1)
    sum_index = np.asarray(sum_index, np.float32).reshape(B, S1)
    aq, ak = _lens(act_q, S1, B), _lens(act_k, S2, B)
    scale = np.float32(scale)
    d_qi, d_ki, d_w = np.zeros_like(qi), np.zeros_like(ki), np.zeros_like(w)
    loss = 0.0
    for b in range(B):
        for s1 in range(min(aq[b], S1)):
            n = min(max(ak[b] - aq[b] + s1 + 1, 0), S2)
            if n <= 0 or sum_index[b, s1] <= 0.0:
                continue
            ki_v = ki[b, :n, 0]
            relu = np.maximum(qi[b, s1] @ ki_v.T, 0.0)                       # [Gi, n]
            student = np.exp(w[b, s1] @ relu - max_index[b, s1]) / max(float(sum_index[b, s1]), EPS)
            p = np.zeros(n, np.float32)
            for n2 in range(N2):
                hs = slice(n2 * G, (n2 + 1) * G)
                sc = (q[b, s1, hs] @ k[b, :n, n2].T + qr[b, s1, hs] @ kr[b, :n, n2].T) * scale
                p += (np.exp(sc - sm_max[b, n2, s1][:, None]) / (sm_sum[b, n2, s1][:, None] + EPS)).sum(axis=0)
            p *= np.float32(1.0 / N1)
            d_i = student - p
            pc, sc_ = np.maximum(p, EPS), np.maximum(student, EPS)
            loss += float(np.sum(pc * (np.log(pc) - np.log(sc_))))
            d_w[b, s1] = relu @ d_i
            ds = (d_i[None, :] * w[b, s1][:, None]) * (relu > 0)
            d_qi[b, s1] = ds @ ki_v
            d_ki[b, :n, 0] += ds.T @ qi[b, s1]
    return dict(dQueryIndex=d_qi, dKeyIndex=d_ki, dW=d_w, loss=np.array([loss], np.float32))


def dense_softmax_stats(q, k, qr, kr, scale, act_q=None, act_k=None):
    """softmax_max / softmax_sum [B,N2,S1,N1/N2] of the dense causal attention forward
    (test_dense_loss_backward_triton.py:181-213, plus valid lengths)."""
    q, k, qr, kr = (np.asarray(x, np.float32) for x in (q, k, qr, kr))
    B, S1, N1, _ = q.shape
    S2, N2 = k.shape[1], k.shape[2]
    G = N1 // N2
    aq, ak = _lens(act_q, S1, B), _lens(act_k, S2, B)
    mx = np.full((B, N2, S1, G), -np.inf, np.float32)
    sm = np.zeros((B, N2, S1, G), np.float32)
    for b in range(B):
        for s1 in range(min(aq[b], S1)):
            n = min(max(ak[b] - aq[b] + s1 + 1, 0), S2)
            if n <= 0:
                continue
            for n2 in range(N2):
                hs = slice(n2 * G, (n2 + 1) * G)
                sc = (q[b, s1, hs] @ k[b, :n, n2].T + qr[b, s1, hs] @ kr[b, :n, n2].T) * np.float32(scale)
                mx[b, n2, s1] = sc.max(axis=1)
                sm[b, n2, s1] = np.exp(sc - sc.max(axis=1)[:, None]).sum(axis=1)
    return mx, sm
