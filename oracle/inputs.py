"""Seeded synthetic inputs for the parity configurations (test infrastructure only).

The reference has no dataset: every test and perf input is `np.random` data
(test_li_triton.py:30-36, test_sfa_triton.py:47-85, perf_sfa_triton.py:35-62).  The
generators below follow that recipe: one RandomState per case, fp32 normal draws in the
order the reference tests draw them, rounded to the io dtype so that the CUDA kernels
and the oracle see identical values.
"""
import numpy as np

from .li_oracle import round_bf16


def round_io(x, dtype):
    if dtype == "fp16":
        return x.astype(np.float16).astype(np.float32)
    return round_bf16(x.astype(np.float32))


def li_inputs(seed, B, S1, S2, N1, N2, D, dtype="bf16", w_scale=None):
    """q, k, w drawn in that order (test_li_triton.py:32-35); w stays fp32."""
    rng = np.random.RandomState(seed)
    q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), dtype)
    k = round_io(rng.randn(B, S2, N2, D).astype(np.float32), dtype)
    w_scale = (1.0 / np.sqrt(N1)) if w_scale is None else w_scale
    w = (rng.randn(B, S1, N1).astype(np.float32) * np.float32(w_scale)).astype(np.float32)
    return q, k, w


def sparse_indices(seed, B, S1, S2, count, block=1, sparse_mode=3, act_q=None, act_k=None):
    """Front-packed ascending distinct block ids inside each row's causal window, -1 padded
    (the contract of test_sfa_triton.py:63-85)."""
    rng = np.random.RandomState(seed)
    si = np.full((B, S1, 1, count), -1, dtype=np.int32)
    for b in range(B):
        aq = S1 if act_q is None else int(act_q[b])
        ak = S2 if act_k is None else int(act_k[b])
        for s1 in range(aq):
            thr = ak if sparse_mode == 0 else ak - aq + s1 + 1
            if thr <= 0:
                continue
            nblk = int(np.ceil(thr / block))
            n = min(count, nblk)
            si[b, s1, 0, :n] = np.sort(rng.permutation(nblk)[:n]).astype(np.int32)
    return si


def sfa_inputs(seed, B, S1, S2, N1, D=512, Dr=64, dtype="bf16"):
    """q, k, v (drawn, unused), q_rope, k_rope in the reference's order (test_sfa_triton.py:54-58)."""
    rng = np.random.RandomState(seed)

    def draw(*shape):
        return round_io(rng.randn(*shape).astype(np.float32), dtype)

    q = draw(B, S1, N1, D)
    k = draw(B, S2, 1, D)
    draw(B, S2, 1, D)  # value: drawn to keep the stream aligned, ignored by the operator
    qr = draw(B, S1, N1, Dr)
    kr = draw(B, S2, 1, Dr)
    return q, k, qr, kr

def sfa_grad_inputs(seed, B, S1, S2, N1, D=512, Dr=64, dtype="bf16"):
    """q, k, v (drawn, unused), q_rope, k_rope, d_out in the order and with the 0.3 scale of the
    reference's backward tests (test_sfa_grad_triton.py:73-86)."""
    rng = np.random.RandomState(seed)

    def draw(*shape):
        return round_io(rng.randn(*shape).astype(np.float32) * np.float32(0.3), dtype)

    q = draw(B, S1, N1, D)
    k = draw(B, S2, 1, D)
    draw(B, S2, 1, D)
    qr = draw(B, S1, N1, Dr)
    kr = draw(B, S2, 1, Dr)
    do = draw(B, S1, N1, D)
    return q, k, qr, kr, do

def sli_grad_inputs(seed, B, S1, S2, N1, D, G, Di, topk, pattern="causal_random", Dr=64, dtype="fp16"):
    """q, k, q_rope, k_rope, q_index, k_index, |w| drawn in the order of the reference's backward
    tests (test_sli_grad_kl_loss_triton.py:82-94), then sparse indices of the given pattern
    (:96-131): "random" anywhere in [0, S2), "causal_random" distinct positions inside each row's
    causal window (zero-padded), "causal_continuous" 0..n-1, "repeated" alternating 0 / 7."""
    rng = np.random.RandomState(seed)
    draw = lambda *shape: round_io(rng.randn(*shape).astype(np.float32), dtype)   # noqa: E731
    q, k = draw(B, S1, N1, D), draw(B, S2, 1, D)
    qr, kr = draw(B, S1, N1, Dr), draw(B, S2, 1, Dr)
    qi, ki = draw(B, S1, G, Di), draw(B, S2, 1, Di)
    w = np.abs(draw(B, S1, G))
    si = np.zeros((B, S1, 1, topk), np.int32)
    if pattern == "random":
        si = rng.randint(0, S2, (B, S1, 1, topk)).astype(np.int32)
    elif pattern == "repeated":
        si[..., 1::2] = min(S2 - 1, 7)
    else:
        for b in range(B):
            for s1 in range(S1):
                visible = min(max(S2 - S1 + s1 + 1, 1), S2)
                n = min(topk, visible)
                si[b, s1, 0, :n] = (rng.choice(visible, size=n, replace=False) if pattern == "causal_random"
                                    else np.arange(n))
    return q, k, qr, kr, qi, ki, w, si

def dense_loss_inputs(seed, B, S1, S2, N1, N2, D, G, Di, Dr=64, dtype="fp16"):
    """q, k, q_rope, k_rope, q_index, k_index, |w| in the order of the reference's dense-loss tests
    (test_dense_loss_backward_triton.py:169-178); the attention key has N2 heads."""
    rng = np.random.RandomState(seed)
    draw = lambda *shape: round_io(rng.randn(*shape).astype(np.float32), dtype)   # noqa: E731
    q, k = draw(B, S1, N1, D), draw(B, S2, N2, D)
    qr, kr = draw(B, S1, N1, Dr), draw(B, S2, N2, Dr)
    qi, ki = draw(B, S1, G, Di), draw(B, S2, 1, Di)
    w = np.abs(draw(B, S1, G))
    return q, k, qr, kr, qi, ki, w


# The two CPU-sized configurations of the benchmark specification.
def config1():
    """LI, seed 0, B=1, S1=S2=512, N1=8, N2=1, D=128, bf16, fp32 w ~ N(0,1)/sqrt(N1), k=64, mode 3."""
    q, k, w = li_inputs(0, 1, 512, 512, 8, 1, 128, "bf16")
    return dict(q=q, k=k, w=w, sparse_count=64, sparse_mode=3)


def config2():
    """SFA, seed 1, B=1, S1=256, S2=1024, N1=16, D=512, Dr=64, k=256 token-wise, mode 3."""
    q, k, qr, kr = sfa_inputs(1, 1, 256, 1024, 16)
    si = sparse_indices(1001, 1, 256, 1024, 256)
    return dict(q=q, k=k, qr=qr, kr=kr, idx=si, scale=1.0 / np.sqrt(576.0), sparse_mode=3)
