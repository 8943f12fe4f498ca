"""GPU parity of the attention backward (sparse_flash_attention_grad_triton) through the C ABI.

Three checkers: the committed outputs of the unmodified reference golden
(tests/golden/sfa_grad_*.npz), the numpy oracle on further shapes and layouts, and - as an
independent derivation of the same formulas - torch autograd through a dense fp64 restatement of
the forward."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import sparse_flash_attention_grad_oracle, sparse_flash_attention_oracle
from oracle import layouts
from oracle.compare import sfa_grad_acceptance_rule, sfa_grad_reference_rule
from oracle.inputs import sfa_grad_inputs, sparse_indices
from tests.golden.cases import SFA_GRAD_CASES, sfa_grad_case_inputs
from tests.util import dev, host, tdtype

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ("d_query", "d_key", "d_value", "d_query_rope", "d_key_rope")
SCATTERED = {"d_key", "d_value", "d_key_rope"}


def _check(got, ref, dtype, S1, strict=True):
    for n, a, b in zip(NAMES, got, ref):
        a = host(a) if isinstance(a, torch.Tensor) else a
        assert sfa_grad_reference_rule(a, b, dtype, scale=math.sqrt(S1) if n in SCATTERED else 1.0), \
            f"{n}: reference rule"
        if strict:
            sfa_grad_acceptance_rule(a, b, dtype, name=n)


@pytest.mark.parametrize("name", sorted(SFA_GRAD_CASES))
@pytest.mark.parametrize("fwd_source", ["oracle", "device"])
def test_grad_matches_the_reference_golden(name, fwd_source):
    """fwd_source="oracle": the forward state is the one the golden was generated with, so the
    backward alone is compared (2 ulp of the io dtype).  fwd_source="device": forward and backward
    both run on the GPU, like the reference's end-to-end test; the rule is the reference's."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_grad_triton, sparse_flash_attention_triton
    q, k, qr, kr, do, idx, act_q, act_k, scale, c = sfa_grad_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = tdtype(c["dtype"])
    tq, tk, tqr, tkr, tdo, tidx = dev(q, dt), dev(k, dt), dev(qr, dt), dev(kr, dt), dev(do, dt), dev(idx)
    kw = dict(scale_value=scale, query_rope=tqr, key_rope=tkr, actual_seq_lengths_query=act_q.tolist(),
              actual_seq_lengths_kv=act_k.tolist(), sparse_block_size=c["block"], sparse_mode=c["mode"])
    if fwd_source == "oracle":
        out, smax, ssum = sparse_flash_attention_oracle(
            q, k, idx, qr, kr, scale, act_q, act_k, sparse_block_size=c["block"], sparse_mode=c["mode"],
            return_softmax_lse=True, dtype=c["dtype"])
        tout, tmax, tsum = dev(out, dt), dev(smax), dev(ssum)
    else:
        tout, tmax, tsum = sparse_flash_attention_triton(tq, tk, tk, tidx, return_softmax_lse=True, **kw)
    got = sparse_flash_attention_grad_triton(tq, tk, tk, tidx, tdo, tout, tmax, tsum, **kw)
    for t, like in zip(got, (tq, tk, tk, tqr, tkr)):
        assert t.shape == like.shape and t.dtype == like.dtype
    _check(got, [g[n] for n in NAMES], c["dtype"], c["S1"], strict=fwd_source == "oracle")


@pytest.mark.parametrize("B,S1,S2,N1,K,D,dtype", [
    (1, 128, 1024, 64, 512, 512, "bf16"),     # test_sfa_grad_triton.py:262 (test_basic shape)
    (2, 64, 512, 32, 256, 256, "fp16"),       # :263
    (1, 16, 2048, 64, 2048, 128, "bf16"),     # :264, top-k 2048
    (1, 40, 300, 20, 100, 512, "bf16"),       # head count not a multiple of 16, odd lengths
])
def test_grad_against_the_oracle_on_larger_shapes(B, S1, S2, N1, K, D, dtype):
    from dsa_triton_ascend_b200 import SparseFlashAttentionGradTriton, SparseFlashAttentionTriton
    q, k, qr, kr, do = sfa_grad_inputs(77, B, S1, S2, N1, D, 64, dtype)
    idx = sparse_indices(1077, B, S1, S2, K, 1, 3)
    scale = 1.0 / math.sqrt(D + 64.0)
    dt = tdtype(dtype)
    tq, tk, tqr, tkr, tdo, tidx = dev(q, dt), dev(k, dt), dev(qr, dt), dev(kr, dt), dev(do, dt), dev(idx)
    fwd = SparseFlashAttentionTriton(scale_value=scale, sparse_mode=3, return_softmax_lse=True)
    tout, tmax, tsum = fwd(tq, tk, tk, tidx, query_rope=tqr, key_rope=tkr)
    got = SparseFlashAttentionGradTriton(scale_value=scale, sparse_mode=3)(
        tq, tk, tk, tidx, tdo, tout, tmax, tsum, query_rope=tqr, key_rope=tkr)
    # the checker consumes the device's forward state, so only the backward is compared
    ref = sparse_flash_attention_grad_oracle(q, k, idx, do, host(tout), host(tmax), host(tsum), qr, kr, scale,
                                             [S1] * B, [S2] * B, sparse_mode=3, dtype=dtype)
    _check(got, ref, dtype, S1)


@pytest.mark.parametrize("kernel", ["tensor", "portable"])
@pytest.mark.parametrize("dtype,D", [("bf16", 512), ("fp16", 512), ("fp16", 256), ("bf16", 128)])
def test_grad_both_kernels(kernel, dtype, D):
    """The backward runs on the tensor cores by default; the CUDA-core kernel stays selectable and both
    meet the same rule (block-wise indices, a head count that leaves a partial chunk, valid lengths)."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_grad as mod
    from dsa_triton_ascend_b200 import sparse_flash_attention_triton
    B, S1, S2, N1, block = 2, 24, 200, 40, 4
    q, k, qr, kr, do = sfa_grad_inputs(55, B, S1, S2, N1, D, 64, dtype)
    act_q, act_k = [24, 13], [200, 57]
    idx = sparse_indices(1055, B, S1, S2, 20, block, 3, act_q, act_k)
    scale = 1.0 / math.sqrt(D + 64.0)
    dt = tdtype(dtype)
    tq, tk, tqr, tkr, tdo, tidx = dev(q, dt), dev(k, dt), dev(qr, dt), dev(kr, dt), dev(do, dt), dev(idx)
    kw = dict(scale_value=scale, query_rope=tqr, key_rope=tkr, actual_seq_lengths_query=act_q,
              actual_seq_lengths_kv=act_k, sparse_block_size=block, sparse_mode=3)
    tout, tmax, tsum = sparse_flash_attention_triton(tq, tk, tk, tidx, return_softmax_lse=True, **kw)
    mod.set_kernel(kernel)
    try:
        got = mod.sparse_flash_attention_grad_triton(tq, tk, tk, tidx, tdo, tout, tmax, tsum, **kw)
    finally:
        mod.set_kernel("auto")
    ref = sparse_flash_attention_grad_oracle(q, k, idx, do, host(tout), host(tmax), host(tsum), qr, kr, scale,
                                             act_q, act_k, sparse_block_size=block, sparse_mode=3, dtype=dtype)
    _check(got, ref, dtype, S1)


def test_grad_fp16_chunk_of_zero_probabilities_before_small_gradients():
    """fp16 operands of the second products are scaled per 32-key chunk from the chunk's largest |dS|.
    The first chunk here has probabilities that underflow to exactly zero (dS = 0) and the chunks after
    it carry gradients around 1e-6: a scale pinned by the all-zero chunk would push them into fp16's
    subnormal range."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_grad_triton
    B, S1, S2, N1, D = 1, 2, 96, 16, 512
    rng = np.random.RandomState(3)
    q = np.full((B, S1, N1, D), 2.0, np.float32)
    qr = np.full((B, S1, N1, 64), 2.0, np.float32)
    k = np.full((B, S2, 1, D), 2.0, np.float32)
    kr = np.full((B, S2, 1, 64), 2.0, np.float32)
    k[:, :32] = -2.0
    kr[:, :32] = -2.0
    k[:, 32:] += (rng.randint(-2, 3, size=(B, S2 - 32, 1, D)) / 64.0).astype(np.float32)   # fp16-exact jitter
    do = (rng.randn(B, S1, N1, D) * 1e-3).astype(np.float16).astype(np.float32)
    idx = np.tile(np.arange(S2, dtype=np.int32), (B, S1, 1, 1))
    scale = 1.0 / 24.0
    out, smax, ssum = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, [S1], [S2], sparse_mode=0,
                                                    return_softmax_lse=True, dtype="fp16")
    ref = sparse_flash_attention_grad_oracle(q, k, idx, do, out, smax, ssum, qr, kr, scale, [S1], [S2],
                                             sparse_mode=0, dtype="fp16")
    assert np.abs(ref[0]).max() > 0 and np.abs(ref[0]).max() < 1e-3
    h = torch.float16
    got = sparse_flash_attention_grad_triton(dev(q, h), dev(k, h), dev(k, h), dev(idx), dev(do, h), dev(out, h),
                                             dev(smax), dev(ssum), scale_value=scale, query_rope=dev(qr, h),
                                             key_rope=dev(kr, h), sparse_mode=0)
    _check(got, ref, "fp16", S1)


def test_grad_tnd_layout_equals_the_padded_bsnd_problem():
    """TND batch with cumulative lengths (sparse_flash_attention_grad_triton.py:566-581 pads it to
    BSND): the token-major gradients equal the oracle's BSND gradients packed back."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_grad_triton, sparse_flash_attention_triton
    lens_q, lens_k = [9, 1, 17, 5], [40, 33, 17, 64]
    B, N1, D, K = 4, 16, 512, 24
    S1, S2 = max(lens_q), max(lens_k)
    q, k, qr, kr, do = sfa_grad_inputs(91, B, S1, S2, N1, D, 64, "bf16")
    idx = sparse_indices(1091, B, S1, S2, K, 1, 3, lens_q, lens_k)
    scale = 1.0 / 24.0
    bf = torch.bfloat16
    pack_q = lambda x: dev(layouts.bsnd_to_tnd(x, lens_q), bf)       # noqa: E731
    pack_k = lambda x: dev(layouts.bsnd_to_tnd(x, lens_k), bf)       # noqa: E731
    tq, tqr, tdo, tk, tkr = pack_q(q), pack_q(qr), pack_q(do), pack_k(k), pack_k(kr)
    tidx = dev(layouts.bsnd_to_tnd(idx, lens_q))
    cq, ck = np.cumsum(lens_q).tolist(), np.cumsum(lens_k).tolist()
    tout, tmax, tsum = sparse_flash_attention_triton(
        tq, tk, tk, tidx, scale_value=scale, actual_seq_lengths_query=cq, actual_seq_lengths_kv=ck,
        query_rope=tqr, key_rope=tkr, layout_query="TND", layout_kv="TND", sparse_mode=3, return_softmax_lse=True)
    got = sparse_flash_attention_grad_triton(
        tq, tk, tk, tidx, tdo, tout, tmax, tsum, scale_value=scale, query_rope=tqr, key_rope=tkr,
        actual_seq_lengths_query=cq, actual_seq_lengths_kv=ck, layout="TND", sparse_mode=3)
    out_b = layouts.tnd_to_bsnd(host(tout), lens_q)
    # statistics [1,T1,N1] -> [B,1,S1,N1]
    st = lambda t: layouts.tnd_to_bsnd(host(t)[0], lens_q)[:, None]   # noqa: E731
    ref = sparse_flash_attention_grad_oracle(q, k, idx, do, out_b, st(tmax), st(tsum), qr, kr, scale, lens_q, lens_k,
                                             sparse_mode=3, dtype="bf16")
    packed = [layouts.bsnd_to_tnd(ref[0], lens_q), layouts.bsnd_to_tnd(ref[1], lens_k),
              layouts.bsnd_to_tnd(ref[2], lens_k), layouts.bsnd_to_tnd(ref[3], lens_q),
              layouts.bsnd_to_tnd(ref[4], lens_k)]
    _check(got, packed, "bf16", S1)


def test_grad_agrees_with_autograd_through_a_dense_forward():
    """Independent derivation: d(sum(out * dO)) / d(inputs) by torch autograd through a dense fp64
    forward with -inf outside the selected keys.  key and value are separate leaves, so autograd's
    d_key is the QK path and d_value the PV path, like the operator's outputs."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_grad_triton, sparse_flash_attention_triton
    B, S1, S2, N1, D, K = 1, 12, 96, 8, 128, 40
    q, k, qr, kr, do = sfa_grad_inputs(5, B, S1, S2, N1, D, 64, "bf16")
    idx = sparse_indices(1005, B, S1, S2, K, 1, 3)
    scale = 1.0 / math.sqrt(D + 64.0)
    bf = torch.bfloat16
    tq, tk, tqr, tkr, tdo, tidx = dev(q, bf), dev(k, bf), dev(qr, bf), dev(kr, bf), dev(do, bf), dev(idx)
    tout, tmax, tsum = sparse_flash_attention_triton(tq, tk, tk, tidx, scale_value=scale, query_rope=tqr,
                                                     key_rope=tkr, sparse_mode=3, return_softmax_lse=True)
    got = sparse_flash_attention_grad_triton(tq, tk, tk, tidx, tdo, tout, tmax, tsum, scale_value=scale,
                                             query_rope=tqr, key_rope=tkr, sparse_mode=3)
    leaves = [torch.tensor(x, dtype=torch.float64, requires_grad=True) for x in (q, k, k, qr, kr)]
    Q, Kt, V, QR, KR = leaves
    mask = torch.full((B, S1, S2), float("-inf"), dtype=torch.float64)
    for s1 in range(S1):
        sel = idx[0, s1, 0]
        mask[0, s1, sel[sel >= 0]] = 0.0
    score = (torch.einsum("bshd,btd->bsht", Q, Kt[:, :, 0]) + torch.einsum("bshd,btd->bsht", QR, KR[:, :, 0])) * scale
    prob = torch.softmax(score + mask[:, :, None, :], dim=-1)
    out = torch.einsum("bsht,btd->bshd", prob, V[:, :, 0])
    (out * torch.tensor(do, dtype=torch.float64)).sum().backward()
    ref = [Q.grad, Kt.grad, V.grad, QR.grad, KR.grad]
    for n, a, b in zip(NAMES, got, ref):
        a, b = host(a), b.numpy()
        # bf16 inputs and a bf16 forward output feed the operator: 2 % of the tensor's scale
        assert np.abs(a - b).max() <= 2e-2 * np.abs(b).max() + 1e-6, f"{n}: {np.abs(a - b).max()} vs {np.abs(b).max()}"


def test_grad_untouched_rows_are_zero_and_repeat_runs_agree():
    """Query rows past the valid length and rows without visible keys get zero gradients; keys nobody
    selected get zero d_key / d_value; two runs agree to the last places (atomics reorder fp32 sums)."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_grad_triton, sparse_flash_attention_triton
    B, S1, S2, N1, D, K = 2, 20, 64, 16, 256, 16
    act_q, act_k = [20, 12], [64, 5]                  # batch 1: rows 0..6 see nothing (12 > 5)
    q, k, qr, kr, do = sfa_grad_inputs(8, B, S1, S2, N1, D, 64, "fp16")
    idx = sparse_indices(1008, B, S1, S2, K, 1, 3, act_q, act_k)
    hf = torch.float16
    tq, tk, tqr, tkr, tdo, tidx = dev(q, hf), dev(k, hf), dev(qr, hf), dev(kr, hf), dev(do, hf), dev(idx)
    kw = dict(scale_value=1.0 / math.sqrt(320.0), query_rope=tqr, key_rope=tkr, actual_seq_lengths_query=act_q,
              actual_seq_lengths_kv=act_k, sparse_mode=3)
    tout, tmax, tsum = sparse_flash_attention_triton(tq, tk, tk, tidx, return_softmax_lse=True, **kw)
    a = sparse_flash_attention_grad_triton(tq, tk, tk, tidx, tdo, tout, tmax, tsum, **kw)
    b = sparse_flash_attention_grad_triton(tq, tk, tk, tidx, tdo, tout, tmax, tsum, **kw)
    dq, dk, dv, dqr, dkr = [host(t) for t in a]
    assert (dq[1, 12:] == 0).all() and (dqr[1, 12:] == 0).all() and (dq[1, :7] == 0).all()
    assert (dk[1, 5:] == 0).all() and (dv[1, 5:] == 0).all() and (dkr[1, 5:] == 0).all()
    used = np.zeros((B, S2), bool)
    for b_ in range(B):
        sel = idx[b_].reshape(-1)
        used[b_, sel[sel >= 0]] = True
    assert (dv[~used] == 0).all() and (dk[~used] == 0).all()
    assert np.abs(dv[used]).max() > 0
    assert torch.equal(a[0], b[0]) and torch.equal(a[3], b[3])          # per-row results: no atomics
    for x, y, n in zip(a, b, NAMES):
        sfa_grad_acceptance_rule(host(x), host(y), "fp16", name=n, ulps=1.0)
