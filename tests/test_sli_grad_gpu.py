"""GPU parity of the indexer's KL-loss backward (sparse_lightning_indexer_grad_kl_loss_triton) through
the C ABI: against the committed outputs of the unmodified reference golden
(tests/golden/sli_grad_*.npz), against the numpy oracle on the reference's shape list, with valid
lengths, bf16, fp32 weights and no rope, and against torch autograd through a dense restatement of
the loss."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import sli_grad_kl_loss_oracle
from oracle.inputs import sli_grad_inputs
from oracle.sli_grad_oracle import softmax_stats
from tests.golden.cases import SLI_GRAD_CASES, sli_grad_case_inputs
from tests.util import dev, host, tdtype

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NEAR_ZERO = 1e-2


def _reference_rule(ref, got, dtype):
    """test_sli_grad_kl_loss_triton.py:178-192: allclose at 2e-3 (fp16) / 1e-2 (bf16) after zeroing
    the elements that are below 1e-2 in both."""
    tol = 2e-3 if dtype == "fp16" else 1e-2
    a, b = np.asarray(ref, np.float32), np.asarray(got, np.float32)
    near = (np.abs(a) < NEAR_ZERO) & (np.abs(b) < NEAR_ZERO)
    np.testing.assert_allclose(np.where(near, 0.0, b), np.where(near, 0.0, a), atol=tol, rtol=tol)


def _acceptance_rule(ref, got, dtype, name, out_dtype=None):
    """This build's rule: within 1.5 units in the last place of the output dtype (the result is
    rounded once from an fp32 sum), plus 1e-5 of the tensor's largest magnitude for sums that cancel."""
    a, b = np.asarray(ref, np.float64), np.asarray(got, np.float64)
    assert np.isfinite(b).all(), name
    mag = np.maximum(np.maximum(np.abs(a), np.abs(b)), 1e-30)
    bits = {"fp16": 10, "bf16": 7, "fp32": 20}[out_dtype or dtype]
    tol = 1.5 * 2.0 ** (np.floor(np.log2(mag)) - bits) + 1e-5 * np.abs(a).max()
    bad = np.abs(a - b) > tol
    assert not bad.any(), f"{name}: {bad.sum()} of {bad.size} outside, max |diff| {np.abs(a - b).max():.3e}"


def _run(q, k, qr, kr, qi, ki, w, si, sm_max, sm_sum, scale, dtype, w_fp32=False, **kw):
    from dsa_triton_ascend_b200 import SparseLightningIndexerGradKLLossTriton
    dt = tdtype(dtype)
    cell = SparseLightningIndexerGradKLLossTriton(scale_value=scale)
    return cell(dev(q, dt), dev(k, dt), dev(qi, dt), dev(ki, dt), dev(w, None if w_fp32 else dt), dev(si),
                dev(sm_max), dev(sm_sum), query_rope=None if qr is None else dev(qr, dt),
                key_rope=None if kr is None else dev(kr, dt), **kw)


def _check(ref, got, dtype, w_dtype=None):
    d_qi, d_ki, d_w, loss = got
    assert loss.shape == (1,) and loss.dtype == torch.float32
    for name, r, g, od in (("d_query_index", ref["dQueryIndex"], d_qi, dtype), ("d_key_index", ref["dKeyIndex"], d_ki, dtype),
                           ("d_weights", ref["dW"], d_w, w_dtype or dtype)):
        assert tuple(g.shape) == r.shape, name
        _reference_rule(r, host(g), dtype)
        _acceptance_rule(r, host(g), dtype, name, od)
    _reference_rule(ref["loss"], host(loss), dtype)
    assert abs(float(loss[0]) - float(ref["loss"][0])) <= 2e-5 * max(abs(float(ref["loss"][0])), 1.0)


@pytest.mark.parametrize("name", sorted(SLI_GRAD_CASES))
def test_sli_grad_matches_the_reference_golden(name):
    q, k, qr, kr, qi, ki, w, si, scale, c = sli_grad_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    got = _run(q, k, qr, kr, qi, ki, w, si, g["sm_max"], g["sm_sum"], scale, "fp16")
    assert got[0].dtype == torch.float16 and got[1].dtype == torch.float16 and got[2].dtype == torch.float16
    _check(g, got, "fp16")


@pytest.mark.parametrize("B,S1,S2,N1,D,G,Di,topk,pattern", [
    (1, 4, 2048, 64, 512, 64, 128, 2048, "causal_random"),    # test_sli_grad_kl_loss_triton.py:48
    (1, 4, 2048, 32, 128, 32, 128, 1024, "causal_random"),    # :49
    (1, 2, 2048, 128, 512, 128, 512, 2048, "causal_random"),  # :51, every dimension at its maximum
    (1, 4, 2048, 64, 128, 32, 256, 1024, "causal_continuous"),   # :55
    (2, 64, 512, 64, 512, 64, 128, 256, "causal_random"),     # more rows than a chunk of keys, two batches
])
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_sli_grad_against_the_oracle_on_the_reference_shapes(B, S1, S2, N1, D, G, Di, topk, pattern, dtype):
    q, k, qr, kr, qi, ki, w, si = sli_grad_inputs(7, B, S1, S2, N1, D, G, Di, topk, pattern, dtype=dtype)
    scale = 1.0 / math.sqrt(D)
    sm_max, sm_sum = softmax_stats(q, k, qr, kr, scale, dtype=dtype)
    ref = sli_grad_kl_loss_oracle(q, k, qr, kr, qi, ki, w, si, sm_max, sm_sum, scale, dtype=dtype)
    _check(ref, _run(q, k, qr, kr, qi, ki, w, si, sm_max, sm_sum, scale, dtype), dtype)


def test_sli_grad_valid_lengths_no_rope_fp32_weights_and_out_of_range_indices():
    """Rows beyond the valid query length and rows without visible keys give zero gradients and no
    loss; indices outside [0, S2) are clipped like the reference clips them (:96); the rope parts are
    optional; weights may be fp32 (d_weights follows their dtype)."""
    B, S1, S2, N1, D, G, Di, topk = 2, 12, 96, 32, 128, 24, 128, 40
    q, k, qr, kr, qi, ki, w, si = sli_grad_inputs(9, B, S1, S2, N1, D, G, Di, topk, "random", dtype="bf16")
    si[0, 3, 0, ::5] = -1
    si[1, 2, 0, ::7] = S2 + 50
    act_q, act_k = [12, 9], [96, 4]              # batch 1: rows 0..4 see no key, rows 9.. are padding
    scale = 1.0 / math.sqrt(D)
    zr, zk = np.zeros((B, S1, N1, 0), np.float32), np.zeros((B, S2, 1, 0), np.float32)
    sm_max, sm_sum = softmax_stats(q, k, zr, zk, scale, act_q, act_k, dtype="bf16")
    sm_max = np.where(np.isfinite(sm_max), sm_max, 0.0).astype(np.float32)
    ref = sli_grad_kl_loss_oracle(q, k, None, None, qi, ki, w, si, sm_max, sm_sum, scale, act_q, act_k, dtype="bf16")
    got = _run(q, k, None, None, qi, ki, w, si, sm_max, sm_sum, scale, "bf16", w_fp32=True,
               actual_seq_qlen=act_q, actual_seq_klen=act_k)
    assert got[2].dtype == torch.float32
    _check(ref, got, "bf16", w_dtype="fp32")
    d_qi, d_ki, d_w, _ = [host(t) for t in got]
    assert (d_qi[1, :5] == 0).all() and (d_qi[1, 9:] == 0).all() and (d_w[1, :5] == 0).all() and (d_w[1, 9:] == 0).all()
    assert np.abs(d_qi[1, 5:9]).max() > 0


def test_sli_grad_agrees_with_autograd_of_the_kl_loss():
    """Independent derivation by torch autograd in fp64.  loss = sum_rows KL(p || softmax(I)) with p
    fixed.  The operator's dI = softmax(I) - p (sli_grad_kl_loss_numpy.py:106) is the gradient of that
    loss when p sums to one; p is the attention distribution restricted to the selected keys, so in
    general it is the gradient of KL + (1 - sum p) * logsumexp(I), which is what is differentiated."""
    B, S1, S2, N1, D, G, Di, topk = 1, 6, 64, 32, 128, 8, 128, 24
    q, k, qr, kr, qi, ki, w, si = sli_grad_inputs(3, B, S1, S2, N1, D, G, Di, topk, "causal_random")
    scale = 1.0 / math.sqrt(D)
    sm_max, sm_sum = softmax_stats(q, k, qr, kr, scale)
    got = _run(q, k, qr, kr, qi, ki, w, si, sm_max, sm_sum, scale, "fp16")
    t = lambda x: torch.tensor(x, dtype=torch.float64)   # noqa: E731
    QI, KI, W = t(qi).requires_grad_(), t(ki).requires_grad_(), t(w).requires_grad_()
    total = torch.zeros((), dtype=torch.float64)
    extra = torch.zeros((), dtype=torch.float64)
    clamped = 0.0
    for s1 in range(S1):
        n = min(topk, S2 - S1 + s1 + 1)
        idx = torch.tensor(si[0, s1, 0, :n].astype(np.int64))
        sc = (t(q[0, s1]) @ t(k[0, :, 0])[idx].T + t(qr[0, s1]) @ t(kr[0, :, 0])[idx].T) * scale
        p = (torch.exp(sc - t(sm_max[0, 0, s1])[:, None]) / t(sm_sum[0, 0, s1])[:, None]).mean(0)
        i_vec = W[0, s1] @ torch.relu(QI[0, s1] @ KI[0, :, 0][idx].T)
        total = total + (p * (torch.log(p) - torch.log_softmax(i_vec, 0))).sum()
        # the reported loss clamps both distributions at 1e-8 (sli_grad_kl_loss_numpy.py:112-116)
        clamped += float((p * (torch.log(p) - torch.log_softmax(i_vec, 0).clamp_min(math.log(1e-8)))).sum().detach())
        extra = extra + (1.0 - p.sum()) * torch.logsumexp(i_vec, 0)
    (total + extra).backward()
    for name, a, b in (("d_query_index", got[0], QI.grad), ("d_key_index", got[1], KI.grad), ("d_weights", got[2], W.grad)):
        a, b = host(a), b.numpy()
        assert np.abs(a - b).max() <= 3e-3 * np.abs(b).max() + 1e-6, f"{name}: {np.abs(a - b).max()} vs {np.abs(b).max()}"
    assert abs(float(got[3][0]) - clamped) <= 1e-3 * abs(clamped)
