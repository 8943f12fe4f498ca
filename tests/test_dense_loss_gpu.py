"""GPU parity of the dense lightning-indexer operators (softmax LSE helper and KL-loss backward)
through the C ABI: against the committed outputs of the numpy baselines in the reference's own test
module (tests/golden/dense_loss_*.npz), and against the oracle on the reference's configuration
list, with valid lengths, bf16, and the statistics computed internally."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import dense_indexer_lse_oracle, dense_loss_backward_oracle
from oracle.dense_loss_oracle import dense_softmax_stats
from oracle.inputs import dense_loss_inputs
from tests.golden.cases import DENSE_LOSS_CASES, dense_loss_case_inputs
from tests.util import dev, host, tdtype

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ATOL = RTOL = 1e-2          # test_dense_loss_backward_triton.py:10-11


def _check(ref, got, dtype):
    d_qi, d_ki, d_w, loss = got
    assert loss.shape == (1,) and loss.dtype == torch.float32
    bits = 10 if dtype == "fp16" else 7
    for name, r, g in (("d_query_index", ref["dQueryIndex"], d_qi), ("d_key_index", ref["dKeyIndex"], d_ki),
                       ("d_weights", ref["dW"], d_w)):
        a, b = np.asarray(r, np.float64), host(g).astype(np.float64)
        assert a.shape == b.shape and np.isfinite(b).all(), name
        np.testing.assert_allclose(b, a, atol=ATOL, rtol=RTOL, err_msg=name)          # the reference's rule
        # this build's rule: 1.5 units in the last place of the output dtype plus the fp32 noise that the
        # exponential of large index scores amplifies (3e-4 of the tensor's largest magnitude)
        mag = np.maximum(np.maximum(np.abs(a), np.abs(b)), 1e-30)
        tol = 1.5 * 2.0 ** (np.floor(np.log2(mag)) - bits) + 3e-4 * np.abs(a).max()
        assert (np.abs(a - b) <= tol).all(), f"{name}: max |diff| {np.abs(a - b).max():.3e}"
    assert abs(float(loss[0]) - float(ref["loss"][0])) <= 3e-4 * max(abs(float(ref["loss"][0])), 1.0)


def _tensors(q, k, qr, kr, qi, ki, w, dtype):
    dt = tdtype(dtype)
    return [dev(x, dt) for x in (q, k, qr, kr, qi, ki, w)]


@pytest.mark.parametrize("name", sorted(DENSE_LOSS_CASES))
def test_dense_operators_match_the_reference_baselines(name):
    from dsa_triton_ascend_b200 import DenseLightningIndexerGradKLLossTriton, DenseLightningIndexerSoftmaxLseTriton
    q, k, qr, kr, qi, ki, w, scale, c = dense_loss_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    tq, tk, tqr, tkr, tqi, tki, tw = _tensors(q, k, qr, kr, qi, ki, w, "fp16")
    mx, sm = DenseLightningIndexerSoftmaxLseTriton()(tqi, tki, tw, layout="BSND", sparse_mode=3)
    assert mx.shape == (c["B"], 1, c["S1"]) and mx.dtype == torch.float32
    np.testing.assert_allclose(host(mx), g["max_index"], rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(host(sm), g["sum_index"], rtol=2e-4)
    # the fixture's statistics, so that only the backward is compared
    got = DenseLightningIndexerGradKLLossTriton()(
        tq, tk, tqi, tki, tw, dev(g["sm_max"]), dev(g["sm_sum"]), dev(g["max_index"]), dev(g["sum_index"]),
        scale_value=scale, query_rope=tqr, key_rope=tkr)
    _check(g, got, "fp16")


_CORE = [(1, 2, 64, 32, 32, d, g, di) for d in (128, 256, 512) for g in (32, 64, 128) for di in (128, 256, 512)]


@pytest.mark.parametrize("B,S1,S2,N1,N2,D,G,Di", _CORE[::3] + [(1, 3, 96, 32, 32, 128, 32, 128),
                                                              (1, 4, 128, 32, 32, 128, 32, 128),
                                                              (1, 64, 512, 64, 1, 512, 64, 128),
                                                              (2, 5, 80, 32, 16, 128, 32, 128),
                                                              (1, 7, 64, 16, 4, 128, 32, 128),
                                                              (1, 40, 256, 32, 32, 128, 32, 128)])
@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_dense_operators_against_the_oracle_on_the_reference_configurations(B, S1, S2, N1, N2, D, G, Di, dtype):
    """test_dense_loss_backward_triton.py:20-31 (every third of the 27 core configurations, the two
    tail configurations) plus an MQA shape with more rows, two grouped-query shapes and a multi-head
    shape whose rows fill several blocks; statistics from the operators themselves,
    and the path that computes the index statistics internally gives the same result (:462-476)."""
    from dsa_triton_ascend_b200 import dense_lightning_indexer_softmax_lse_triton, dense_loss_backward_triton
    q, k, qr, kr, qi, ki, w = dense_loss_inputs(11, B, S1, S2, N1, N2, D, G, Di, dtype=dtype)
    scale = 1.0 / math.sqrt(D + 64.0)
    sm_max, sm_sum = dense_softmax_stats(q, k, qr, kr, scale)
    tq, tk, tqr, tkr, tqi, tki, tw = _tensors(q, k, qr, kr, qi, ki, w, dtype)
    mx, sm = dense_lightning_indexer_softmax_lse_triton(tqi, tki, tw)
    ref_mx, ref_sm = dense_indexer_lse_oracle(qi, ki, w)
    np.testing.assert_allclose(host(mx), ref_mx, rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(host(sm), ref_sm, rtol=3e-4)
    ref = dense_loss_backward_oracle(q, k, qr, kr, qi, ki, w, sm_max, sm_sum, host(mx), host(sm), scale)
    got = dense_loss_backward_triton(tq, tk, tqi, tki, tw, dev(sm_max), dev(sm_sum), mx, sm, scale,
                                     query_rope=tqr, key_rope=tkr)
    assert got[0].dtype == tqi.dtype and got[1].dtype == tki.dtype and got[2].dtype == tw.dtype
    _check(ref, got, dtype)
    auto = dense_loss_backward_triton(tq, tk, tqi, tki, tw, dev(sm_max), dev(sm_sum), scale_value=scale,
                                      query_rope=tqr, key_rope=tkr)
    # (the index scores of a row are summed over head chunks with fp32 atomics: two runs agree to
    # summation noise, not bit for bit)
    _check(ref, auto, dtype)
    assert abs(float(auto[3][0]) - float(got[3][0])) <= 3e-4 * abs(float(got[3][0]))


def test_dense_operators_with_valid_lengths_gqa_and_no_rope():
    B, S1, S2, N1, N2, D, G, Di = 2, 10, 72, 32, 4, 128, 24, 128
    q, k, qr, kr, qi, ki, w = dense_loss_inputs(13, B, S1, S2, N1, N2, D, G, Di, dtype="bf16")
    act_q, act_k = [10, 7], [72, 3]            # batch 1: rows 0..3 see no key, rows 7.. are padding
    scale = 1.0 / math.sqrt(D)
    zq, zk = np.zeros((B, S1, N1, 0), np.float32), np.zeros((B, S2, N2, 0), np.float32)
    sm_max, sm_sum = dense_softmax_stats(q, k, zq, zk, scale, act_q, act_k)
    sm_max = np.where(np.isfinite(sm_max), sm_max, 0.0).astype(np.float32)
    from dsa_triton_ascend_b200 import DenseLossBackwardTriton, npu_dense_lightning_indexer_softmax_lse_triton
    tq, tk, _, _, tqi, tki, tw = _tensors(q, k, qr, kr, qi, ki, w, "bf16")
    tw = tw.float()
    w32 = host(tw)
    mx, sm = npu_dense_lightning_indexer_softmax_lse_triton(tqi, tki, tw, actual_seq_qlen=act_q, actual_seq_klen=act_k)
    ref_mx, ref_sm = dense_indexer_lse_oracle(qi, ki, w32, act_q, act_k)
    assert np.array_equal(np.isinf(host(mx)), np.isinf(ref_mx)) and (host(sm)[ref_sm == 0] == 0).all()
    fin = np.isfinite(ref_mx)
    np.testing.assert_allclose(host(mx)[fin], ref_mx[fin], rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(host(sm), ref_sm, rtol=3e-4)
    ref = dense_loss_backward_oracle(q, k, None, None, qi, ki, w32, sm_max, sm_sum, host(mx), host(sm), scale,
                                     act_q, act_k)
    got = DenseLossBackwardTriton(scale_value=scale)(tq, tk, tqi, tki, tw, dev(sm_max), dev(sm_sum), mx, sm,
                                                     actual_seq_qlen=act_q, actual_seq_klen=act_k)
    assert got[2].dtype == torch.float32
    _check(ref, got, "bf16")
    d_qi = host(got[0])
    assert (d_qi[1, :4] == 0).all() and (d_qi[1, 7:] == 0).all() and np.abs(d_qi[1, 4:7]).max() > 0
