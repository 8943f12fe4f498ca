"""Pins the numpy restatement under oracle/ to outputs of the unmodified reference goldens.

tests/golden/*.npz were produced by tests/golden/make_golden.py from
lightning_indexer_numpy.lightning_indexer_golden_bsnd and
sparse_flash_attention_numpy.sparse_flash_attention_golden_bsnd (and, for the backward cases,
sparse_flash_attention_grad_numpy.sparse_flash_attention_grad_golden_bsnd) on the seeded inputs
of tests/golden/cases.py; the forward restatements have to reproduce them bit for bit, the
backward one to the last place of the io dtype.
"""
import os

import numpy as np
import pytest

from oracle import (dense_indexer_lse_oracle, dense_loss_backward_oracle, lightning_indexer_oracle,
                    sli_grad_kl_loss_oracle, sparse_flash_attention_grad_oracle, sparse_flash_attention_oracle)
from tests.golden.cases import (DENSE_LOSS_CASES, LI_CASES, SFA_CASES, SFA_GRAD_CASES, SLI_GRAD_CASES,
                                dense_loss_case_inputs, li_case_inputs, sfa_case_inputs, sfa_grad_case_inputs,
                                sli_grad_case_inputs)

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(LI_CASES))
@pytest.mark.parametrize("rank", ["io", "fp32"])
def test_li_oracle_matches_reference_golden(name, rank):
    q, k, w, act_q, act_k, c = li_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    rows = [tuple(r) for r in g["rows"].tolist()]
    idx, val = lightning_indexer_oracle(
        q, k, w, act_q, act_k, sparse_count=c["k"], sparse_mode=c["mode"], return_value=True,
        value_dtype=c["dtype"], rank_dtype=None if rank == "io" else "fp32", rows=rows)
    sel = g["rows"]
    got_idx, got_val = idx[sel[:, 0], sel[:, 1]], val[sel[:, 0], sel[:, 1]]
    np.testing.assert_array_equal(got_idx, g[f"idx_{rank}"])
    if rank == "io":
        np.testing.assert_array_equal(got_val, g["val_io"])
    else:
        # the patched reference emits un-rounded values; the oracle rounds what it emits
        from oracle import quantize
        np.testing.assert_array_equal(got_val, quantize(g["val_fp32"], c["dtype"]))


@pytest.mark.parametrize("name", sorted(SFA_CASES))
def test_sfa_oracle_matches_reference_golden(name):
    q, k, qr, kr, idx, act_q, act_k, scale, c = sfa_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    rows = [tuple(r) for r in g["rows"].tolist()]
    out, smax, ssum = sparse_flash_attention_oracle(
        q, k, idx, qr, kr, scale, act_q, act_k, sparse_block_size=c["block"],
        sparse_mode=c["mode"], return_softmax_lse=True, dtype=c["dtype"], rows=rows)
    sel = g["rows"]
    np.testing.assert_array_equal(out[sel[:, 0], sel[:, 1]], g["out"].astype(np.float32))
    np.testing.assert_array_equal(smax[sel[:, 0], 0, sel[:, 1]], g["smax"])
    np.testing.assert_array_equal(ssum[sel[:, 0], 0, sel[:, 1]], g["ssum"])

def _ulp(x, dtype):
    """Spacing of the io dtype at |x| (bf16: 8 mantissa bits, fp16: 11; fp16 subnormal floor)."""
    a = np.maximum(np.abs(x).astype(np.float64), 1e-30)
    e = np.floor(np.log2(a))
    return np.where(dtype == "bf16", 2.0 ** (e - 7), np.maximum(2.0 ** (e - 10), 2.0 ** -24))


@pytest.mark.parametrize("name", sorted(SFA_GRAD_CASES))
def test_sfa_grad_oracle_matches_reference_golden(name):
    """The forward state comes from the forward oracle (bit-identical to the forward golden that the
    fixture generator used).  The backward restatement sums the same fp32 terms as the golden in
    another order (matrix products instead of a per-head loop), so results agree except where the
    two fp32 sums round to neighbouring io-dtype values: at most one unit in the last place apart
    (plus the fp32 noise of sums that cancel), and equal on nearly every element."""
    q, k, qr, kr, do, idx, act_q, act_k, scale, c = sfa_grad_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    out, smax, ssum = sparse_flash_attention_oracle(
        q, k, idx, qr, kr, scale, act_q, act_k, sparse_block_size=c["block"], sparse_mode=c["mode"],
        return_softmax_lse=True, dtype=c["dtype"])
    got = sparse_flash_attention_grad_oracle(
        q, k, idx, do, out, smax, ssum, qr, kr, scale, act_q, act_k, sparse_block_size=c["block"],
        sparse_mode=c["mode"], dtype=c["dtype"])
    for n, a in zip(("d_query", "d_key", "d_value", "d_query_rope", "d_key_rope"), got):
        b = g[n]
        assert a.shape == b.shape, n
        noise = 1e-6 * np.abs(b).max()
        assert (np.abs(a - b) <= _ulp(b, c["dtype"]) + noise).all(), f"{n}: more than one ulp apart"
        assert (a == b).mean() >= 0.98, f"{n}: {(a == b).mean():.4f} equal"
    # rows the golden never visits (past the valid query length) stay exactly zero
    for b_ in range(c["B"]):
        assert (got[0][b_, int(act_q[b_]):] == 0).all() and (got[3][b_, int(act_q[b_]):] == 0).all()
        assert (got[1][b_, int(act_k[b_]):] == 0).all() and (got[2][b_, int(act_k[b_]):] == 0).all()

@pytest.mark.parametrize("name", sorted(SLI_GRAD_CASES))
def test_sli_grad_oracle_matches_reference_golden(name):
    """sli_grad_kl_loss_numpy.numpy_reference returns un-rounded fp32 results; the restatement does the
    same sums with the heads of a row batched into matrix products, so the two agree to fp32
    summation noise: 2e-5 of each tensor's largest magnitude.  The statistics stored beside the
    outputs (the golden file's own `_compute_sm_stats`, which rounds scores to fp16 first) also pin
    `oracle.sli_grad_oracle.softmax_stats` to within that rounding."""
    from oracle.sli_grad_oracle import softmax_stats
    q, k, qr, kr, qi, ki, w, si, scale, c = sli_grad_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    got = sli_grad_kl_loss_oracle(q, k, qr, kr, qi, ki, w, si, g["sm_max"], g["sm_sum"], scale)
    for n in ("dQueryIndex", "dKeyIndex", "dW", "loss"):
        a, b = got[n], g[n]
        assert a.shape == b.shape, n
        assert np.abs(a - b).max() <= 2e-5 * max(np.abs(b).max(), 1e-3), f"{n}: {np.abs(a - b).max()}"
    m, s_ = softmax_stats(q, k, qr, kr, scale)
    np.testing.assert_allclose(m, g["sm_max"], rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(np.log(s_), np.log(g["sm_sum"]), rtol=0, atol=2e-2)

@pytest.mark.parametrize("name", sorted(DENSE_LOSS_CASES))
def test_dense_loss_oracle_matches_reference_baselines(name):
    """Fixtures: outputs of the numpy baselines in the reference's own test module
    (_dense_indexer_lse_numpy, _compute_softmax_stats, _dense_loss_backward_numpy).  The restatement
    batches the heads of a row into matrix products: agreement to fp32 summation noise, which the
    exponential of index scores in the hundreds amplifies to a few 1e-4 of a tensor's magnitude."""
    from oracle.dense_loss_oracle import dense_softmax_stats
    q, k, qr, kr, qi, ki, w, scale, c = dense_loss_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    mx_i, sm_i = dense_indexer_lse_oracle(qi, ki, w)
    np.testing.assert_allclose(mx_i, g["max_index"], rtol=1e-5, atol=1e-4)
    np.testing.assert_allclose(sm_i, g["sum_index"], rtol=1e-4)
    mx, sm = dense_softmax_stats(q, k, qr, kr, scale)
    np.testing.assert_allclose(mx, g["sm_max"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(sm, g["sm_sum"], rtol=1e-4)
    got = dense_loss_backward_oracle(q, k, qr, kr, qi, ki, w, g["sm_max"], g["sm_sum"], g["max_index"],
                                     g["sum_index"], scale)
    for n in ("dQueryIndex", "dKeyIndex", "dW", "loss"):
        a, b = got[n], g[n]
        assert a.shape == b.shape, n
        assert np.abs(a - b).max() <= 3e-4 * max(np.abs(b).max(), 1e-3), f"{n}: {np.abs(a - b).max()}"


def test_li_oracle_layout_adapters_roundtrip():
    from oracle import layouts
    rng = np.random.RandomState(3)
    lens = [5, 0, 9]
    x = rng.randn(14, 2, 4).astype(np.float32)
    dense = layouts.tnd_to_bsnd(x, lens)
    assert dense.shape == (3, 9, 2, 4) and (dense[0, 5:] == 0).all()
    np.testing.assert_array_equal(layouts.bsnd_to_tnd(dense, lens), x)
    cache = rng.randn(6, 4, 1, 3).astype(np.float32)
    bt = np.array([[2, 5, -1], [0, -1, 1]], dtype=np.int32)
    d = layouts.pa_to_bsnd(cache, bt, 12)
    np.testing.assert_array_equal(d[0, 4:8], cache[5])
    assert (d[0, 8:] == 0).all() and (d[1, 4:8] == 0).all()
    np.testing.assert_array_equal(d[1, 8:12], cache[1])
