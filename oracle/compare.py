"""Comparison rules used by the parity tests (test infrastructure only).

Two families:
  * the reference's own test rules, restated from test_li_triton.py:195-237 (valid-count
    equality, boundary-tie tolerance for set differences, banded relative error on the
    selected values) and test_sfa_triton.py:88-123 (percentage of elements inside
    rtol/atol, no outlier with relative error >= 10);
    (test_sfa_grad_triton.py:89-121 for the backward: rtol 6e-2 / atol 5e-2 in bf16, 3e-2 / 2e-2 in
    fp16, atol scaled by sqrt(S1) for the scatter-added gradients, 99.5 % inside);
  * the stricter acceptance rules of this build: positional index equality wherever
    the fp32 gap between the k-th and (k+1)-th score exceeds 1e-3 relative; attention
    output within atol = rtol = 2e-2 (bf16) and softmax statistics within 1e-3 relative.
"""
import numpy as np


def li_reference_rule(idx, val, ref_idx, ref_val, rtol=5e-3, atol=2.5e-5,
                      diff_thd=0.01, max_diff_hd=0.1, pct_thd=0.05):
    """Raises AssertionError unless (idx, val) agrees with (ref_idx, ref_val) under the
    reference test's semantics.  Arrays are [..., k]; rows are compared independently."""
    k = idx.shape[-1]
    ti, ri = idx.reshape(-1, k), ref_idx.reshape(-1, k)
    tv, rv = val.reshape(-1, k).astype(np.float32), ref_val.reshape(-1, k).astype(np.float32)
    tv_all, rv_all = [], []
    for r in range(ti.shape[0]):
        tm, rm = ti[r] != -1, ri[r] != -1
        assert tm.sum() == rm.sum(), f"row {r}: valid count {tm.sum()} != {rm.sum()}"
        a, b = np.sort(tv[r][tm]), np.sort(rv[r][rm])
        tv_all.append(a)
        rv_all.append(b)
        only = set(ti[r][tm].tolist()) - set(ri[r][rm].tolist())
        if only and b.size:
            bound = b[0]
            for s2 in only:
                v = tv[r][np.where(ti[r] == s2)[0][0]]
                assert abs(v - bound) <= rtol * abs(bound) + atol, \
                    f"row {r}: index {s2} (value {v}) is not a boundary tie of {bound}"
    a = np.concatenate(tv_all) if tv_all else np.zeros(0, np.float32)
    b = np.concatenate(rv_all) if rv_all else np.zeros(0, np.float32)
    close = np.isclose(a, b, rtol=rtol, atol=atol)
    band = np.maximum(np.maximum(np.abs(a), np.abs(b)), (1.0 / (1 << 14)) / diff_thd) + 1e-9
    err = np.abs(a - b) / band
    fulfil = close.mean() * 100.0 if close.size else 100.0
    worst = err[~close].max() if (~close).any() else 0.0
    assert fulfil >= (1 - pct_thd) * 100.0 and worst < max_diff_hd, \
        f"selected values: {fulfil:.3f}% close, worst banded error {worst:.4f}"


def li_positional_rule(idx, ref_idx, gap_ok_rows=None):
    """Positional equality of index rows; `gap_ok_rows` (bool per row) limits the check to
    rows whose k/(k+1) fp32 score gap is large enough to make the order unambiguous."""
    k = idx.shape[-1]
    a, b = idx.reshape(-1, k), ref_idx.reshape(-1, k)
    same = (a == b).all(axis=1)
    if gap_ok_rows is not None:
        same = same | ~np.asarray(gap_ok_rows).reshape(-1)
    bad = np.nonzero(~same)[0]
    assert bad.size == 0, f"{bad.size} rows differ positionally, first {bad[:8].tolist()}"


def sfa_reference_rule(a, b, dtype="bf16", pct_thd=None, rtol=None, atol=None):
    """True when `a` is close to `b` in the sense of test_sfa_triton.py:88-123."""
    if dtype == "bf16":
        rtol = 7.8125e-3 if rtol is None else rtol
        atol = 7e-4 if atol is None else atol
    else:
        rtol = 5e-3 if rtol is None else rtol
        atol = 2.5e-4 if atol is None else atol
    pct_thd = 99.5 if pct_thd is None else pct_thd
    a = np.asarray(a, np.float32).ravel()
    b = np.asarray(b, np.float32).ravel()
    assert a.shape == b.shape
    close = np.isclose(a, b, rtol=rtol, atol=atol, equal_nan=True)
    if close.mean() * 100.0 < pct_thd:
        return False
    rel = np.abs(a - b) / (np.maximum(np.abs(a), np.abs(b)) + 1e-10)
    return not np.any(rel[~close] >= 10)


def sfa_acceptance_rule(out, smax, ssum, ref_out, ref_smax, ref_ssum, tol_out=2e-2, tol_stat=1e-3):
    """atol = rtol = tol_out on the output; tol_stat relative on both statistics."""
    out, ref_out = np.asarray(out, np.float32), np.asarray(ref_out, np.float32)
    bad = ~np.isclose(out, ref_out, rtol=tol_out, atol=tol_out)
    assert not bad.any(), f"attention_out: {bad.sum()} elements outside {tol_out}, " \
                          f"max |diff| {np.abs(out - ref_out).max():.4e}"
    for name, x, y in (("softmax_max", smax, ref_smax), ("softmax_sum", ssum, ref_ssum)):
        x, y = np.asarray(x, np.float32), np.asarray(y, np.float32)
        bad = ~np.isclose(x, y, rtol=tol_stat, atol=tol_stat * 1e-2)
        assert not bad.any(), f"{name}: {bad.sum()} elements outside {tol_stat} relative, " \
                              f"max |diff| {np.abs(x - y).max():.4e}"


def sfa_grad_reference_rule(a, b, dtype="bf16", scale=1.0):
    """True when gradient `a` is close to `b` in the sense of test_sfa_grad_triton.py:89-121."""
    rtol = 6e-2 if dtype == "bf16" else 3e-2
    atol = (5e-2 if dtype == "bf16" else 2e-2) * scale
    return sfa_reference_rule(a, b, dtype, pct_thd=99.5, rtol=rtol, atol=atol)


def sfa_grad_acceptance_rule(a, b, dtype="bf16", name="gradient", ulps=2.0, noise=2e-6):
    """Stricter rule of this build for a gradient given the SAME forward state as the checker: every
    element within `ulps` units in the last place of the io dtype (taken at the larger magnitude of
    the two), plus `noise` times the largest magnitude of the tensor for fp32 sums that cancel."""
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    assert a.shape == b.shape, f"{name}: shape {a.shape} vs {b.shape}"
    assert np.isfinite(a).all(), f"{name}: non-finite values"
    mag = np.maximum(np.maximum(np.abs(a), np.abs(b)).astype(np.float64), 1e-30)
    e = np.floor(np.log2(mag))
    ulp = 2.0 ** (e - 7) if dtype == "bf16" else np.maximum(2.0 ** (e - 10), 2.0 ** -24)
    tol = ulps * ulp + noise * float(np.abs(b).max())
    bad = np.abs(a.astype(np.float64) - b) > tol
    assert not bad.any(), f"{name}: {bad.sum()} of {bad.size} elements more than {ulps} ulp apart, " \
                          f"max |diff| {np.abs(a - b).max():.4e} at |ref| max {np.abs(b).max():.4e}"
