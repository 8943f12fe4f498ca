"""Ordered top-k on rows built to stress the selection: scores are set exactly (one non-zero product
per head), so the expected order (score descending, position ascending) is known bit for bit.

Rows of up to 8192 keys run li_topk_bins_kernel, longer ones li_topk_bins_stream_kernel.
Covers what random normal data never shows the histogram-based kernels: every score equal, a handful
of distinct values (bins holding hundreds of ties), an outlier that dominates the row's scale,
sign changes and zeros around the threshold, lengths at and next to sparse_count, fp16."""
import numpy as np
import pytest
import torch

from tests.util import host

pytestmark = pytest.mark.gpu


def _run(values, K, dtype=torch.bfloat16):
    """values [rows, S2] (exactly representable in `dtype`) -> indices, values of the operator.
    Two heads: q = (+e0, -e0), w = (+1, -1), k[:, 0] = value: score = relu(v) - relu(-v) = v."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton
    rows, S2 = values.shape
    q = torch.zeros(1, rows, 2, 128, dtype=dtype, device="cuda")
    q[0, :, 0, 0] = 1.0
    q[0, :, 1, 0] = -1.0
    w = torch.tensor([1.0, -1.0], device="cuda").repeat(1, rows, 1)
    out_i, out_v = [], []
    for r in range(rows):                      # one key tensor per row pattern
        k = torch.zeros(1, S2, 1, 128, dtype=dtype, device="cuda")
        k[0, :, 0, 0] = torch.from_numpy(values[r]).to(dtype).cuda()
        i, v = lightning_indexer_triton(q[:, r:r + 1], k, w[:, r:r + 1], sparse_count=K, sparse_mode=0,
                                        return_value=True)
        out_i.append(host(i)[0, 0, 0])
        out_v.append(host(v)[0, 0, 0])
    return np.stack(out_i), np.stack(out_v)


def _expected(values, K):
    rows, S2 = values.shape
    idx = np.full((rows, K), -1, np.int32)
    val = np.zeros((rows, K), np.float32)
    for r in range(rows):
        v = values[r] + 0.0                                        # -0 ranks as +0
        order = np.lexsort((np.arange(S2), -v))[:K]                # score descending, position ascending
        idx[r, :len(order)] = order
        val[r, :len(order)] = values[r][order]
    return idx, val


def _bf16(x):
    return torch.from_numpy(np.asarray(x, np.float32)).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("S2,K", [(8192, 2048), (8192, 512), (5000, 2048), (2048, 2048), (2049, 2048),
                                  (2047, 2048), (300, 1024), (1, 64),
                                  (8193, 2048), (20000, 2048), (70001, 300)])   # longer rows: the streaming kernel
def test_constructed_rows_select_and_order_exactly(S2, K):
    rng = np.random.RandomState(S2 + K)
    pos = np.arange(S2)
    rows = [
        np.full(S2, 1.0),                                                   # every score equal
        np.where(pos % 2 == 1, 2.0, 1.0),                                   # two values, ties cut by position
        rng.choice([-3.0, -0.5, 0.0, 0.25, 7.0], size=S2),                  # five keys, hundreds of ties each
        _bf16(rng.randn(S2)),                                               # zero-mean: threshold near 0
        _bf16(np.concatenate([[3.0e4], rng.randn(S2 - 1)]) if S2 > 1 else [3.0e4]),   # one huge outlier
        _bf16(np.concatenate([np.full(min(S2, 40), 1.0e6), rng.randn(max(S2 - 40, 0)) * 1e-3])),   # outliers set the scale
        _bf16(-np.abs(rng.randn(S2)) - 1.0),                                # all negative
        _bf16(np.linspace(-4.0, 4.0, S2)),                                  # increasing: best keys last
        np.where(rng.rand(S2) < 0.7, 0.0, _bf16(rng.randn(S2))),            # mostly exact zeros (and -0 below)
        _bf16(np.exp(rng.randn(S2) * 2.0)),                                 # heavy tail
    ]
    rows[8][::7] = -0.0
    values = np.stack([np.asarray(r, np.float32) for r in rows])
    got_i, got_v = _run(values, K)
    exp_i, exp_v = _expected(values, K)
    for r in range(values.shape[0]):
        np.testing.assert_array_equal(got_i[r], exp_i[r], err_msg=f"row pattern {r}")
        np.testing.assert_array_equal(got_v[r] + 0.0, exp_v[r] + 0.0, err_msg=f"row pattern {r}")


def test_constructed_rows_fp16():
    rng = np.random.RandomState(5)
    S2, K = 4096, 1024
    f16 = lambda x: np.asarray(x, np.float32).astype(np.float16).astype(np.float32)   # noqa: E731
    values = np.stack([f16(rng.randn(S2)), f16(rng.choice([0.5, 0.5009765625, -2.0], size=S2)),
                       f16(np.full(S2, 3.0)), f16(np.exp(rng.randn(S2)))])
    got_i, got_v = _run(values, K, torch.float16)
    exp_i, exp_v = _expected(values, K)
    np.testing.assert_array_equal(got_i, exp_i)
    np.testing.assert_array_equal(got_v, exp_v)
