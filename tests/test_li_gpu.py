"""GPU parity of lightning_indexer against the reference goldens (fixtures) and the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import lightning_indexer_oracle
from oracle.compare import li_reference_rule
from oracle import layouts
from tests.golden.cases import LI_CASES, li_case_inputs
from tests.util import dev, host, li_gap_ok, tdtype

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _li():
    import dsa_triton_ascend_b200.lightning_indexer as li
    return li


def _check_rows(idx, val, ref_idx, ref_val, gap_ok, min_positional=0.97):
    """Reference rule on everything; identical index sets on unambiguous rows; positional
    equality on nearly all rows (accumulation-order noise can flip a rounding boundary)."""
    li_reference_rule(idx, val, ref_idx, ref_val)
    k = idx.shape[-1]
    a, b = idx.reshape(-1, k), ref_idx.reshape(-1, k)
    g = gap_ok.reshape(-1)
    for r in range(a.shape[0]):
        if g[r]:
            assert set(a[r].tolist()) == set(b[r].tolist()), f"row {r}: index set differs from the golden"
    same = (a == b).all(axis=1)
    assert same.mean() >= min_positional, f"only {same.mean():.4f} of rows match position for position"
    # emitted values must equal the golden's wherever the position matches
    av, bv = val.reshape(-1, k), ref_val.reshape(-1, k)
    m = (a == b)
    assert np.isclose(av[m], bv[m], rtol=8e-3, atol=1e-6).all()


@pytest.mark.parametrize("name", sorted(LI_CASES))
@pytest.mark.parametrize("rank", ["io", "fp32"])
def test_li_matches_reference_golden(name, rank):
    li = _li()
    q, k, w, act_q, act_k, c = li_case_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    dt = tdtype(c["dtype"])
    li.set_rank_mode("io_dtype" if rank == "io" else "fp32")
    try:
        full = "act_q" not in c and "act_k" not in c
        idx, val = li.lightning_indexer_triton(
            dev(q, dt), dev(k, dt), dev(w),
            actual_seq_lengths_query=None if full else act_q.tolist(),
            actual_seq_lengths_key=None if full else act_k.tolist(),
            sparse_count=c["k"], sparse_mode=c["mode"], return_value=True)
    finally:
        li.set_rank_mode("io_dtype")
    assert idx.shape == (c["B"], c["S1"], c["N2"], c["k"]) and idx.dtype == torch.int32
    assert val.dtype == dt
    idx, val = host(idx), host(val)
    sel = g["rows"]
    rows = [tuple(r) for r in sel.tolist()]
    got_i, got_v = idx[sel[:, 0], sel[:, 1]], val[sel[:, 0], sel[:, 1]]
    ref_i = g[f"idx_{rank}"]
    ref_v = g["val_io"] if rank == "io" else g["val_fp32"]
    gap = li_gap_ok(q, k, w, act_q, act_k, rows, c["N2"], c["k"], c["mode"])
    _check_rows(got_i, got_v, ref_i, ref_v, gap)
    # rows past act_q are untouched by the golden: -1 / 0
    for b in range(c["B"]):
        assert (idx[b, int(act_q[b]):] == -1).all() and (val[b, int(act_q[b]):] == 0).all()


def test_li_config1_is_positionally_exact():
    """Benchmark configuration 1 (seed 0): every row equals the reference golden slot for slot."""
    li = _li()
    q, k, w, act_q, act_k, c = li_case_inputs("li_config1")
    g = np.load(os.path.join(GOLDEN, "li_config1.npz"))
    idx, val = li.lightning_indexer_triton(dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(w),
                                           sparse_count=64, sparse_mode=3, return_value=True)
    same = (host(idx)[0] == g["idx_io"]).all(axis=(1, 2))
    assert same.mean() >= 0.99, f"{same.sum()} of 512 rows match"


def test_li_tnd_matches_oracle():
    li = _li()
    rng = np.random.RandomState(5)
    lens_q, lens_k = [37, 1, 64], [50, 9, 64]
    N1, N2, D, K = 16, 2, 128, 24
    from oracle.inputs import round_io
    q = round_io(rng.randn(sum(lens_q), N1, D).astype(np.float32), "bf16")
    k = round_io(rng.randn(sum(lens_k), N2, D).astype(np.float32), "bf16")
    w = (rng.randn(sum(lens_q), N1) / 4).astype(np.float32)
    cu_q, cu_k = np.cumsum(lens_q), np.cumsum(lens_k)
    ref_i, ref_v = layouts.li_oracle_tnd(q, k, w, cu_q, cu_k, sparse_count=K, sparse_mode=3, return_value=True)
    for lens_arg in ("list", "tensor"):
        aq = cu_q.tolist() if lens_arg == "list" else torch.tensor(cu_q, dtype=torch.int32).cuda()
        ak = cu_k.tolist() if lens_arg == "list" else torch.tensor(cu_k, dtype=torch.int32).cuda()
        idx, val = li.lightning_indexer_triton(
            dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(w), actual_seq_lengths_query=aq,
            actual_seq_lengths_key=ak, layout_query="TND", layout_key="TND", sparse_count=K,
            sparse_mode=3, return_value=True)
        assert idx.shape == (sum(lens_q), N2, K)
        li_reference_rule(host(idx), host(val), ref_i, ref_v)
        assert (host(idx) == ref_i).all(axis=(1, 2)).mean() >= 0.97


def test_li_paged_key_matches_unpaged_oracle():
    """PA_BSND keys (an extension: the reference raises): result == BSND run on the un-paged cache."""
    li = _li()
    rng = np.random.RandomState(6)
    B, S1, N1, D, K, bs = 3, 2, 16, 128, 40, 16
    lens_k = [100, 33, 64]
    max_blocks = 7
    nblk = 32
    from oracle.inputs import round_io
    cache = round_io(rng.randn(nblk, bs, 1, D).astype(np.float32), "bf16")
    q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), "bf16")
    w = (rng.randn(B, S1, N1) / 4).astype(np.float32)
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, dtype=np.int32)
    used = 0
    for b in range(B):
        need = -(-lens_k[b] // bs)
        bt[b, :need] = perm[used:used + need]
        used += need
    dense = layouts.pa_to_bsnd(cache, bt, max_blocks * bs)
    ref_i, ref_v = lightning_indexer_oracle(q, dense, w, [S1] * B, lens_k, sparse_count=K, sparse_mode=3,
                                            return_value=True)
    idx, val = li.lightning_indexer_triton(
        dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(w), actual_seq_lengths_key=lens_k,
        block_table=torch.from_numpy(bt).cuda(), layout_key="PA_BSND", sparse_count=K, sparse_mode=3,
        return_value=True)
    li_reference_rule(host(idx), host(val), ref_i, ref_v)
    assert (host(idx) == ref_i).all(axis=(2, 3)).mean() >= 0.97


@pytest.mark.parametrize("bs", [16, 64, 128, 256])
def test_li_paged_key_on_the_tensor_core_path(bs):
    """64 heads x 128 dims over a paged cache runs the tcgen05 kernel: a 128-key tile is 128/bs
    whole-block loads (or part of one block), rows come from the block table, and a block that is
    absent inside the valid length reads as zeros like the reference's un-paging."""
    li = _li()
    from dsa_triton_ascend_b200 import _cabi
    rng = np.random.RandomState(60 + bs)
    B, S1, N1, D, K = 3, 2, 64, 128, 256
    lens_k = [1500, 700, 2300]
    max_blocks = -(-max(lens_k) // bs) + 1
    need = [-(-L // bs) for L in lens_k]
    nblk = sum(need) + 5
    from oracle.inputs import round_io
    cache = round_io(rng.randn(nblk, bs, 1, D).astype(np.float32), "bf16")
    q = round_io(rng.randn(B, S1, N1, D).astype(np.float32), "bf16")
    w = (rng.randn(B, S1, N1) / 8).astype(np.float32)
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, dtype=np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
    bt[2, 3] = -1                       # a hole inside sequence 2
    dense = layouts.pa_to_bsnd(cache, bt, max_blocks * bs)
    ref_i, ref_v = lightning_indexer_oracle(q, dense, w, [S1] * B, lens_k, sparse_count=K, sparse_mode=3,
                                            return_value=True)
    args = (dev(q, torch.bfloat16), dev(cache, torch.bfloat16), dev(w))
    kw = dict(actual_seq_lengths_key=lens_k, block_table=torch.from_numpy(bt).cuda(), layout_key="PA_BSND",
              sparse_count=K, sparse_mode=3, return_value=True)
    li.set_kernel("tensor")
    try:
        idx, val = li.lightning_indexer_triton(*args, **kw)
    finally:
        li.set_kernel("auto")
    li_reference_rule(host(idx), host(val), ref_i, ref_v)
    assert (host(idx) == ref_i).mean() >= 0.99
    li.set_kernel("portable")
    try:
        idx_p, val_p = li.lightning_indexer_triton(*args, **kw)
    finally:
        li.set_kernel("auto")
    assert (host(idx) == host(idx_p)).mean() >= 0.99


def test_li_is_bitwise_repeatable_and_ordered():
    """No atomics on the data path: two runs agree bit for bit; values come out descending and
    the indices of a row are distinct, inside the causal window and front-packed."""
    li = _li()
    g = torch.Generator(device="cuda").manual_seed(2)
    S, N1, D, K = 2048, 64, 128, 512
    q = torch.randn(1, S, N1, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(1, S, 1, D, generator=g, device="cuda").bfloat16()
    w = torch.randn(1, S, N1, generator=g, device="cuda") / 8
    i1, v1 = li.lightning_indexer_triton(q, k, w, sparse_count=K, return_value=True)
    i2, v2 = li.lightning_indexer_triton(q, k, w, sparse_count=K, return_value=True)
    assert torch.equal(i1, i2) and torch.equal(v1, v2)
    idx, val = i1[0, :, 0], v1[0, :, 0].float()
    pos = torch.arange(S, device="cuda")[:, None]
    slot = torch.arange(K, device="cuda")[None, :]
    valid = slot < torch.clamp(pos + 1, max=K)
    assert torch.equal(idx >= 0, valid)
    assert bool(((idx <= pos) | ~valid).all())
    assert bool((val[:, :-1] >= val[:, 1:])[valid[:, 1:]].all())
    srt = torch.sort(torch.where(valid, idx, -1 - slot), dim=1).values
    assert bool((srt[:, 1:] != srt[:, :-1]).all())


def test_li_full_size_sampled_rows():
    """Configuration 3 shape (S=8192, 64 heads, k=2048): sampled rows against the oracle."""
    li = _li()
    g = torch.Generator(device="cuda").manual_seed(2)
    S, N1, D, K = 8192, 64, 128, 2048
    q = torch.randn(1, S, N1, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(1, S, 1, D, generator=g, device="cuda").bfloat16()
    w = torch.randn(1, S, N1, generator=g, device="cuda") / 8
    idx, val = li.lightning_indexer_triton(q, k, w, sparse_count=K, return_value=True)
    rows = [(0, s) for s in (0, 1, 2047, 2048, 2049, 4100, 6001, 8191)]
    qn, kn, wn = host(q), host(k), host(w)
    ref_i, ref_v = lightning_indexer_oracle(qn, kn, wn, [S], [S], sparse_count=K, sparse_mode=3,
                                            return_value=True, rows=rows)
    sel = np.asarray(rows)
    got_i, got_v = host(idx)[0, sel[:, 1]], host(val)[0, sel[:, 1]]
    gap = li_gap_ok(qn, kn, wn, [S], [S], rows, 1, K, 3)
    _check_rows(got_i, got_v, ref_i[0, sel[:, 1]], ref_v[0, sel[:, 1]], gap, min_positional=0.5)


def test_li_production_shape_runs_on_the_tensor_core_path():
    """64 heads x D=128 BSND goes through the tcgen05 kernel; it must agree with the portable
    CUDA-core kernel on every row and leave a clean device status word."""
    import ctypes
    from dsa_triton_ascend_b200 import _cabi
    li = _li()
    g = torch.Generator(device="cuda").manual_seed(9)
    B, S1, S2, K = 2, 300, 1000, 256
    q = torch.randn(B, S1, 64, 128, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, S2, 1, 128, generator=g, device="cuda").bfloat16()
    w = torch.randn(B, S1, 64, generator=g, device="cuda") / 8
    p, keep, idx, val, _ = li._build_params(q, k, w, [300, 77], [1000, 640], None, "BSND", "BSND", K, 3, True)
    assert _cabi.lib.dsa_li_uses_tensor_path(ctypes.byref(p)) == 1
    n = ctypes.c_size_t(0)
    _cabi.check(_cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(n)), "ws")
    ws = torch.empty(n.value, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.check(_cabi.lib.dsa_li_forward(ctypes.byref(p), ws.data_ptr(), ws.numel(), stream), "tensor")
    assert _cabi.lib.dsa_read_device_status(ws.data_ptr(), stream) == 0
    scores_t = ws[256:].view(torch.float32).clone()
    idx_t, val_t = idx.clone(), val.clone()
    p.kernel = _cabi.KERNEL_PORTABLE
    assert _cabi.lib.dsa_li_uses_tensor_path(ctypes.byref(p)) == 0
    _cabi.check(_cabi.lib.dsa_li_forward(ctypes.byref(p), ws.data_ptr(), ws.numel(), stream), "portable")
    torch.cuda.synchronize()
    scores_p = ws[256:].view(torch.float32)
    # compare the visible prefixes of the raw fp32 scores (the rest of the scratch is never written)
    ld = (S2 + 3) // 4 * 4
    st, sp = scores_t.view(-1)[:B * S1 * ld].view(B, S1, ld), scores_p.view(-1)[:B * S1 * ld].view(B, S1, ld)
    for b, (aq, ak) in enumerate([(300, 1000), (77, 640)]):
        for s in (0, 1, aq // 2, aq - 1):
            vis = min(max(ak - aq + s + 1, 0), ak)
            assert torch.allclose(st[b, s, :vis], sp[b, s, :vis], rtol=2e-5, atol=2e-5)
    same = (idx_t == idx).all(dim=-1).float().mean().item()
    assert same >= 0.97, f"tensor and portable paths agree on {same:.4f} of the rows"
    del keep


def test_li_tnd_production_shape_on_the_tensor_core_path():
    """TND query and key with 64 heads x D=128 run on the tcgen05 kernel (ragged sequences, lengths
    that are not multiples of the 8-row work items)."""
    import ctypes
    from dsa_triton_ascend_b200 import _cabi
    li = _li()
    rng = np.random.RandomState(15)
    lens_q, lens_k = [37, 1, 200, 64], [150, 9, 200, 300]
    K = 48
    from oracle.inputs import round_io
    q = round_io(rng.randn(sum(lens_q), 64, 128).astype(np.float32), "bf16")
    k = round_io(rng.randn(sum(lens_k), 1, 128).astype(np.float32), "bf16")
    w = (rng.randn(sum(lens_q), 64) / 8).astype(np.float32)
    cu_q, cu_k = np.cumsum(lens_q).tolist(), np.cumsum(lens_k).tolist()
    ref_i, ref_v = layouts.li_oracle_tnd(q, k, w, cu_q, cu_k, sparse_count=K, sparse_mode=3, return_value=True)
    qd, kd, wd = dev(q, torch.bfloat16), dev(k, torch.bfloat16), dev(w)
    p, keep, _, _, _ = li._build_params(qd, kd, wd, cu_q, cu_k, None, "TND", "TND", K, 3, True)
    assert _cabi.lib.dsa_li_uses_tensor_path(ctypes.byref(p)) == 1
    del keep
    idx, val = li.lightning_indexer_triton(qd, kd, wd, actual_seq_lengths_query=cu_q, actual_seq_lengths_key=cu_k,
                                           layout_query="TND", layout_key="TND", sparse_count=K, sparse_mode=3,
                                           return_value=True)
    li_reference_rule(host(idx), host(val), ref_i, ref_v)
    assert (host(idx) == ref_i).all(axis=(1, 2)).mean() >= 0.97


def test_li_full_mode_on_the_tensor_core_path():
    """sparse_mode=0 (no causal mask, only act_k) with the production head shape, fp16."""
    li = _li()
    from oracle.inputs import li_inputs
    B, S1, S2, K = 2, 40, 300, 64
    q, k, w = li_inputs(23, B, S1, S2, 64, 1, 128, "fp16", w_scale=0.125)
    act_q, act_k = [40, 17], [300, 129]
    ref_i, ref_v = lightning_indexer_oracle(q, k, w, act_q, act_k, sparse_count=K, sparse_mode=0,
                                            return_value=True, value_dtype="fp16")
    idx, val = li.lightning_indexer_triton(dev(q, torch.float16), dev(k, torch.float16), dev(w),
                                           actual_seq_lengths_query=act_q, actual_seq_lengths_key=act_k,
                                           sparse_count=K, sparse_mode=0, return_value=True)
    li_reference_rule(host(idx), host(val), ref_i, ref_v)
    assert (host(idx) == ref_i).all(axis=(2, 3)).mean() >= 0.97
