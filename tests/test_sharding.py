"""Host logic of the multi-GPU path: row slices are balanced, cover every row once, and a slice run
as a stand-alone problem reproduces the rows of the full problem (checked with the oracle, and
across two gloo ranks on CPU)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dsa_triton_ascend_b200.sharding import causal_work, row_slices, slice_lengths
from oracle import lightning_indexer_oracle, sparse_flash_attention_oracle
from oracle.inputs import li_inputs, sfa_inputs, sparse_indices


@pytest.mark.parametrize("act_q,act_k,world,cap", [(8192, 8192, 8, 0), (8192, 8192, 4, 2048), (1000, 4000, 3, 0),
                                                   (300, 100, 2, 0), (64, 64, 8, 16), (7, 7, 4, 0)])
def test_row_slices_cover_and_balance(act_q, act_k, world, cap):
    sl = row_slices(act_q, act_k, world, cap)
    assert len(sl) == world and sl[0][0] == 0 and sl[-1][1] == act_q
    assert all(a[1] == b[0] for a, b in zip(sl, sl[1:])) and all(a <= b for a, b in sl)
    work = [causal_work(act_q, act_k, a, b, cap) for a, b in sl]
    assert sum(work) == causal_work(act_q, act_k, 0, act_q, cap)
    if act_q >= 64 * world:
        assert max(work) <= 1.15 * sum(work) / world, work


def test_slice_is_a_standalone_problem_for_the_indexer():
    B, S1, S2, N1, D, K = 1, 96, 160, 8, 64, 24
    q, k, w = li_inputs(3, B, S1, S2, N1, 1, D, "bf16")
    aq, ak = [80], [150]
    full_i, full_v = lightning_indexer_oracle(q, k, w, aq, ak, sparse_count=K, sparse_mode=3, return_value=True)
    for r0, r1 in row_slices(aq[0], ak[0], 3):
        lq, lk = slice_lengths(aq[0], ak[0], r0, r1)
        i, v = lightning_indexer_oracle(q[:, r0:r1], k, w[:, r0:r1], [lq], [lk], sparse_count=K, sparse_mode=3,
                                        return_value=True)
        np.testing.assert_array_equal(i[:, :lq], full_i[:, r0:r1])
        np.testing.assert_array_equal(v[:, :lq], full_v[:, r0:r1])


def _rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, S1, S2, N1, D, K = 1, 40, 96, 8, 128, 16
        q, k, qr, kr = sfa_inputs(5, B, S1, S2, N1, D)
        idx = sparse_indices(6, B, S1, S2, K)
        scale = 1.0 / np.sqrt(D + 64.0)
        r0, r1 = row_slices(S1, S2, world)[rank]
        lq, lk = slice_lengths(S1, S2, r0, r1)
        out, smax, ssum = sparse_flash_attention_oracle(q[:, r0:r1], k, idx[:, r0:r1], qr[:, r0:r1], kr, scale,
                                                        [lq], [lk], sparse_mode=3, dtype="bf16")
        # every rank ends up with all rows: this gather is outside the hot path
        parts = [None] * world
        dist.all_gather_object(parts, (r0, r1, out, smax, ssum))
        if rank == 0:
            full = sparse_flash_attention_oracle(q, k, idx, qr, kr, scale, [S1], [S2], sparse_mode=3, dtype="bf16")
            got = np.concatenate([p[2] for p in sorted(parts, key=lambda p: p[0])], axis=1)
            got_m = np.concatenate([p[3] for p in sorted(parts, key=lambda p: p[0])], axis=2)
            np.testing.assert_array_equal(got, full[0])
            np.testing.assert_array_equal(got_m, full[1])
            open(os.path.join(tmp, "ok"), "w").write("ok")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_full_problem(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok").exists()


def test_sequence_shards_cover_and_balance():
    """Decode sharding: every sequence on exactly one rank, cached keys per rank nearly equal."""
    from dsa_triton_ascend_b200.sharding import sequence_shards
    rng = np.random.RandomState(4)
    lens = rng.randint(16384, 65537, size=64)
    for world in (1, 2, 4, 8):
        shards = sequence_shards(lens, world)
        assert sorted(b for s in shards for b in s) == list(range(64))
        loads = [int(lens[s].sum()) for s in shards]
        assert max(loads) - min(loads) <= 65536
        assert all(len(s) == 64 // world for s in shards) or world == 1 or max(loads) / min(loads) < 1.05
    assert sequence_shards([5, 1], 4) == [[0], [1], [], []]
    with pytest.raises(ValueError):
        sequence_shards([1], 0)


def _decode_rank_main(rank, world, port, tmp):
    """Decode: each rank runs indexer -> attention on its own sequences (its own paged cache in the
    real path; the un-paged equivalent here), nothing crosses ranks but the final gather."""
    from dsa_triton_ascend_b200.sharding import sequence_shards
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, S1, S2, N1, D, K = 5, 2, 160, 8, 128, 24
        rng = np.random.RandomState(17)
        lens = rng.randint(40, S2 + 1, size=B)
        iq, ik, iw = li_inputs(18, B, S1, S2, N1, 1, D)
        q, k, qr, kr = sfa_inputs(19, B, S1, S2, 8, 512)
        scale = 1.0 / 24.0

        def step(sel):
            lk = [int(lens[b]) for b in sel]
            idx, _ = lightning_indexer_oracle(iq[sel], ik[sel], iw[sel], [S1] * len(sel), lk, sparse_count=K,
                                              sparse_mode=3, return_value=True)
            out = sparse_flash_attention_oracle(q[sel], k[sel], idx, qr[sel], kr[sel], scale, [S1] * len(sel), lk,
                                                sparse_mode=3, dtype="bf16")
            return idx, out[0]

        mine = sequence_shards(lens, world)[rank]
        res = step(mine) if mine else None
        parts = [None] * world
        dist.all_gather_object(parts, (mine, res))
        if rank == 0:
            full_idx, full_out = step(list(range(B)))
            for sel, r in parts:
                for j, b in enumerate(sel):
                    np.testing.assert_array_equal(r[0][j], full_idx[b])
                    np.testing.assert_array_equal(r[1][j], full_out[b])
            assert sorted(b for sel, _ in parts for b in sel) == list(range(B))
            open(os.path.join(tmp, "ok_decode"), "w").write("ok")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_decode_their_own_sequences(tmp_path):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_decode_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok_decode").exists()


def test_tnd_token_slices_cover_balance_and_reproduce_the_full_problem():
    """Token ranges of a TND batch (the configuration-4 split): they cover every token once, are
    balanced by clipped causal work, and each range run as a stand-alone TND problem (its own
    cumulative lengths, the key rows it needs) reproduces the rows of the full problem."""
    from dsa_triton_ascend_b200.sharding import tnd_slice, tnd_token_slices
    from oracle import layouts
    lens = [8192, 4096, 2048, 1024]
    cum = np.cumsum(lens).tolist()
    for world in (2, 4, 8):
        sl = tnd_token_slices(cum, cum, world, cap=2048)
        assert sl[0][0] == 0 and sl[-1][1] == cum[-1] and all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
        work = []
        for t0, t1 in sl:
            cq, ck, ranges = tnd_slice(cum, cum, t0, t1)
            assert (cq[-1] if cq else 0) == t1 - t0 and len(cq) == len(ck) == len(ranges)
            tot, pq, pk = 0, 0, 0
            for a, b in zip(cq, ck):
                tot += causal_work(a - pq, b - pk, 0, a - pq, 2048)
                pq, pk = a, b
            work.append(tot)
        assert sum(work) == sum(causal_work(L, L, 0, L, 2048) for L in lens)
        assert max(work) <= 1.05 * sum(work) / world, work
    # a small batch through the oracle: slices that cut through sequences
    lens = [37, 12, 25]
    cum = np.cumsum(lens).tolist()
    T, N1, D, K = cum[-1], 8, 64, 8
    rng = np.random.RandomState(11)
    from oracle.inputs import round_io
    q = round_io(rng.randn(T, N1, D).astype(np.float32), "bf16")
    k = round_io(rng.randn(T, 1, D).astype(np.float32), "bf16")
    w = rng.randn(T, N1).astype(np.float32)
    full_i, full_v = layouts.li_oracle_tnd(q, k, w, cum, cum, sparse_count=K, sparse_mode=3, return_value=True)
    for t0, t1 in tnd_token_slices(cum, cum, 3, align=1):
        cq, ck, ranges = tnd_slice(cum, cum, t0, t1)
        ks = np.concatenate([k[a:b] for a, b in ranges], axis=0)
        i, v = layouts.li_oracle_tnd(q[t0:t1], ks, w[t0:t1], cq, ck, sparse_count=K, sparse_mode=3, return_value=True)
        np.testing.assert_array_equal(i, full_i[t0:t1])
        np.testing.assert_array_equal(v, full_v[t0:t1])
