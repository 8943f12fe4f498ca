"""Benchmark of the DSA forward hot path: lightning_indexer (score + top-k) feeding
sparse_flash_attention forward, at S=8K, topk=2048.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]

One step = one pass of the hot path over one synthetic batch:
  * indexer:   B=1, S1=S2=8192, 64 heads, D=128, bf16, fp32 weights, sparse_count=2048, mode 3
  * attention: TND, sequence lengths 8192/4096/2048/1024 (15360 tokens), 128 heads, D=512+64,
               bf16, top-k 2048 token-wise, mode 3, indices taken from an indexer run over the
               same token layout (done once, outside the timed region), softmax stats returned.
`value` is attention forward TFLOP/s of the whole job (valid query-key pairs x 128 heads x
2*(576+512) flop / the slowest rank's time); the indexer's query-tokens/s (score + top-k) is
reported beside it.  The inputs are the seeded tensors of dsa_triton_ascend_b200.synthetic
(numpy RandomState(2) / RandomState(3)).  With N GPUs the SAME problem is split (strong
scaling): indexer rows and attention tokens in contiguous ranges balanced by causal work, keys
replicated, no collective on the data path; the timed region is bracketed by a barrier and a
device synchronise, timed with CUDA events on the launch stream, max over ranks.  `e2e` repeats
the step through the public Python operators with pinned HOST buffers: host->device copies of
every input and device->host copies of every result are inside its timed region.

`--impl reference` times the CPU implementation of the same path (the numpy restatement of the
reference goldens under oracle/, run over all host cores) on a bounded sample of the same
workload and prints the same JSON line with "impl": "reference".
"""
import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "SFA-fwd TFLOP/s at S=8K, topk=2048 (LI+top-k query-tokens/s beside it)"
UNIT = "TFLOP/s"
SEQ_LENS = [8192, 4096, 2048, 1024]
TOPK = 2048
LI_S, LI_HEADS, LI_D = 8192, 64, 128
SFA_HEADS, SFA_D, SFA_DR = 128, 512, 64
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def sfa_flops(lens=SEQ_LENS, topk=TOPK, heads=SFA_HEADS, d=SFA_D, dr=SFA_DR):
    """2 flop per multiply-add over valid (token, key) pairs: QK^T over d+dr, PV over d."""
    pairs = sum(sum(min(topk, s + 1) for s in range(L)) for L in lens)
    return float(pairs) * heads * 2.0 * (d + dr + d), pairs


def li_flops(S=LI_S, heads=LI_HEADS, d=LI_D):
    pairs = S * (S + 1) // 2
    return float(pairs) * heads * 2.0 * d, pairs


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs (read-only
    NVML queries from a thread every few milliseconds; falls back to an `nvidia-smi -lms` child)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.sm, self.mask, self.max_mhz = index, [], 0, None
        self._stop, self._thread, self._proc = threading.Event(), None, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.mask |= int(get_reasons(h))
                    except Exception:
                        pass
                    time.sleep(0.008)
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            # the first queries of a process are the slow ones (milliseconds): have them done before
            # the caller enters its timed region, where a host stall of that size shows at small steps
            t_end = time.time() + 0.5
            while not self.sm and time.time() < t_end:
                time.sleep(0.002)
            return
        except Exception:
            self._thread = None
        try:
            q = "clocks.sm,clocks.max.sm"
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms",
                                           "50", "-i", str(self.index)], stdout=subprocess.PIPE,
                                          stderr=subprocess.DEVNULL, text=True)

            def read():
                for line in self._proc.stdout:
                    c = [x.strip() for x in line.split(",")]
                    try:
                        self.sm.append(float(c[0]))
                        self.max_mhz = float(c[1])
                    except (ValueError, IndexError):
                        pass
            threading.Thread(target=read, daemon=True).start()
        except OSError:
            self._proc = None

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self._proc is not None:
            self._proc.terminate()
        reasons = sorted(name for bit, name in self.REASONS.items() if self.mask & bit)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(index):
    """Restrict this process to the CPUs NVML reports as local to GPU `index` (a read-only query),
    so that pinned host buffers land on that GPU's NUMA node.  Returns the CPU count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cpus = [w * 64 + b for w, m in enumerate(words) for b in range(64) if (int(m) >> b) & 1]
        cpus = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def pct(xs):
    xs = np.asarray(xs, np.float64)
    return {"mean": float(xs.mean()), "median": float(np.median(xs)), "p20": float(np.percentile(xs, 20)),
            "p80": float(np.percentile(xs, 80))}


def training_side(torch, flush, iters=3):
    """The three backward operators of the path at the shapes the reference's perf scripts time
    (perf_sfa_grad_triton.py:23, perf_sli_grad_kl_loss_triton.py:97, perf_dense_loss_backward_triton.py:18),
    seeded normal inputs x 0.3, causal random indices.  CUDA-core kernels: reported beside the
    headline numbers, median of `iters` calls, algorithmic flops = 2 x multiply-adds of the
    contractions over the valid (row, key) pairs."""
    from dsa_triton_ascend_b200 import (dense_lightning_indexer_softmax_lse_triton, dense_loss_backward_triton,
                                        sparse_flash_attention_grad_triton, sparse_flash_attention_triton,
                                        sparse_lightning_indexer_grad_kl_loss_triton)
    g = torch.Generator(device="cuda").manual_seed(77)
    bf = torch.bfloat16

    def rnd(*shape):
        return (torch.randn(*shape, generator=g, device="cuda") * 0.3).to(bf)

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        ts = []
        for i in range(iters):
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts))

    out = {}
    # attention backward: B, S1, S2, N1, top-k = 1, 512, 4096, 64, 2048 (D 512 + 64)
    S1, S2, N1, K, D, Dr = 512, 4096, 64, 2048, 512, 64
    q, k, qr, kr, do = rnd(1, S1, N1, D), rnd(1, S2, 1, D), rnd(1, S1, N1, Dr), rnd(1, S2, 1, Dr), rnd(1, S1, N1, D)
    idx = torch.full((S1, K), -1, dtype=torch.int32, device="cuda")
    vis = S2 - S1 + torch.arange(S1, device="cuda") + 1
    idx[:] = torch.arange(K, device="cuda", dtype=torch.int32)[None, :]      # the first K visible keys of a row
    idx = idx.masked_fill(torch.arange(K, device="cuda")[None, :] >= vis[:, None], -1).view(1, S1, 1, K)
    pairs = int((idx >= 0).sum())
    sc = 1.0 / float(np.sqrt(D + Dr))
    o, mx, sm = sparse_flash_attention_triton(q, k, k, idx, scale_value=sc, query_rope=qr, key_rope=kr, sparse_mode=3,
                                              return_softmax_lse=True)
    ms = timed(lambda: sparse_flash_attention_grad_triton(q, k, k, idx, do, o, mx, sm, scale_value=sc, query_rope=qr,
                                                          key_rope=kr, sparse_mode=3))
    fl = pairs * N1 * 2 * ((D + Dr) * 3 + D * 2)
    out["sfa_grad"] = {"shape": "B1 S1 512 S2 4096 N1 64 k 2048 D 512+64", "ms": ms, "tflops": fl / ms / 1e9}
    # sparse indexer KL-loss backward: 1, 512, 4096, 64, 512, 64, 128, 2048
    G, Di = 64, 128
    qi, ki, w = rnd(1, S1, G, Di), rnd(1, S2, 1, Di), rnd(1, S1, G).abs()
    idx_c = idx.clamp_min(0)
    ms = timed(lambda: sparse_lightning_indexer_grad_kl_loss_triton(q, k, qi, ki, w, idx_c, mx, sm, query_rope=qr,
                                                                    key_rope=kr, scale_value=sc))
    fl = pairs * 2 * (N1 * (D + Dr) + G * Di * 4)
    out["sli_grad_kl_loss"] = {"shape": "B1 S1 512 S2 4096 N1 64 D 512+64 G 64 Di 128 k 2048", "ms": ms,
                               "tflops": fl / ms / 1e9}
    # dense indexer loss backward: 1, 512, 4096, 64, 64, 128, 64, 128 (MHA keys)
    N2, D2 = 64, 128
    q2, k2, qr2, kr2 = rnd(1, S1, N1, D2), rnd(1, S2, N2, D2), rnd(1, S1, N1, Dr), rnd(1, S2, N2, Dr)
    mx2 = torch.zeros(1, N2, S1, 1, device="cuda")
    sm2 = torch.full((1, N2, S1, 1), float(S2), device="cuda")
    lse = dense_lightning_indexer_softmax_lse_triton(qi, ki, w)
    ms_lse = timed(lambda: dense_lightning_indexer_softmax_lse_triton(qi, ki, w))
    ms = timed(lambda: dense_loss_backward_triton(q2, k2, qi, ki, w, mx2, sm2, lse[0], lse[1], 1.0 / float(np.sqrt(D2 + Dr)),
                                                  query_rope=qr2, key_rope=kr2))
    dpairs = int(vis.sum())
    fl = dpairs * 2 * (N1 * (D2 + Dr) + G * Di * 4)
    out["dense_loss_backward"] = {"shape": "B1 S1 512 S2 4096 N1 64 N2 64 D 128+64 G 64 Di 128", "ms": ms,
                                  "tflops": fl / ms / 1e9, "softmax_lse_ms": ms_lse}
    return out


def decode_c5(torch, rank, world, flush, iters=5):
    """Configuration 5 (decode): lightning_indexer then sparse_flash_attention over paged caches,
    B=64 sequences dealt out over the ranks by cached length (sharding.sequence_shards), S1=2, KV
    lengths uniform in [16384, 65536] from RandomState(4), block 128.  Reported beside the headline
    numbers; the indexer here is bound by reading the index-K cache."""
    from dsa_triton_ascend_b200 import lightning_indexer_triton, sparse_flash_attention_triton
    from dsa_triton_ascend_b200.sharding import sequence_shards
    S1, bs, K = 2, 128, TOPK
    all_lens = np.random.RandomState(4).randint(16384, 65537, size=64)
    mine = sequence_shards(all_lens.tolist(), world)[rank]
    lens = all_lens[mine]
    B = len(mine)
    rng = np.random.RandomState(4000 + rank)
    need = [int(-(-L // bs)) for L in lens]
    nblk, max_blocks = sum(need), max(need)
    perm = rng.permutation(nblk)
    bt = np.full((B, max_blocks), -1, np.int32)
    used = 0
    for b in range(B):
        bt[b, :need[b]] = perm[used:used + need[b]]
        used += need[b]
    g = torch.Generator(device="cuda").manual_seed(4000 + rank)
    bf = torch.bfloat16

    def randn_bf16(*shape):
        out = torch.empty(shape, dtype=bf, device="cuda")
        step = max(1, (1 << 26) // int(np.prod(shape[1:])))
        for i in range(0, shape[0], step):
            out[i:i + step] = torch.randn((min(step, shape[0] - i),) + tuple(shape[1:]), generator=g, device="cuda")
        return out

    ik, kv, kr = randn_bf16(nblk, bs, 1, LI_D), randn_bf16(nblk, bs, 1, SFA_D), randn_bf16(nblk, bs, 1, SFA_DR)
    iq, iw = randn_bf16(B, S1, LI_HEADS, LI_D), torch.randn(B, S1, LI_HEADS, generator=g, device="cuda") / 8
    q, qr = randn_bf16(B, S1, SFA_HEADS, SFA_D), randn_bf16(B, S1, SFA_HEADS, SFA_DR)
    table = torch.from_numpy(bt).cuda()
    lens_l = [int(v) for v in lens]
    scale = 1.0 / np.sqrt(SFA_D + SFA_DR)

    def li():
        return lightning_indexer_triton(iq, ik, iw, actual_seq_lengths_key=lens_l, block_table=table,
                                        layout_key="PA_BSND", sparse_count=K, sparse_mode=3)[0]

    def sfa(idx):
        return sparse_flash_attention_triton(q, kv, kv, idx, scale_value=scale, block_table=table,
                                             actual_seq_lengths_kv=lens_l, query_rope=qr, key_rope=kr,
                                             layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
                                             block_size=bs)

    idx = li()
    sfa(idx)
    torch.cuda.synchronize()
    t_li, t_sfa = [], []
    for i in range(iters):
        flush.fill_(i & 0xFF)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        idx = li()
        e[1].record()
        sfa(idx)
        e[2].record()
        torch.cuda.synchronize()
        t_li.append(e[0].elapsed_time(e[1]))
        t_sfa.append(e[1].elapsed_time(e[2]))
    li_ms, sfa_ms = float(np.median(t_li)), float(np.median(t_sfa))
    # the same step captured once in a CUDA graph (lengths in a device tensor) and replayed
    lens_t = torch.tensor(lens_l, dtype=torch.int32, device="cuda")

    def step_dev():
        i_ = lightning_indexer_triton(iq, ik, iw, actual_seq_lengths_key=lens_t, block_table=table,
                                      layout_key="PA_BSND", sparse_count=K, sparse_mode=3)[0]
        return sparse_flash_attention_triton(q, kv, kv, i_, scale_value=scale, block_table=table,
                                             actual_seq_lengths_kv=lens_t, query_rope=qr, key_rope=kr,
                                             layout_kv="PA_BSND", sparse_mode=3, return_softmax_lse=True,
                                             block_size=bs)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step_dev()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step_dev()
    torch.cuda.current_stream().wait_stream(side)
    t_g = []
    for i in range(iters):
        flush.fill_(i & 0xFF)
        e = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        e[0].record()
        graph.replay()
        e[1].record()
        torch.cuda.synchronize()
        t_g.append(e[0].elapsed_time(e[1]))
    graph_ms = float(np.median(t_g))
    ik_bytes = float(sum(lens_l)) * LI_D * 2                     # index-K rows the indexer must read
    gathered = float(B * S1 * K) * (SFA_D + SFA_DR) * 2          # KV rows the attention gathers
    return {"workload": "64 sequences over %d rank(s) (%d here), S1=2, L~U[16384,65536] paged block 128, "
                        "LI 64x128 -> top-%d -> SFA 128x(512+64)" % (world, B, K),
            "li_ms": li_ms, "sfa_ms": sfa_ms, "step_ms": li_ms + sfa_ms, "graph_replay_step_ms": graph_ms,
            "li_index_k_GBps": ik_bytes / (li_ms * 1e-3) / 1e9, "sfa_gather_GBps": gathered / (sfa_ms * 1e-3) / 1e9}


def run_gpu(args):
    import ctypes
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    numa_cpus = bind_to_gpu_numa_node(local)          # before any pinned allocation
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from dsa_triton_ascend_b200 import _cabi, lightning_indexer_triton, sparse_flash_attention_triton, synthetic
    from dsa_triton_ascend_b200.sharding import (row_slices, slice_lengths, tnd_slice, tnd_token_slices)
    import dsa_triton_ascend_b200.lightning_indexer as li_mod

    # ---- the seeded problem (host), this rank's share of it (device)
    c3 = synthetic.config3(None, args.scale)
    c4 = synthetic.config4(None, args.scale, args.lens)
    S, topk = c3["S"], c3["sparse_count"]
    lens, cum, T = c4["lens"], c4["cum"], c4["T"]
    scale = c4["scale"]
    flops_sfa, _ = sfa_flops(lens, topk)
    flops_li, _ = li_flops(S)
    r0, r1 = row_slices(S, S, world)[rank]                                   # indexer rows of this rank
    t0, t1 = tnd_token_slices(cum, cum, world, cap=topk)[rank]               # attention tokens of this rank
    cq, ck, kranges = tnd_slice(cum, cum, t0, t1)
    my_li_pairs = sum(s + 1 for s in range(r0, r1))
    my_sfa_pairs = 0
    pq = 0
    for cqe, L in zip(cum, lens):
        for t in range(max(t0, pq), min(t1, cqe)):
            my_sfa_pairs += min(topk, t - pq + 1)
        pq = cqe
    dev = lambda x: x.cuda(non_blocking=False)
    cat = lambda t: torch.cat([t[a:b] for a, b in kranges], dim=0) if len(kranges) != 1 else t[kranges[0][0]:kranges[0][1]]
    li_lq, li_lk = slice_lengths(S, S, r0, r1)
    b = {"li_q": dev(c3["q"][:, r0:r1]), "li_k": dev(c3["k"]), "li_w": dev(c3["w"][:, r0:r1]),
         "q": dev(c4["q"][t0:t1]), "qr": dev(c4["qr"][t0:t1]), "k": dev(cat(c4["k"])), "kr": dev(cat(c4["kr"]))}
    # the attention's indices come from the indexer over the same tokens (once, outside the timed region)
    idx, _ = lightning_indexer_triton(dev(c4["qi"][t0:t1]), dev(cat(c4["ki"])), dev(c4["wi"][t0:t1]),
                                      actual_seq_lengths_query=cq, actual_seq_lengths_key=ck, layout_query="TND",
                                      layout_key="TND", sparse_count=topk, sparse_mode=3,
                                      max_seqlen_key=max(lens))
    b["idx"] = idx.contiguous()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def li_step():
        return lightning_indexer_triton(b["li_q"], b["li_k"], b["li_w"], actual_seq_lengths_query=[li_lq],
                                        actual_seq_lengths_key=[li_lk], sparse_count=topk, sparse_mode=3)

    def sfa_step():
        return sparse_flash_attention_triton(
            b["q"], b["k"], b["k"], b["idx"], scale_value=scale, actual_seq_lengths_query=cq,
            actual_seq_lengths_kv=ck, query_rope=b["qr"], key_rope=b["kr"], layout_query="TND", layout_kv="TND",
            sparse_mode=3, return_softmax_lse=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        li_out = li_step()
        sfa_out = sfa_step()
    barrier()

    sampler = ClockSampler(local)
    sampler.start()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    launches0 = int(_cabi.lib.dsa_kernel_launch_count())
    # no collector pauses on the host while steps of about a millisecond are being enqueued (N = 8)
    gc.collect()
    gc.disable()
    t_wall = time.perf_counter()
    for s in range(args.steps):
        flush.fill_(s & 0xFF)  # evict L2 between timed iterations
        ev[s][0].record()
        li_out = li_step()
        ev[s][1].record()
        sfa_out = sfa_step()
        ev[s][2].record()
    barrier()
    t_wall = time.perf_counter() - t_wall
    gc.enable()
    launches = int(_cabi.lib.dsa_kernel_launch_count()) - launches0
    clocks = sampler.stop()
    li_all = [e[0].elapsed_time(e[1]) for e in ev]
    sfa_all = [e[1].elapsed_time(e[2]) for e in ev]
    li_ms, sfa_ms = float(np.mean(li_all)), float(np.mean(sfa_all))
    from dsa_triton_ascend_b200 import check_status
    check_status()

    # score / top-k split of the indexer (same inputs, phases launched separately)
    p, keep, _, _, _ = li_mod._build_params(b["li_q"], b["li_k"], b["li_w"], [li_lq], [li_lk], None,
                                            "BSND", "BSND", topk, 3, False)
    nbytes = ctypes.c_size_t(0)
    _cabi.check(_cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)), "li")
    ws = torch.empty(nbytes.value, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    tensor_li = bool(_cabi.lib.dsa_li_uses_tensor_path(ctypes.byref(p)))
    phase_ms = {}
    for name, ph in (("score", _cabi.PHASE_SCORE), ("topk", _cabi.PHASE_TOPK)):
        p.phases = ph
        times = []
        for i in range(args.warmup + args.steps):
            flush.fill_(i & 0xFF)
            a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            _cabi.check(_cabi.lib.dsa_li_forward(ctypes.byref(p), ws.data_ptr(), ws.numel(), stream), "li")
            b_.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(a.elapsed_time(b_))
        phase_ms[name] = float(np.mean(times))
    del keep, ws

    # ---- end to end through the public operators with pinned HOST buffers.  Rows are independent,
    # so the step is run as a pipeline over row chunks: chunk i+1 is uploaded and chunk i-1 is
    # downloaded (separate copy streams, PCIe is full duplex) while chunk i computes.  The small
    # key tensors are uploaded once per step; every byte of input and output crosses PCIe inside
    # the timed region.
    host_in = {k_: v.cpu().pin_memory() for k_, v in b.items()}
    n_tok, n_row = t1 - t0, r1 - r0
    out_h = torch.empty((n_tok, SFA_HEADS, SFA_D), dtype=torch.bfloat16).pin_memory()
    st_h = torch.empty((2, n_tok, SFA_HEADS), dtype=torch.float32).pin_memory()
    idx_h = torch.empty((n_row, 1, topk), dtype=torch.int32).pin_memory()
    h2d = sum(host_in[k_].numel() * host_in[k_].element_size() for k_ in host_in)
    d2h = out_h.numel() * 2 + st_h.numel() * 4 + idx_h.numel() * 4
    chunk = max(256, 1024 // args.scale)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    comp = torch.cuda.current_stream()
    # this rank's attention tokens as (local token range, sequence key range, row range in the sequence, lengths)
    pieces, pq, pk, loc = [], 0, 0, 0
    for cqe, cke in zip(cq, ck):
        Lq, Lk = cqe - pq, cke - pk
        for a0 in range(0, Lq, chunk):
            a1 = min(Lq, a0 + chunk)
            pieces.append((loc + a0, loc + a1, pk, cke) + slice_lengths(Lq, Lk, a0, a1))
        loc += Lq
        pq, pk = cqe, cke

    def upload(t, keep):
        with torch.cuda.stream(s_in):
            d = t.cuda(non_blocking=True)
        d.record_stream(comp)
        keep.append(d)
        return d

    def e2e_step():
        keep = []
        # indexer: key + per-chunk query rows / weights in, indices out
        lik = upload(host_in["li_k"], keep)
        k_d, kr_d = upload(host_in["k"], keep), upload(host_in["kr"], keep)
        for a0 in range(0, n_row, 2 * chunk):
            a1 = min(n_row, a0 + 2 * chunk)
            q_c = upload(host_in["li_q"][:, a0:a1], keep)
            w_c = upload(host_in["li_w"][:, a0:a1], keep)
            e_ = torch.cuda.Event()
            e_.record(s_in)
            comp.wait_event(e_)
            lq, lk = slice_lengths(li_lq, li_lk, a0, a1)
            i_c, _ = lightning_indexer_triton(q_c, lik, w_c, actual_seq_lengths_query=[lq],
                                              actual_seq_lengths_key=[lk], sparse_count=topk, sparse_mode=3)
            e2 = torch.cuda.Event()
            e2.record(comp)
            s_out.wait_event(e2)
            with torch.cuda.stream(s_out):
                idx_h[a0:a1].copy_(i_c[0], non_blocking=True)
            i_c.record_stream(s_out)
        # attention: one sequence at a time, rows in chunks
        for (l0, l1, k0, k1, lq, lk) in pieces:
            sl = slice(l0, l1)
            q_c, qr_c = upload(host_in["q"][sl], keep), upload(host_in["qr"][sl], keep)
            i_c = upload(host_in["idx"][sl], keep)
            e_ = torch.cuda.Event()
            e_.record(s_in)
            comp.wait_event(e_)
            o, m, s_ = sparse_flash_attention_triton(
                q_c[None], k_d[k0:k1][None], None, i_c[None], scale_value=scale,
                actual_seq_lengths_query=[lq], actual_seq_lengths_kv=[lk], query_rope=qr_c[None],
                key_rope=kr_d[k0:k1][None], sparse_mode=3, return_softmax_lse=True)
            e2 = torch.cuda.Event()
            e2.record(comp)
            s_out.wait_event(e2)
            with torch.cuda.stream(s_out):
                out_h[sl].copy_(o[0], non_blocking=True)
                st_h[0, sl].copy_(m[0, 0], non_blocking=True)
                st_h[1, sl].copy_(s_[0, 0], non_blocking=True)
            for t_ in (o, m, s_):
                t_.record_stream(s_out)
        comp.wait_stream(s_out)
        comp.wait_stream(s_in)

    e2e_steps = max(1, min(args.steps, 5))
    if args.no_e2e:
        e2e_ms = 1e30
    else:
        e2e_step()
        barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(e2e_steps):
            e2e_step()
        b_.record()
        barrier()
        e2e_ms = a.elapsed_time(b_) / e2e_steps

    def gather(x):
        if world == 1:
            return [float(x)]
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        allr = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allr, t)
        return [float(v.item()) for v in allr]

    # per-rank device times, work shares and clocks (the headline uses the slowest rank)
    per_rank = {"li_ms": gather(li_ms), "sfa_ms": gather(sfa_ms), "e2e_ms": gather(e2e_ms),
                "sfa_pairs": gather(my_sfa_pairs), "li_pairs": gather(my_li_pairs),
                "h2d_GBps": gather((h2d) / (e2e_ms * 1e-3) / 1e9), "d2h_GBps": gather(d2h / (e2e_ms * 1e-3) / 1e9),
                "sm_mhz": gather(float(clocks.get("sm_mhz") or 0.0)),
                "throttle_reasons": gather(float(len(clocks.get("reasons") or []))),
                "numa_cpus": gather(float(numa_cpus or 0))}
    h2d_tot, d2h_tot = sum(gather(h2d)), sum(gather(d2h))
    launches_tot = int(sum(gather(launches)))
    li_max, sfa_max, e2e_max = max(per_rank["li_ms"]), max(per_rank["sfa_ms"]), max(per_rank["e2e_ms"])
    step_max = max(x + y for x, y in zip(per_rank["li_ms"], per_rank["sfa_ms"]))
    pk = peaks()
    sfa_tf = flops_sfa / (sfa_max * 1e-3) / 1e12                  # whole job
    sfa_tf_gpu = (my_sfa_pairs * SFA_HEADS * 2.0 * (2 * SFA_D + SFA_DR)) / (sfa_ms * 1e-3) / 1e12   # this GPU's kernel
    li_score_tf = (my_li_pairs * LI_HEADS * 2.0 * LI_D) / (phase_ms["score"] * 1e-3) / 1e12
    topk_bytes = float(my_li_pairs) * 4.0 + float(n_row) * topk * 4.0
    workload = "LI B=1 S=%d N1=64 D=128 k=%d + SFA TND lens=%s N1=128 D=512+64 topk=%d, mode 3" % (S, topk, lens, topk)
    line = {
        "metric": METRIC, "value": sfa_tf, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_max, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "quick": bool(args.quick)},
        "l2": "256 MiB buffer written between timed iterations; inputs (q 1.9 GiB at one GPU) exceed L2",
        "inputs": "dsa_triton_ascend_b200.synthetic: numpy RandomState(2) indexer / RandomState(3) attention, "
                  "bf16; N GPUs split the same problem by causal work, keys replicated",
        "li_topk_qtok_per_s": S / (li_max * 1e-3),
        "li_ms": li_max, "li_score_ms": phase_ms["score"], "li_topk_ms": phase_ms["topk"],
        "li_topk_share": phase_ms["topk"] / (phase_ms["score"] + phase_ms["topk"]),
        "li_score_tflops": li_score_tf,
        "sfa_ms": sfa_max, "sfa_tflops_per_gpu": sfa_tf_gpu,
        "timing": {"sfa_ms": pct(sfa_all), "li_ms": pct(li_all), "sfa_ms_steps": [round(x, 3) for x in sfa_all],
                   "note": "this rank's steps; value uses the mean"},
        "shard_imbalance": {"sfa_max_over_mean": sfa_max / float(np.mean(per_rank["sfa_ms"])),
                            "li_max_over_mean": li_max / float(np.mean(per_rank["li_ms"]))},
        "li_tensor_path": tensor_li,
        "roofline": {"bound": "tensor", "achieved": sfa_tf_gpu, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": sfa_tf_gpu / pk["bf16_tflops"],
                     # dram read + write of sfa_fwd_sm100_kernel per launch: q + out dominate and grow with
                     # the token count; ncu capture of a 3840-token case (1.0435 GB) scaled by tokens
                     "traffic": 1.0435e9 * n_tok / 3840.0, "kernel": "sfa_fwd_sm100_kernel",
                     "peak_source": pk["source"] + " (burst bf16 GEMM)",
                     "frac_of_sustained": sfa_tf_gpu / pk["bf16_tflops_sustained"]},
        "roofline_li_score": {"bound": "tensor", "achieved": li_score_tf, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                              "frac": li_score_tf / pk["bf16_tflops"]},
        # top-k: reads every visible fp32 score once, writes k int32 indices per row
        "roofline_li_topk": {"bound": "hbm", "achieved": topk_bytes / (phase_ms["topk"] * 1e-3) / 1e9,
                             "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": topk_bytes / (phase_ms["topk"] * 1e-3) / 1e9 / pk["hbm_gbs"],
                             "note": "instruction-bound (ordered selection), not memory-bound"},
        "e2e": {"value": flops_sfa / (e2e_max * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_max,
                "h2d_bytes_per_step": int(h2d_tot), "d2h_bytes_per_step": int(d2h_tot),
                "li_topk_qtok_per_s": S / (e2e_max * 1e-3)},
        "gpu_launches": launches_tot,
        "clocks": clocks, "wall_s": t_wall,
    }
    if args.no_e2e:
        line["e2e"] = None
        per_rank.pop("e2e_ms")
    if world > 1:
        line["per_rank"] = per_rank
    else:
        line["host_GBps"] = {"h2d": per_rank["h2d_GBps"][0], "d2h": per_rank["d2h_GBps"][0], "numa_cpus": numa_cpus}
    if rank == 0 and not args.no_cpu:
        # the CPU leg also checks rows of the TIMED outputs of this rank against the oracle
        line["verified_rows"] = verify_rows(torch, c3, c4, r0, r1, t0, t1, li_out, sfa_out, b["idx"], topk)
        if world == 1:
            line["cpu_baseline"] = cpu_reference(sample_s=args.cpu_seconds, procs=1, lens=lens, topk=topk)
    if args.scale == 1 and not args.quick and not args.no_decode:
        del host_in, out_h
        dec = decode_c5(torch, rank, world, flush)
        steps = gather(dec["step_ms"])
        graphs = gather(dec["graph_replay_step_ms"])
        dec["step_ms"], dec["graph_replay_step_ms"] = max(steps), max(graphs)
        dec["tokens_per_s"] = 64 * 2 / (max(steps) * 1e-3)
        dec["per_rank_step_ms"] = steps
        dec["roofline_li"] = {"bound": "hbm", "achieved": dec["li_index_k_GBps"], "peak": pk["hbm_gbs"],
                              "unit": "GB/s", "frac": dec["li_index_k_GBps"] / pk["hbm_gbs"],
                              "note": "this rank's index-K cache bytes / indexer time (score + top-k)"}
        line["decode_c5"] = dec
    if rank == 0 and args.scale == 1 and not args.quick and not args.no_training:
        line["training_side"] = training_side(torch, flush)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def verify_rows(torch, c3, c4, r0, r1, t0, t1, li_out, sfa_out, idx_dev, topk):
    """Part of the CPU leg: a few rows of the outputs the timed region produced, against the oracle
    (reference rule for the indexer, atol = rtol = 2e-2 / 1e-3 for the attention).  Returns the
    number of rows checked; raises on a mismatch."""
    from oracle import lightning_indexer_oracle, sparse_flash_attention_oracle
    from oracle.compare import li_reference_rule, sfa_acceptance_rule
    f32 = lambda t: t.detach().float().cpu().numpy()
    S = c3["S"]
    n = 0
    rows = sorted(set(int(x) for x in np.linspace(r0, r1 - 1, 3)))
    ri, _ = lightning_indexer_oracle(f32(c3["q"]), f32(c3["k"]), f32(c3["w"]), [S], [S], sparse_count=topk,
                                     sparse_mode=3, return_value=False, rows=[(0, s) for s in rows])
    got = li_out[0].detach().cpu().numpy()
    for s in rows:
        a_, b_ = got[0, s - r0, 0], ri[0, s, 0]
        assert ((a_ >= 0) == (b_ >= 0)).all() and (a_ == b_).mean() >= 0.97, "indexer row %d differs from the oracle" % s
        n += 1
    cum, lens = c4["cum"], c4["lens"]
    out, smax, ssum = sfa_out
    idx_h = idx_dev.detach().cpu().numpy()
    for t in sorted(set(int(x) for x in np.linspace(t0, t1 - 1, 3))):
        bseq = int(np.searchsorted(cum, t, side="right"))
        s0 = 0 if bseq == 0 else int(cum[bseq - 1])
        s, L = t - s0, lens[bseq]
        qq = np.zeros((1, L, SFA_HEADS, SFA_D), np.float32)
        qq[0, s] = f32(c4["q"][t])
        qqr = np.zeros((1, L, SFA_HEADS, SFA_DR), np.float32)
        qqr[0, s] = f32(c4["qr"][t])
        ii = np.full((1, L, 1, topk), -1, np.int32)
        ii[0, s] = idx_h[t - t0]
        ref = sparse_flash_attention_oracle(qq, f32(c4["k"][s0:s0 + L])[None], ii, qqr, f32(c4["kr"][s0:s0 + L])[None],
                                            c4["scale"], [L], [L], sparse_mode=3, dtype="bf16", rows=[(0, s)])
        sfa_acceptance_rule(f32(out[t - t0]), f32(smax[0, t - t0]), f32(ssum[0, t - t0]), ref[0][0, s], ref[1][0, 0, s],
                            ref[2][0, 0, s])
        n += 1
    return n


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle (numpy restatement of the reference goldens) on a bounded sample
# ----------------------------------------------------------------------------------------------
def _one_blas_thread():
    try:
        from threadpoolctl import threadpool_limits
        return threadpool_limits(limits=1)
    except Exception:  # pragma: no cover
        import contextlib
        return contextlib.nullcontext()


def _cpu_sfa_rows(args):
    """Oracle attention for query tokens at positions `tokens` of one L-token sequence.  Each token
    is one oracle call with S1=1, act_q=1, act_k=pos+1, which gives the causal threshold pos+1."""
    seed, tokens, L, topk = args
    from oracle import sparse_flash_attention_oracle
    from oracle.inputs import round_io
    rng = np.random.RandomState(seed)
    k = round_io(rng.randn(1, L, 1, SFA_D).astype(np.float32), "bf16")
    kr = round_io(rng.randn(1, L, 1, SFA_DR).astype(np.float32), "bf16")
    work = []
    for s in tokens:
        q = round_io(rng.randn(1, 1, SFA_HEADS, SFA_D).astype(np.float32), "bf16")
        qr = round_io(rng.randn(1, 1, SFA_HEADS, SFA_DR).astype(np.float32), "bf16")
        n = min(topk, s + 1)
        idx = np.full((1, 1, 1, topk), -1, np.int32)
        idx[0, 0, 0, :n] = np.sort(rng.choice(s + 1, n, replace=False))
        work.append((s, q, qr, idx, n))
    pairs = 0
    with _one_blas_thread():
        t = time.perf_counter()
        for s, q, qr, idx, n in work:
            sparse_flash_attention_oracle(q, k, idx, qr, kr, 1.0 / np.sqrt(576.0), [1], [s + 1], sparse_mode=3,
                                          dtype="bf16")
            pairs += n
        t = time.perf_counter() - t
    return t, pairs


def _cpu_li_rows(args):
    """Oracle indexer (score, mask, round, rank) for query rows at positions `rows` (one call per row
    with S1=1, act_q=1, act_k=pos+1)."""
    seed, rows, S, topk = args
    from oracle import lightning_indexer_oracle
    from oracle.inputs import round_io
    rng = np.random.RandomState(seed)
    k = round_io(rng.randn(1, S, 1, LI_D).astype(np.float32), "bf16")
    work = []
    for s in rows:
        q = round_io(rng.randn(1, 1, LI_HEADS, LI_D).astype(np.float32), "bf16")
        w = (rng.randn(1, 1, LI_HEADS) / 8).astype(np.float32)
        work.append((s, q, w))
    with _one_blas_thread():
        t = time.perf_counter()
        for s, q, w in work:
            lightning_indexer_oracle(q, k, w, [1], [s + 1], sparse_count=topk, sparse_mode=3)
        t = time.perf_counter() - t
    return t, sum(s + 1 for s in rows)


def cpu_reference(sample_s=12.0, procs=None, lens=SEQ_LENS, topk=TOPK):
    """Times the CPU implementation on evenly spaced rows of the same workload and scales by the
    work measure (valid query-key pairs).  `procs` worker processes, one BLAS thread each."""
    import multiprocessing as mp
    procs = procs or len(os.sched_getaffinity(0))
    L = lens[0]
    # a short calibration decides how many rows fit the time limit
    t0, p0 = _cpu_sfa_rows((11, [L - 1], L, topk))
    n_sfa = max(procs, int(sample_s * 0.7 / max(t0, 1e-3)) * procs)
    tok = np.unique(np.linspace(0, L - 1, n_sfa).astype(int)).tolist()
    t1, p1 = _cpu_li_rows((12, [L - 1], L, topk))
    n_li = max(procs, int(sample_s * 0.3 / max(t1, 1e-3)) * procs)
    rows = np.unique(np.linspace(0, L - 1, n_li).astype(int)).tolist()
    ctx = mp.get_context("fork")
    t = time.perf_counter()
    with ctx.Pool(procs) as pool:
        r_sfa = pool.map(_cpu_sfa_rows, [(100 + i, tok[i::procs], L, topk) for i in range(procs)])
        t_sfa = time.perf_counter() - t
        t = time.perf_counter()
        r_li = pool.map(_cpu_li_rows, [(12, rows[i::procs], L, topk) for i in range(procs)])
        t_li = time.perf_counter() - t
    # input generation inside the workers is excluded: use the slowest worker's compute time
    t_sfa_c = max(r[0] for r in r_sfa)
    t_li_c = max(r[0] for r in r_li)
    pairs_sfa = sum(r[1] for r in r_sfa)
    pairs_li = sum(r[1] for r in r_li)
    sfa_tf = pairs_sfa * SFA_HEADS * 2.0 * (SFA_D + SFA_DR + SFA_D) / t_sfa_c / 1e12
    _, li_pairs_full = li_flops(L)
    li_qtok = L / (t_li_c * li_pairs_full / pairs_li)
    return {"value": sfa_tf, "unit": UNIT, "cores": procs, "kind": "port",
            "sample": "%d attention tokens (evenly spaced positions of an %d-token sequence, all 128 heads, "
                      "top-%d) and %d indexer rows; scaled by valid query-key pairs" % (len(tok), L, topk, len(rows)),
            "li_topk_qtok_per_s": li_qtok, "sfa_seconds": t_sfa_c, "li_seconds": t_li_c,
            "wall_seconds": t_sfa + t_li}


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    lens = [L // args.scale for L in SEQ_LENS]
    topk = TOPK // args.scale
    vals, last = [], None
    for _ in range(max(1, min(args.steps, 3))):
        last = cpu_reference(sample_s=args.cpu_seconds, lens=lens, topk=topk)
        vals.append(last["value"])
    v = float(np.mean(vals))
    flops, _ = sfa_flops(lens, topk)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": int(args.gpus),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": flops / (v * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "LI B=1 S=%d N1=64 D=128 k=%d + SFA TND lens=%s N1=128 D=512+64 topk=%d, mode 3"
                               % (lens[0], topk, lens, topk), "quick": bool(args.quick)},
        "sample": last["sample"],
        "li_topk_qtok_per_s": last["li_topk_qtok_per_s"],
        "cpu_baseline": dict(last, value=v),
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--quick", action="store_true", help="1/8-size workload (debugging only; not a bench value)")
    ap.add_argument("--scale", type=int, default=1,
                    help="divide sequence lengths and top-k by this (profiling captures; not a bench value)")
    ap.add_argument("--lens", type=lambda v: [int(x) for x in v.split(",")], default=None,
                    help="attention sequence lengths instead of 8192,4096,2048,1024 (profiling captures; not a bench value)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the configuration-5 (paged decode) side measurement")
    ap.add_argument("--no-training", action="store_true", help="skip the backward operators' side measurement")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    if args.quick:
        args.scale = max(args.scale, 8)
    args.quick = args.scale > 1 or args.lens is not None
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_gpu(args)


if __name__ == "__main__":
    main()
