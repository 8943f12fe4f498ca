"""Per-role cycle counters of the attention kernel (development aid).

Builds the library with -DDSA_SFA_PROFILE next to the regular one, runs the attention operator on
one T-token sequence with top-k 2048 (TND, 128 heads, causal random indices) and prints, for both
CTAs of the first cluster, how many cycles per 64-key tile each role spent in each of its phases
(waiting for which barrier, issuing, computing).

    python dsa_triton_ascend_b200/csrc/probes/sfa_role_cycles.py [T=4096]
"""
import ctypes
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.dirname(HERE)
ROOT = os.path.dirname(os.path.dirname(CSRC))
LIB = os.path.join(HERE, "libdsa_b200_profile.so")


def build():
    src = os.path.join(CSRC, "dsa_cabi.cu")
    if os.path.exists(LIB) and os.path.getmtime(LIB) > max(
            os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))):
        return
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                    "-shared", "-lcuda", "-DDSA_SFA_PROFILE", src, "-o", LIB], check=True)


def main():
    build()
    os.environ["DSA_B200_LIB"] = LIB
    sys.path.insert(0, ROOT)
    import numpy as np
    import torch
    from dsa_triton_ascend_b200 import _cabi, sparse_flash_attention_triton
    T = int(sys.argv[1]) if len(sys.argv) > 1 else 4096
    K = 2048
    g = torch.Generator(device="cuda").manual_seed(1)
    bf = torch.bfloat16
    q = torch.randn(T, 128, 512, generator=g, device="cuda").to(bf)
    qr = torch.randn(T, 128, 64, generator=g, device="cuda").to(bf)
    k = torch.randn(T, 1, 512, generator=g, device="cuda").to(bf)
    kr = torch.randn(T, 1, 64, generator=g, device="cuda").to(bf)
    pos = torch.arange(T, device="cuda")
    r = torch.rand(T, T, device="cuda").masked_fill(pos[None, :] > pos[:, None], -1)
    tk = torch.topk(r, min(K, T), dim=1)
    top = torch.where(tk.values >= 0, tk.indices.int(), 2 ** 30)
    top = torch.sort(top, dim=1).values
    idx = torch.full((T, 1, K), -1, dtype=torch.int32, device="cuda")
    idx[:, 0, :top.shape[1]] = torch.where(top == 2 ** 30, -1, top)
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        sparse_flash_attention_triton(q, k, k, idx, scale_value=1 / 24., actual_seq_lengths_query=[T],
                                      actual_seq_lengths_kv=[T], query_rope=qr, key_rope=kr, layout_query="TND",
                                      layout_kv="TND", sparse_mode=3, return_softmax_lse=True)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    pairs = sum(min(K, s + 1) for s in range(T))
    print("ms (with counters) %.3f  TFLOP/s %.1f" % (ms, pairs * 128 * 2176 / ms / 1e9))
    f = _cabi.lib.dsa_debug_sfa_profile
    buf = (ctypes.c_longlong * 128)()
    f(buf)
    prof = np.array(buf[:])
    ntile = sum((min(K, s + 1) + 63) // 64 for s in range(0, T, 74))
    print("tiles of the first cluster:", ntile, " cycles per tile (1965 MHz): %.0f" % (ms * 1e-3 * 1.965e9 / ntile))
    tile = ["wait S", "load S + signal", "max/exp", "exchange + reference", "wait P buffer", "P + signal", "epilogue", "other"]
    roles = {0: ("K gather", ["loop", "wait slot", "issue"]),
             1: ("V copier", ["loop", "wait K landed", "load + release K", "wait V slot", "store + signal"]),
             2: ("QK issuer 0", ["loop", "wait K", "wait peer K", "wait S free", "issue", "wait Q"]),
             3: ("PV issuer", ["loop", "wait V", "wait peer V", "wait P", "issue", "wait O free"]),
             4: ("softmax group 0", tile), 5: ("softmax group 1", tile)}
    for cta in (0, 1):
        print("== CTA", cta, "(cycles per tile of the cluster; a softmax group owns every other tile)")
        for r_, (name, cols) in roles.items():
            v = prof[cta * 64 + r_ * 8: cta * 64 + r_ * 8 + 8]
            print("  %-16s" % name, "  ".join("%s=%d" % (c, x / ntile) for c, x in zip(cols, v)))


if __name__ == "__main__":
    main()
