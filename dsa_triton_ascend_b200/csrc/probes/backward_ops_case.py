"""One call of each backward operator on a small seeded case (profiling aid).

    python dsa_triton_ascend_b200/csrc/probes/backward_ops_case.py [S1=128]

B=1, S2=4096, 64 attention heads (D=512+64), 64 index heads (D=128), top-k 2048, causal: the shapes
of the reference's perf scripts with fewer query rows.  Prints the time of each call (CUDA events,
second call)."""
import math
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))))


def main():
    import torch
    from dsa_triton_ascend_b200 import (dense_lightning_indexer_softmax_lse_triton, dense_loss_backward_triton,
                                        sparse_flash_attention_grad_triton, sparse_flash_attention_triton,
                                        sparse_lightning_indexer_grad_kl_loss_triton)
    S1 = int(sys.argv[1]) if len(sys.argv) > 1 else 128
    S2, N1, K, D, Dr, G, Di = 4096, 64, 2048, 512, 64, 64, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    rnd = lambda *s: (torch.randn(*s, generator=g, device="cuda") * 0.3).to(torch.bfloat16)   # noqa: E731
    q, k, qr, kr, do = rnd(1, S1, N1, D), rnd(1, S2, 1, D), rnd(1, S1, N1, Dr), rnd(1, S2, 1, Dr), rnd(1, S1, N1, D)
    qi, ki, w = rnd(1, S1, G, Di), rnd(1, S2, 1, Di), rnd(1, S1, G).abs()
    vis = S2 - S1 + torch.arange(S1, device="cuda") + 1
    idx = torch.arange(K, device="cuda", dtype=torch.int32)[None, :].repeat(S1, 1)
    idx = idx.masked_fill(torch.arange(K, device="cuda")[None, :] >= vis[:, None], -1).view(1, S1, 1, K)
    sc = 1.0 / math.sqrt(D + Dr)
    o, mx, sm = sparse_flash_attention_triton(q, k, k, idx, scale_value=sc, query_rope=qr, key_rope=kr, sparse_mode=3,
                                              return_softmax_lse=True)

    def timed(name, fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        print(f"{name}: {e0.elapsed_time(e1):.3f} ms")

    timed("sparse_flash_attention_grad", lambda: sparse_flash_attention_grad_triton(
        q, k, k, idx, do, o, mx, sm, scale_value=sc, query_rope=qr, key_rope=kr, sparse_mode=3))
    timed("sparse_lightning_indexer_grad_kl_loss", lambda: sparse_lightning_indexer_grad_kl_loss_triton(
        q, k, qi, ki, w, idx.clamp_min(0), mx, sm, query_rope=qr, key_rope=kr, scale_value=sc))
    lse = dense_lightning_indexer_softmax_lse_triton(qi, ki, w)
    dmx = torch.zeros(1, 1, S1, N1, device="cuda")
    dsm = torch.full((1, 1, S1, N1), float(S2), device="cuda")
    timed("dense_loss_backward", lambda: dense_loss_backward_triton(
        q, k, qi, ki, w, dmx, dsm, lse[0], lse[1], sc, query_rope=qr, key_rope=kr))


if __name__ == "__main__":
    main()
