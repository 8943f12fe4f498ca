"""Case table shared by the fixture generator and the parity tests.

Shapes follow the reference's own parametrisations (test_li_triton.py:143-163,
test_sfa_triton.py:129-140, test_sfa_grad_triton.py:126-138) plus the two CPU-sized benchmark
configurations.
"""

# name -> dict(seed, B, S1, S2, N1, N2, D, k, dtype, mode, act_q, act_k)
LI_CASES = {
    "li_config1":      dict(seed=0, B=1, S1=512, S2=512, N1=8, N2=1, D=128, k=64, dtype="bf16", mode=3),
    "li_single_row":   dict(seed=11, B=1, S1=1, S2=128, N1=8, N2=1, D=128, k=32, dtype="bf16", mode=3),
    "li_odd_heads":    dict(seed=12, B=2, S1=4, S2=256, N1=7, N2=1, D=96, k=32, dtype="fp16", mode=3),
    "li_gqa2":         dict(seed=13, B=1, S1=8, S2=128, N1=16, N2=2, D=64, k=64, dtype="bf16", mode=3),
    "li_gqa4":         dict(seed=14, B=2, S1=3, S2=256, N1=12, N2=4, D=256, k=32, dtype="fp16", mode=3),
    "li_square":       dict(seed=15, B=1, S1=128, S2=128, N1=64, N2=1, D=128, k=64, dtype="bf16", mode=3),
    "li_s2_gt_s1":     dict(seed=16, B=2, S1=64, S2=512, N1=64, N2=1, D=128, k=128, dtype="fp16", mode=3),
    "li_s1_gt_s2":     dict(seed=17, B=1, S1=320, S2=256, N1=64, N2=1, D=128, k=128, dtype="bf16", mode=3),
    "li_ragged":       dict(seed=18, B=3, S1=96, S2=384, N1=64, N2=1, D=128, k=100, dtype="bf16", mode=3,
                            act_q=[96, 40, 7], act_k=[384, 130, 300]),
    "li_full_mode":    dict(seed=19, B=1, S1=16, S2=256, N1=32, N2=1, D=128, k=48, dtype="bf16", mode=0,
                            act_k=[200]),
    "li_k_gt_s2":      dict(seed=20, B=1, S1=8, S2=48, N1=16, N2=1, D=128, k=64, dtype="bf16", mode=3),
    "li_mid":          dict(seed=21, B=1, S1=1024, S2=1024, N1=64, N2=1, D=128, k=512, dtype="bf16", mode=3,
                            rows_every=37),
}

# name -> dict(seed, B, S1, S2, N1, D, k, block, mode, dtype, act_q, act_k, rows_every)
SFA_CASES = {
    "sfa_config2":     dict(seed=1, B=1, S1=256, S2=1024, N1=16, D=512, k=256, block=1, mode=3, dtype="bf16",
                            rows_every=8),
    "sfa_tiny":        dict(seed=31, B=1, S1=4, S2=128, N1=8, D=512, k=64, block=1, mode=3, dtype="bf16"),
    "sfa_tiny_full":   dict(seed=32, B=1, S1=4, S2=128, N1=8, D=512, k=64, block=1, mode=0, dtype="fp16"),
    "sfa_multi_batch": dict(seed=33, B=2, S1=16, S2=256, N1=16, D=512, k=128, block=1, mode=3, dtype="bf16"),
    "sfa_block2":      dict(seed=34, B=1, S1=8, S2=128, N1=8, D=512, k=32, block=2, mode=3, dtype="bf16"),
    "sfa_block4":      dict(seed=35, B=1, S1=8, S2=256, N1=16, D=256, k=32, block=4, mode=3, dtype="fp16"),
    "sfa_single_row":  dict(seed=36, B=1, S1=1, S2=128, N1=8, D=128, k=16, block=1, mode=3, dtype="bf16"),
    "sfa_topk2048":    dict(seed=37, B=1, S1=4, S2=2048, N1=8, D=512, k=2048, block=1, mode=3, dtype="bf16"),
    "sfa_heads128":    dict(seed=38, B=1, S1=6, S2=512, N1=128, D=512, k=320, block=1, mode=3, dtype="bf16",
                            rows_every=2),
    "sfa_ragged":      dict(seed=39, B=3, S1=24, S2=192, N1=16, D=512, k=96, block=1, mode=3, dtype="bf16",
                            act_q=[24, 10, 3], act_k=[192, 7, 100]),
}

# backward cases: same keys as SFA_CASES (shapes of test_sfa_grad_triton.py:126-138, plus a full-mode
# and a ragged case)
SFA_GRAD_CASES = {
    "sfa_grad_tiny":        dict(seed=51, B=1, S1=4, S2=128, N1=8, D=512, k=64, block=1, mode=3, dtype="bf16"),
    "sfa_grad_multi_batch": dict(seed=52, B=2, S1=16, S2=256, N1=16, D=128, k=128, block=1, mode=3, dtype="fp16"),
    "sfa_grad_block2":      dict(seed=53, B=1, S1=8, S2=128, N1=8, D=256, k=32, block=2, mode=3, dtype="bf16"),
    "sfa_grad_block4":      dict(seed=54, B=1, S1=8, S2=256, N1=16, D=512, k=32, block=4, mode=3, dtype="fp16"),
    "sfa_grad_single_row":  dict(seed=55, B=1, S1=1, S2=128, N1=8, D=128, k=16, block=1, mode=3, dtype="bf16"),
    "sfa_grad_one_head":    dict(seed=56, B=1, S1=4, S2=128, N1=1, D=512, k=64, block=1, mode=3, dtype="bf16"),
    "sfa_grad_heads128":    dict(seed=57, B=1, S1=4, S2=128, N1=128, D=256, k=64, block=1, mode=3, dtype="bf16"),
    "sfa_grad_topk2048":    dict(seed=58, B=1, S1=4, S2=2048, N1=8, D=128, k=2048, block=1, mode=3, dtype="fp16"),
    "sfa_grad_full_mode":   dict(seed=59, B=1, S1=4, S2=128, N1=8, D=256, k=64, block=1, mode=0, dtype="fp16"),
    "sfa_grad_ragged":      dict(seed=60, B=3, S1=24, S2=192, N1=16, D=512, k=96, block=1, mode=3, dtype="bf16",
                                 act_q=[24, 10, 3], act_k=[192, 7, 100]),
}

# indexer KL-loss backward: shapes of test_sli_grad_kl_loss_triton.py:17-20,46-64 scaled to what the
# numpy golden finishes in seconds; pattern = how sparse_indices are drawn (:96-131)
SLI_GRAD_CASES = {
    "sli_grad_strict":   dict(seed=61, B=1, S1=4, S2=1024, N1=64, D=512, G=16, Di=128, k=512, pattern="causal_random"),
    "sli_grad_small":    dict(seed=62, B=2, S1=6, S2=256, N1=32, D=128, G=32, Di=128, k=128, pattern="causal_random"),
    "sli_grad_heads128": dict(seed=63, B=1, S1=3, S2=384, N1=128, D=256, G=128, Di=128, k=256, pattern="causal_random"),
    "sli_grad_random":   dict(seed=64, B=1, S1=5, S2=300, N1=32, D=512, G=8, Di=256, k=200, pattern="random"),
    "sli_grad_repeated": dict(seed=65, B=1, S1=4, S2=128, N1=32, D=128, G=64, Di=128, k=96, pattern="repeated"),
    "sli_grad_k_gt_s2":  dict(seed=66, B=1, S1=8, S2=48, N1=32, D=256, G=16, Di=512, k=64, pattern="causal_continuous"),
}

# dense indexer LSE + KL-loss backward (test_dense_loss_backward_triton.py:20-58); N2 = key heads
DENSE_LOSS_CASES = {
    "dense_loss_core":    dict(seed=71, B=1, S1=2, S2=64, N1=32, N2=32, D=128, G=32, Di=128),
    "dense_loss_tail":    dict(seed=72, B=1, S1=3, S2=96, N1=32, N2=32, D=256, G=64, Di=256),
    "dense_loss_mqa":     dict(seed=73, B=1, S1=3, S2=128, N1=64, N2=1, D=512, G=128, Di=256),
    "dense_loss_gqa":     dict(seed=74, B=2, S1=5, S2=80, N1=32, N2=8, D=128, G=32, Di=128),
}


def li_case_inputs(name):
    """Seeded inputs of one LI case: (q, k, w, act_q, act_k, spec)."""
    import numpy as np
    from oracle.inputs import li_inputs
    c = LI_CASES[name]
    q, k, w = li_inputs(c["seed"], c["B"], c["S1"], c["S2"], c["N1"], c["N2"], c["D"], c["dtype"])
    act_q = np.asarray(c.get("act_q", [c["S1"]] * c["B"]), dtype=np.int32)
    act_k = np.asarray(c.get("act_k", [c["S2"]] * c["B"]), dtype=np.int32)
    return q, k, w, act_q, act_k, c


def sfa_case_inputs(name):
    """Seeded inputs of one SFA case: (q, k, q_rope, k_rope, idx, act_q, act_k, scale, spec)."""
    import numpy as np
    from oracle.inputs import sfa_inputs, sparse_indices
    c = SFA_CASES[name]
    q, k, qr, kr = sfa_inputs(c["seed"], c["B"], c["S1"], c["S2"], c["N1"], c["D"], 64, c["dtype"])
    act_q = np.asarray(c.get("act_q", [c["S1"]] * c["B"]), dtype=np.int32)
    act_k = np.asarray(c.get("act_k", [c["S2"]] * c["B"]), dtype=np.int32)
    idx = sparse_indices(c["seed"] + 1000, c["B"], c["S1"], c["S2"], c["k"], c["block"], c["mode"],
                         act_q, act_k)
    scale = 1.0 / np.sqrt(c["D"] + 64.0)
    return q, k, qr, kr, idx, act_q, act_k, scale, c

def sfa_grad_case_inputs(name):
    """Seeded inputs of one backward case:
    (q, k, q_rope, k_rope, d_out, idx, act_q, act_k, scale, spec)."""
    import numpy as np
    from oracle.inputs import sfa_grad_inputs, sparse_indices
    c = SFA_GRAD_CASES[name]
    q, k, qr, kr, do = sfa_grad_inputs(c["seed"], c["B"], c["S1"], c["S2"], c["N1"], c["D"], 64, c["dtype"])
    act_q = np.asarray(c.get("act_q", [c["S1"]] * c["B"]), dtype=np.int32)
    act_k = np.asarray(c.get("act_k", [c["S2"]] * c["B"]), dtype=np.int32)
    idx = sparse_indices(c["seed"] + 1000, c["B"], c["S1"], c["S2"], c["k"], c["block"], c["mode"],
                         act_q, act_k)
    scale = 1.0 / np.sqrt(c["D"] + 64.0)
    return q, k, qr, kr, do, idx, act_q, act_k, scale, c

def sli_grad_case_inputs(name):
    """Seeded inputs of one indexer-loss backward case:
    (q, k, qr, kr, qi, ki, w, si, scale, spec); fp16-rounded fp32 arrays."""
    import numpy as np
    from oracle.inputs import sli_grad_inputs
    c = SLI_GRAD_CASES[name]
    arrs = sli_grad_inputs(c["seed"], c["B"], c["S1"], c["S2"], c["N1"], c["D"], c["G"], c["Di"], c["k"],
                           c["pattern"])
    return arrs + (1.0 / np.sqrt(float(c["D"])), c)

def dense_loss_case_inputs(name):
    """Seeded inputs of one dense-loss case: (q, k, qr, kr, qi, ki, w, scale, spec)."""
    import numpy as np
    from oracle.inputs import dense_loss_inputs
    c = DENSE_LOSS_CASES[name]
    arrs = dense_loss_inputs(c["seed"], c["B"], c["S1"], c["S2"], c["N1"], c["N2"], c["D"], c["G"], c["Di"])
    return arrs + (1.0 / np.sqrt(c["D"] + 64.0), c)


def case_rows(c, act_q):
    """(b, s1) pairs stored for a case: every `rows_every`-th valid row (all rows by default)."""
    step = c.get("rows_every", 1)
    rows = [(b, s1) for b in range(c["B"]) for s1 in range(int(act_q[b]))]
    return rows[::step] if step > 1 else rows
