"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def tdtype(name):
    return torch.bfloat16 if name == "bf16" else torch.float16


def dev(x, dtype=None):
    """numpy fp32 array (already rounded to the io dtype) -> CUDA tensor of that dtype."""
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def li_gap_ok(q, k, w, act_q, act_k, rows, n2_count, sparse_count, sparse_mode, rel=1e-3):
    """Per (row, n2): True when the fp32 scores of the k-th and (k+1)-th best visible keys differ
    by more than `rel` relative (or when nothing is cut), so set membership is unambiguous."""
    from oracle.li_oracle import causal_limit, row_scores
    S2 = k.shape[1]
    group = q.shape[2] // n2_count
    ok = np.ones((len(rows), n2_count), dtype=bool)
    for i, (b, s1) in enumerate(rows):
        lim = causal_limit(int(act_q[b]), int(act_k[b]), s1, S2, sparse_mode)
        if lim <= sparse_count:
            continue
        for n2 in range(n2_count):
            sc = np.sort(row_scores(q[b, s1], k[b], w[b, s1], n2, group)[:lim])[::-1]
            a, c = float(sc[sparse_count - 1]), float(sc[sparse_count])
            ok[i, n2] = abs(a - c) > rel * max(abs(a), abs(c), 1e-30)
    return ok
