"""Generate tests/golden/*.npz from the UNMODIFIED reference goldens.

Run in a container that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference
It imports lightning_indexer_numpy.lightning_indexer_golden_bsnd,
sparse_flash_attention_numpy.sparse_flash_attention_golden_bsnd and
sparse_flash_attention_grad_numpy.sparse_flash_attention_grad_golden_bsnd from that checkout,
runs them on the seeded inputs of tests/golden/cases.py and stores only the outputs (inputs
are regenerated from the seeds; the backward cases take their forward state from the forward
golden).  sli_grad_kl_loss_numpy.py (numpy_reference and _compute_sm_stats, both plain numpy) imports
mindspore at module level only to set a context; an empty stand-in module satisfies that import.
The dense-loss baselines live in the reference's test module (test_dense_loss_backward_triton.py:
_dense_indexer_lse_numpy, _compute_softmax_stats, _dense_loss_backward_numpy); they take and return
mindspore tensors only to call .asnumpy() on them, so the stand-in's Tensor is a thin holder of a
numpy array.  For cases with `rows_every` only the listed rows are kept.
The stored arrays pin the numpy restatement under oracle/ (tests/test_oracle_golden.py).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.golden.cases import (DENSE_LOSS_CASES, LI_CASES, SFA_CASES, SFA_GRAD_CASES, SLI_GRAD_CASES,  # noqa: E402
                                case_rows, dense_loss_case_inputs, li_case_inputs, sfa_case_inputs,
                                sfa_grad_case_inputs, sli_grad_case_inputs)


def main(ref_dir):
    sys.path.insert(0, ref_dir)
    import lightning_indexer_numpy as ref_li
    import sparse_flash_attention_numpy as ref_sfa
    import sparse_flash_attention_grad_numpy as ref_grad

    for name in LI_CASES:
        q, k, w, act_q, act_k, c = li_case_inputs(name)
        out = {}
        for tag, patch in (("io", False), ("fp32", True)):
            # "fp32" ranks un-rounded scores: the reference golden with its score
            # quantisation switched off (what the device path's fp32 top-k ranks).
            saved = ref_li._quantize
            if patch:
                ref_li._quantize = lambda x, value_dtype: x
            try:
                idx, val = ref_li.lightning_indexer_golden_bsnd(
                    q, k, w, act_q, act_k, sparse_count=c["k"], sparse_mode=c["mode"],
                    return_value=True, value_dtype=c["dtype"])
            finally:
                ref_li._quantize = saved
            rows = case_rows(c, act_q)
            sel = np.asarray(rows, dtype=np.int64).reshape(-1, 2)
            out[f"idx_{tag}"] = idx[sel[:, 0], sel[:, 1]]
            out[f"val_{tag}"] = val[sel[:, 0], sel[:, 1]]
            out["rows"] = sel
            if "rows_every" not in c:
                # untouched rows (s1 >= act_q) must stay -1 / 0 in the full output
                assert (idx[~_row_mask(idx.shape, sel)] == -1).all()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {k_: v.shape for k_, v in out.items()})

    for name in SFA_CASES:
        q, k, qr, kr, idx, act_q, act_k, scale, c = sfa_case_inputs(name)
        dt = ref_sfa.BF16 if c["dtype"] == "bf16" else np.float16
        o, smax, ssum = ref_sfa.sparse_flash_attention_golden_bsnd(
            q, k, k, idx, qr, kr, scale, act_q, act_k, sparse_block_size=c["block"],
            sparse_mode=c["mode"], return_softmax_lse=True, dtype=dt)
        rows = case_rows(c, act_q)
        sel = np.asarray(rows, dtype=np.int64).reshape(-1, 2)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"), rows=sel,
            out=o[sel[:, 0], sel[:, 1]].astype(np.float16 if c["dtype"] == "fp16" else np.float32),
            smax=smax[sel[:, 0], 0, sel[:, 1]], ssum=ssum[sel[:, 0], 0, sel[:, 1]])
        print(name, o.shape, len(rows))

    for name in SFA_GRAD_CASES:
        q, k, qr, kr, do, idx, act_q, act_k, scale, c = sfa_grad_case_inputs(name)
        dt = ref_sfa.BF16 if c["dtype"] == "bf16" else np.float16
        o, smax, ssum = ref_sfa.sparse_flash_attention_golden_bsnd(
            q, k, k, idx, qr, kr, scale, act_q, act_k, sparse_block_size=c["block"],
            sparse_mode=c["mode"], return_softmax_lse=True, dtype=dt)
        grads = ref_grad.sparse_flash_attention_grad_golden_bsnd(
            q, k, k, idx, do, o, smax, ssum, qr, kr, scale, act_q, act_k,
            sparse_block_size=c["block"], sparse_mode=c["mode"], dtype=dt)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            **{n: g.astype(np.float32) for n, g in
                               zip(("d_query", "d_key", "d_value", "d_query_rope", "d_key_rope"), grads)})
        print(name, [g.shape for g in grads])

    import types
    if "mindspore" not in sys.modules:
        stub = types.ModuleType("mindspore")
        stub.GRAPH_MODE = 0
        stub.set_context = lambda **kw: None
        stub.float16, stub.bfloat16, stub.float32 = "float16", "bfloat16", "float32"

        class _Holder:
            def __init__(self, a, dtype=None):
                self.a = np.asarray(a)
                self.shape = self.a.shape

            def asnumpy(self):
                return self.a

        stub.Tensor = _Holder
        sys.modules["mindspore"] = stub
    import sli_grad_kl_loss_numpy as ref_sli
    for name in SLI_GRAD_CASES:
        q, k, qr, kr, qi, ki, w, si, scale, c = sli_grad_case_inputs(name)
        sm_max, sm_sum = ref_sli._compute_sm_stats(q, k, qr, kr, scale)
        res = ref_sli.numpy_reference(q, k, qr, kr, qi, ki, w, si, sm_max, sm_sum, scale)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), sm_max=sm_max, sm_sum=sm_sum,
                            **{n: res[n].astype(np.float32) for n in ("dQueryIndex", "dKeyIndex", "dW", "loss")})
        print(name, float(res["loss"][0]), res["dKeyIndex"].shape)
    import test_dense_loss_backward_triton as ref_dense
    T = sys.modules["mindspore"].Tensor
    for name in DENSE_LOSS_CASES:
        q, k, qr, kr, qi, ki, w, scale, c = dense_loss_case_inputs(name)
        mx_i, sm_i = ref_dense._dense_indexer_lse_numpy(T(qi), T(ki), T(w))
        mx, sm = ref_dense._compute_softmax_stats(T(q), T(k), T(qr), T(kr), scale)
        res = ref_dense._dense_loss_backward_numpy(T(q), T(k), T(qr), T(kr), T(qi), T(ki), T(w), mx, sm, mx_i, sm_i, scale)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), sm_max=mx.asnumpy(), sm_sum=sm.asnumpy(),
                            max_index=mx_i.asnumpy(), sum_index=sm_i.asnumpy(),
                            **{n: r.asnumpy().astype(np.float32) for n, r in
                               zip(("dQueryIndex", "dKeyIndex", "dW", "loss"), res)})
        print(name, float(res[3].asnumpy()[0]))


def _row_mask(shape, sel):
    m = np.zeros(shape[:2], dtype=bool)
    m[sel[:, 0], sel[:, 1]] = True
    return m


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of WhFanatic/dsa_triton_ascend>")
    main(sys.argv[1])
