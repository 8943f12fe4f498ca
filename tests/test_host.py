"""CPU-only checks of the host side: library loads and exports the declared C ABI, struct layouts
match the header, argument guards raise like the reference wrappers, row sharding is exact."""
import ctypes
import os
import re
import subprocess
import sys
import tempfile

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "dsa_b200.h")


def test_library_exports_every_declared_symbol():
    from dsa_triton_ascend_b200 import _cabi
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(dsa_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(_cabi.lib, name), f"{name} is declared in include/dsa_b200.h but not exported"
    assert set(_cabi.EXPORTS) <= declared
    assert _cabi.lib.dsa_abi_version() >= 1
    assert _cabi.status_string(0) == "ok" and "NULL" in _cabi.status_string(-1)


def test_ctypes_structs_match_the_c_header():
    from dsa_triton_ascend_b200 import _cabi
    src = '#include <stdio.h>\n#include <stddef.h>\n#include "dsa_b200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",' \
          'sizeof(DsaLiParams),sizeof(DsaSfaParams),offsetof(DsaLiParams,phases),' \
          'offsetof(DsaSfaParams,scale),offsetof(DsaLiParams,out_indices),sizeof(DsaSfaGradParams),' \
          'offsetof(DsaSfaGradParams,d_value),offsetof(DsaSfaGradParams,key_rows),sizeof(DsaSliGradParams),' \
          'offsetof(DsaSliGradParams,scale),sizeof(DsaDenseLseParams),' \
          'offsetof(DsaSliGradParams,softmax_sum_index));return 0;}\n'
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        li, sfa, off_ph, off_sc, off_oi, grad, off_dv, off_kr, sli, off_ss, lse, off_si = map(
            int, subprocess.check_output([exe]).split())
    assert lse == ctypes.sizeof(_cabi.DsaDenseLseParams)
    assert off_si == _cabi.DsaSliGradParams.softmax_sum_index.offset
    assert sli == ctypes.sizeof(_cabi.DsaSliGradParams) and off_ss == _cabi.DsaSliGradParams.scale.offset
    assert grad == ctypes.sizeof(_cabi.DsaSfaGradParams)
    assert off_dv == _cabi.DsaSfaGradParams.d_value.offset and off_kr == _cabi.DsaSfaGradParams.key_rows.offset
    assert li == ctypes.sizeof(_cabi.DsaLiParams) and sfa == ctypes.sizeof(_cabi.DsaSfaParams)
    assert off_ph == _cabi.DsaLiParams.phases.offset
    assert off_sc == _cabi.DsaSfaParams.scale.offset
    assert off_oi == _cabi.DsaLiParams.out_indices.offset


def test_abi_rejects_bad_arguments_without_a_gpu():
    from dsa_triton_ascend_b200 import _cabi
    n = ctypes.c_size_t(0)
    p = _cabi.DsaLiParams()
    assert _cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -2  # struct_size 0
    p.struct_size = ctypes.sizeof(p)
    assert _cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -1  # NULL pointers
    p.query = p.key = p.weights = p.out_indices = 256
    p.batch, p.s1, p.s2, p.n1, p.n2, p.d = 1, 8, 64, 8, 3, 128
    p.sparse_count, p.sparse_mode, p.phases = 16, 3, 3
    assert _cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -3  # n1 % n2
    p.n2 = 1
    assert _cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == 0
    assert n.value >= 8 * 64 * 4
    p.sparse_count = 1 << 20
    assert _cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -8
    p.sparse_count = 16
    # forward refuses a missing / misaligned workspace before touching the device
    assert _cabi.lib.dsa_li_forward(ctypes.byref(p), None, 0, None) == -4
    s = _cabi.DsaSfaParams()
    s.struct_size = ctypes.sizeof(s)
    s.query = s.query_rope = s.key = s.key_rope = s.sparse_indices = s.out = 256
    s.batch, s.s1, s.s2, s.n1, s.d, s.d_rope = 1, 4, 64, 8, 192, 64
    s.sparse_count, s.sparse_block_size, s.sparse_mode = 16, 1, 3
    assert _cabi.lib.dsa_sfa_workspace_bytes(ctypes.byref(s), ctypes.byref(n)) == -3  # D not in {128,256,512}
    s.d, s.sparse_block_size = 512, 3
    assert _cabi.lib.dsa_sfa_workspace_bytes(ctypes.byref(s), ctypes.byref(n)) == -3
    s.sparse_block_size = 4
    assert _cabi.lib.dsa_sfa_workspace_bytes(ctypes.byref(s), ctypes.byref(n)) == 0


def _sfa_args(D=512, Dr=64, N1=8, N2=1):
    bf = torch.bfloat16
    q = torch.zeros(1, 4, N1, D, dtype=bf)
    k = torch.zeros(1, 32, N2, D, dtype=bf)
    qr = torch.zeros(1, 4, N1, Dr, dtype=bf)
    kr = torch.zeros(1, 32, N2, Dr, dtype=bf)
    si = torch.zeros(1, 4, 1, 8, dtype=torch.int32)
    return q, k, qr, kr, si


@pytest.mark.parametrize("kw", [
    dict(attention_mode=1), dict(pre_tokens=5), dict(next_tokens=0), dict(sparse_mode=2),
    dict(sparse_block_size=3), dict(sparse_block_size=256), dict(sparse_block_size=0),
    dict(layout_kv="PA_BSND"),
])
def test_sfa_guards_raise_value_error_like_the_reference(kw):
    """sparse_flash_attention_triton.py:1341-1351,1377-1378."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_triton
    q, k, qr, kr, si = _sfa_args()
    with pytest.raises(ValueError):
        sparse_flash_attention_triton(q, k, k, si, query_rope=qr, key_rope=kr, **kw)


def test_sfa_shape_guards_raise_value_error():
    """sparse_flash_attention_triton.py:1391-1398 and the missing-rope guard (:1347-1348)."""
    from dsa_triton_ascend_b200 import sparse_flash_attention_triton
    q, k, qr, kr, si = _sfa_args()
    with pytest.raises(ValueError):
        sparse_flash_attention_triton(q, k, k, si, query_rope=None, key_rope=kr)
    q, k, qr, kr, si = _sfa_args(D=192)
    with pytest.raises(ValueError):
        sparse_flash_attention_triton(q, k, k, si, query_rope=qr, key_rope=kr)
    q, k, qr, kr, si = _sfa_args(Dr=32)
    with pytest.raises(ValueError):
        sparse_flash_attention_triton(q, k, k, si, query_rope=qr, key_rope=kr)
    q, k, qr, kr, si = _sfa_args(N2=2)
    with pytest.raises(ValueError):
        sparse_flash_attention_triton(q, k, k, si, query_rope=qr, key_rope=kr)


def test_sfa_grad_guards_raise_value_error_like_the_reference():
    """test_sfa_grad_triton.py:307-340 (test_guards): every unsupported interface knob raises at the
    host gate, before any tensor is touched; plus the shape guards of
    sparse_flash_attention_grad_triton.py:587-594 and the ABI's own validation."""
    from dsa_triton_ascend_b200 import SparseFlashAttentionGradTriton, _cabi, sparse_flash_attention_grad_triton as gfn
    q, k, qr, kr, si = _sfa_args()
    do = out = q
    smax = torch.zeros(1, 1, 4, 8)
    ssum = torch.ones(1, 1, 4, 8)

    def call(**kw):
        base = dict(scale_value=1.0 / 24.0, query_rope=qr, key_rope=kr, sparse_mode=3)
        base.update(kw)
        return gfn(q, k, k, si, do, out, smax, ssum, **base)

    for kw in (dict(pre_tokens=0), dict(next_tokens=0), dict(sparse_mode=1), dict(deterministic=True),
               dict(sparse_block_size=3), dict(query_rope=None), dict(layout="PA_BSND")):
        with pytest.raises(ValueError):
            call(**kw)
    for bad in (dict(D=192), dict(Dr=32), dict(N2=2)):
        q2, k2, qr2, kr2, si2 = _sfa_args(**bad)
        with pytest.raises(ValueError):
            gfn(q2, k2, k2, si2, q2, q2, smax, ssum, query_rope=qr2, key_rope=kr2)
    with pytest.raises(ValueError):  # statistics of the wrong shape
        gfn(q, k, k, si, do, out, smax[:, :, :2], ssum, query_rope=qr, key_rope=kr)
    with pytest.raises(RuntimeError):  # CPU tensors: there is no CPU path
        SparseFlashAttentionGradTriton(scale_value=1.0)(q, k, k, si, do, out, smax, ssum, query_rope=qr, key_rope=kr)
    n = ctypes.c_size_t(0)
    g = _cabi.DsaSfaGradParams()
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -2
    g.struct_size = ctypes.sizeof(g)
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -1
    for f in ("query", "query_rope", "key", "key_rope", "sparse_indices", "d_out", "out", "softmax_max",
              "softmax_sum", "d_query", "d_query_rope", "d_key", "d_key_rope", "d_value"):
        setattr(g, f, 256)
    g.batch, g.s1, g.s2, g.n1, g.d, g.d_rope = 1, 4, 64, 8, 512, 64
    g.sparse_count, g.sparse_block_size, g.sparse_mode, g.key_rows = 16, 1, 3, 64
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == 0
    assert n.value == 256 + 64 * (2 * 512 + 64) * 4
    g.layout_kv = 2                                   # paged caches are not differentiated
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -3
    g.layout_kv, g.kernel = 0, 2                      # tensor-core and CUDA-core kernels take every legal shape
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == 0
    g.d = 256
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == 0
    g.kernel = 7
    assert _cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -5
    g.kernel = 0
    assert _cabi.lib.dsa_sfa_grad(ctypes.byref(g), None, 0, None) == -4


def test_sli_grad_guards_and_abi_validation():
    """sparse_lightning_indexer_grad_kl_loss_triton.py:511-515 (layout / sparse_mode / one key head) and
    the ABI's own checks, without a GPU."""
    from dsa_triton_ascend_b200 import _cabi, sparse_lightning_indexer_grad_kl_loss_triton as fn
    hf = torch.float16
    q, k = torch.zeros(1, 4, 32, 128, dtype=hf), torch.zeros(1, 64, 1, 128, dtype=hf)
    qi, ki = torch.zeros(1, 4, 8, 128, dtype=hf), torch.zeros(1, 64, 1, 128, dtype=hf)
    w, si = torch.zeros(1, 4, 8, dtype=hf), torch.zeros(1, 4, 1, 16, dtype=torch.int32)
    mx, sm = torch.zeros(1, 1, 4, 32), torch.ones(1, 1, 4, 32)
    for kw in (dict(layout="TND"), dict(sparse_mode=0)):
        with pytest.raises(ValueError):
            fn(q, k, qi, ki, w, si, mx, sm, **kw)
    with pytest.raises(ValueError):
        fn(q, k, qi, ki, w, si.repeat(1, 1, 2, 1), mx, sm)
    with pytest.raises(ValueError):
        fn(q, k, qi[..., :96], ki[..., :96], w, si, mx, sm)
    with pytest.raises(ValueError):
        fn(q, k, qi, ki, w, si, mx[..., :8], sm)
    with pytest.raises(RuntimeError):   # CPU tensors: there is no CPU path
        fn(q, k, qi, ki, w, si, mx, sm)
    n = ctypes.c_size_t(0)
    g = _cabi.DsaSliGradParams()
    assert _cabi.lib.dsa_sli_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -2
    g.struct_size = ctypes.sizeof(g)
    assert _cabi.lib.dsa_sli_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -1
    for f in ("query", "key", "query_index", "key_index", "weights", "sparse_indices", "softmax_max", "softmax_sum",
              "d_query_index", "d_key_index", "d_weights", "loss"):
        setattr(g, f, 256)
    g.batch, g.s1, g.s2, g.n1, g.d, g.d_rope, g.g, g.d_idx, g.topk = 1, 4, 64, 32, 128, 0, 8, 128, 16
    assert _cabi.lib.dsa_sli_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == 0
    assert n.value == 256 + 2 * 256 + 256 + 256 + 64 * 128 * 4
    g.d_rope = 64                                   # rope width given but no rope tensors
    assert _cabi.lib.dsa_sli_grad_workspace_bytes(ctypes.byref(g), ctypes.byref(n)) == -1
    g.d_rope = 0
    assert _cabi.lib.dsa_sli_grad(ctypes.byref(g), None, 0, None) == -4


def test_li_guards_raise_value_error_like_the_reference():
    """lightning_indexer_triton.py:501-502 (block_table without a paged layout), :524-525."""
    from dsa_triton_ascend_b200 import LightningIndexerTriton, lightning_indexer_triton
    bf = torch.bfloat16
    q = torch.zeros(1, 4, 8, 128, dtype=bf)
    k = torch.zeros(1, 16, 1, 128, dtype=bf)
    w = torch.zeros(1, 4, 8)
    with pytest.raises(ValueError):
        lightning_indexer_triton(q, k, w, block_table=torch.zeros(1, 1, dtype=torch.int32))
    with pytest.raises(ValueError):
        lightning_indexer_triton(q, torch.zeros(1, 16, 3, 128, dtype=bf), w)
    with pytest.raises(ValueError):
        lightning_indexer_triton(q, k, w, sparse_mode=1)
    with pytest.raises(ValueError):
        lightning_indexer_triton(q[0], k, w, layout_query="TND")  # TND needs cumulative lengths
    cell = LightningIndexerTriton(sparse_count=4)
    assert cell.sparse_mode == 3 and cell.layout_query == "BSND" and not cell.return_value
    with pytest.raises(RuntimeError):  # CPU tensors: there is no CPU path
        cell(q, k, w)


def test_product_package_never_imports_the_oracle():
    code = "import sys, dsa_triton_ascend_b200; assert not any(m == 'oracle' or m.startswith('oracle.') " \
           "for m in sys.modules), 'oracle imported by the product package'"
    subprocess.check_call([sys.executable, "-c", code], cwd=ROOT)
    for dirpath, _, files in os.walk(os.path.join(ROOT, "dsa_triton_ascend_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().replace("numpy golden", ""), f


def test_dense_loss_guards_raise_like_the_reference():
    """dense_loss_backward_triton.py:599-705: layout / sparse_mode / window guards, shape and dtype
    checks, statistics given together; and the LSE entry point's ABI validation."""
    from dsa_triton_ascend_b200 import _cabi, dense_lightning_indexer_softmax_lse_triton as lse
    from dsa_triton_ascend_b200 import dense_loss_backward_triton as fn
    hf = torch.float16
    q, k = torch.zeros(1, 2, 32, 128, dtype=hf), torch.zeros(1, 64, 32, 128, dtype=hf)
    qi, ki, w = torch.zeros(1, 2, 32, 128, dtype=hf), torch.zeros(1, 64, 1, 128, dtype=hf), torch.zeros(1, 2, 32, dtype=hf)
    mx, sm = torch.zeros(1, 32, 2, 1), torch.ones(1, 32, 2, 1)
    for kw in (dict(layout="TND"), dict(sparse_mode=0), dict(pre_tokens=0), dict(next_tokens=0)):
        with pytest.raises(ValueError):
            fn(q, k, qi, ki, w, mx, sm, **kw)
        with pytest.raises(ValueError):
            lse(qi, ki, w, **kw)
    with pytest.raises(ValueError):
        fn(q, k[:, :, :5], qi, ki, w, mx, sm)                       # N1 not divisible by N2
    with pytest.raises(ValueError):
        fn(q, k, qi, ki, w, mx[:, :1], sm)                          # statistics of the wrong shape
    with pytest.raises(ValueError):
        fn(q, k, qi, ki, w, mx, sm, softmax_max_index=torch.zeros(1, 1, 2))      # only one of the pair
    with pytest.raises(TypeError):
        fn(q, k, qi, ki, w, mx.half(), sm)
    with pytest.raises(TypeError):
        fn(q, k, qi.bfloat16(), ki.bfloat16(), w, mx, sm)
    with pytest.raises(ValueError):
        fn(q, k, qi, ki, w, mx, sm, query_rope=torch.zeros(1, 2, 32, 64, dtype=hf))
    with pytest.raises(ValueError):
        lse(qi[..., :96], ki[..., :96], w)
    with pytest.raises(RuntimeError):   # CPU tensors: there is no CPU path
        lse(qi, ki, w)
    p = _cabi.DsaDenseLseParams()
    n = ctypes.c_size_t(0)
    assert _cabi.lib.dsa_dense_li_lse_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -2
    p.struct_size = ctypes.sizeof(p)
    assert _cabi.lib.dsa_dense_li_lse_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -1
    p.query_index = p.key_index = p.weights = p.softmax_max_index = p.softmax_sum_index = 256
    p.batch, p.s1, p.s2, p.g, p.d_idx = 1, 2, 64, 32, 100
    assert _cabi.lib.dsa_dense_li_lse_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == -3
    p.d_idx = 128
    assert _cabi.lib.dsa_dense_li_lse_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == 0
    assert n.value == 256 + 2 * 64 * 4
    assert _cabi.lib.dsa_dense_li_lse(ctypes.byref(p), None, 0, None) == -4


def test_length_lists_are_uploaded_once():
    """seq_tensor caches the device copy of a list of lengths (an upload per call stalls the stream);
    tensors pass through untouched."""
    import torch
    from dsa_triton_ascend_b200 import _host
    a, host_a = _host.seq_tensor([3, 5, 8], "cpu")
    b, _ = _host.seq_tensor((3, 5, 8), "cpu")
    c, _ = _host.seq_tensor([3, 5, 9], "cpu")
    assert a is b and a is not c and host_a == [3, 5, 8]
    assert a.dtype == torch.int32 and a.tolist() == [3, 5, 8] and c.tolist() == [3, 5, 9]
    t = torch.tensor([1, 2], dtype=torch.int32)
    d, host_d = _host.seq_tensor(t, "cpu")
    assert d.tolist() == [1, 2] and host_d == [1, 2]
    assert _host.seq_tensor(None, "cpu") == (None, None)
