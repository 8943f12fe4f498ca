"""sparse_flash_attention forward on B200: the reference's public operator, unchanged signature.

Mirrors `sparse_flash_attention_triton` and `SparseFlashAttentionTriton`
(sparse_flash_attention_triton.py:1295-1509): same argument names, defaults, ValueError
guards, layouts (BSND / TND query, BSND / TND / PA_BSND key-value), block-wise indices, the
-1 convention and the (attention_out, softmax_max, softmax_sum) outputs.  TND, paged caches
and block-wise indices are resolved inside the kernels (no padded copies, no un-paging, no
expanded index tensor, no host syncs).
"""
import ctypes

import torch

from . import _cabi
from ._host import (INT64_MAX, current_stream, dtype_code, max_len_from_cumulative, note_launch, ptr,
                    require_cuda, seq_tensor, workspace)

_VALID_D = (128, 256, 512)
_D_ROPE = 64
_kernel = _cabi.KERNEL_AUTO


def set_kernel(kind):
    """"auto", "portable" (CUDA-core kernel) or "tensor" (tcgen05 path, error if not eligible)."""
    global _kernel
    _kernel = {"auto": _cabi.KERNEL_AUTO, "portable": _cabi.KERNEL_PORTABLE, "tensor": _cabi.KERNEL_TENSOR}[kind]


def sparse_flash_attention_triton(
    query,
    key,
    value,
    sparse_indices,
    scale_value: float = 1.0,
    block_table=None,
    actual_seq_lengths_query=None,
    actual_seq_lengths_kv=None,
    query_rope=None,
    key_rope=None,
    sparse_block_size: int = 1,
    layout_query: str = "BSND",
    layout_kv: str = "BSND",
    sparse_mode: int = 0,
    pre_tokens: int = INT64_MAX,
    next_tokens: int = INT64_MAX,
    attention_mode: int = 2,
    return_softmax_lse: bool = False,
    block_size: int = 0,
):
    """MLA-absorb sparse attention over index-selected keys (one KV head).

    Args (as sparse_flash_attention_triton.py:1317-1339):
        query: [B,S1,N1,D] BSND or [T1,N1,D] TND, fp16/bf16 (D in 128/256/512)
        key:   [B,S2,1,D] BSND / [T2,1,D] TND / [block_num,block_size,1,D] PA_BSND
        value: ignored (value = key[..., :D]); kept for signature parity
        sparse_indices: [B,S1,1,K] or [T1,1,K] int32 block ids, -1 = unused
        scale_value: softmax scale
        block_table: [B, max_blocks] int32, required for PA_BSND
        actual_seq_lengths_query/kv: [B] int32 / list / None; cumulative for TND,
            per-batch for BSND and PA_BSND
        query_rope / key_rope: [..., 64], required
        sparse_block_size: power of two in [1, 128]
        sparse_mode: 0 full / 3 rightDownCausal
        return_softmax_lse: also return the softmax statistics (zeros otherwise)
        block_size: paged block length (defaults to key.shape[1])

    Returns:
        (attention_out, softmax_max, softmax_sum); statistics are fp32 [B,1,S1,N1] (BSND)
        or [1,T1,N1] (TND).
    """
    if attention_mode != 2:
        raise ValueError("Only attention_mode=2 (MLA-absorb) is supported")
    if pre_tokens != INT64_MAX or next_tokens != INT64_MAX:
        raise ValueError("pre_tokens/next_tokens only support default INT64_MAX")
    if sparse_mode not in (0, 3):
        raise ValueError("Only sparse_mode 0 (full) / 3 (rightDownCausal) supported")
    if query_rope is None or key_rope is None:
        raise ValueError("query_rope and key_rope are required (no empty rope)")
    if sparse_block_size < 1 or (sparse_block_size & (sparse_block_size - 1)) != 0 or sparse_block_size > 128:
        raise ValueError("sparse_block_size must be a power of 2 in [1,128]")
    if layout_query not in ("BSND", "TND"):
        raise ValueError(f"layout_query must be BSND or TND, got {layout_query}")
    if layout_kv not in ("BSND", "TND", "PA_BSND"):
        raise ValueError(f"layout_kv must be BSND, TND or PA_BSND, got {layout_kv}")

    is_tnd_q = layout_query == "TND"
    is_tnd_kv = layout_kv == "TND"
    is_pa = layout_kv == "PA_BSND"
    if is_pa and block_table is None:
        raise ValueError("PA_BSND requires block_table")
    dev = query.device

    if is_tnd_q:
        if actual_seq_lengths_query is None:
            raise ValueError("TND query requires cumulative actual_seq_lengths_query")
        s1, N1, D = query.shape
        batch_dim = None
    else:
        batch_dim, s1, N1, D = query.shape
    d_rope = query_rope.shape[-1]

    seq_q, _ = seq_tensor(actual_seq_lengths_query, dev)
    seq_k, host_k = seq_tensor(actual_seq_lengths_kv, dev)
    B = seq_q.shape[0] if is_tnd_q else batch_dim

    pa_block = max_blocks = 0
    if is_tnd_kv:
        if seq_k is None:
            raise ValueError("TND key requires cumulative actual_seq_lengths_kv")
        n2 = key.shape[1]
        s2 = max_len_from_cumulative(host_k, key.shape[0])
    elif is_pa:
        if seq_k is None:
            raise ValueError("PA_BSND requires actual_seq_lengths_kv")
        pa_block = block_size or key.shape[1]
        if pa_block != key.shape[1]:
            raise ValueError("block_size must equal the cache's block dimension")
        n2 = key.shape[2]
        block_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        max_blocks = block_table.shape[1]
        s2 = max_blocks * pa_block
    else:
        s2, n2 = key.shape[1], key.shape[2]

    if D not in _VALID_D:
        raise ValueError(f"D must be one of {_VALID_D}, got {D}")
    if d_rope != _D_ROPE or key_rope.shape[-1] != _D_ROPE:
        raise ValueError(f"rope dim must be {_D_ROPE}, got {d_rope}")
    if n2 != 1:
        raise ValueError("Only N2=1 (MQA) is supported")
    if N1 < 1:
        raise ValueError(f"N1 must be positive, got {N1}")
    if key.shape[-1] != D:
        raise ValueError(f"query and key head dims differ: {D} vs {key.shape[-1]}")
    if not (query.dtype == key.dtype == query_rope.dtype == key_rope.dtype):
        raise ValueError("query, key, query_rope and key_rope must share a dtype")
    require_cuda(query, key, sparse_indices, query_rope, key_rope, block_table)

    query, query_rope = query.contiguous(), query_rope.contiguous()
    key, key_rope = key.contiguous(), key_rope.contiguous()
    sparse_indices = sparse_indices.to(torch.int32).contiguous()
    topk = sparse_indices.shape[-1]
    rows = s1 if is_tnd_q else B * s1

    out = torch.empty_like(query)
    stat_shape = (1, s1, N1) if is_tnd_q else (B, 1, s1, N1)
    if return_softmax_lse:
        sm_max = torch.empty(stat_shape, dtype=torch.float32, device=dev)
        sm_sum = torch.empty(stat_shape, dtype=torch.float32, device=dev)
    else:
        sm_max = sm_sum = None

    p = _cabi.DsaSfaParams()
    p.struct_size = ctypes.sizeof(_cabi.DsaSfaParams)
    p.kernel = _kernel
    p.query, p.query_rope, p.key, p.key_rope = ptr(query), ptr(query_rope), ptr(key), ptr(key_rope)
    p.sparse_indices = ptr(sparse_indices)
    p.seq_q, p.seq_k, p.block_table = ptr(seq_q), ptr(seq_k), ptr(block_table if is_pa else None)
    p.out, p.softmax_max, p.softmax_sum = ptr(out), ptr(sm_max), ptr(sm_sum)
    p.layout_q, p.layout_kv = _cabi.LAYOUTS[layout_query], _cabi.LAYOUTS[layout_kv]
    p.dtype = dtype_code(query, (torch.bfloat16, torch.float16), "query")
    p.seq_q_cumulative = 1 if is_tnd_q else 0
    p.seq_k_cumulative = 1 if is_tnd_kv else 0
    p.batch, p.s1, p.s2 = B, s1, s2
    p.n1, p.d, p.d_rope = N1, D, d_rope
    p.block_size, p.max_blocks = pa_block, max_blocks
    p.sparse_count, p.sparse_block_size = topk, sparse_block_size
    p.sparse_mode = sparse_mode
    p.return_lse = 1 if return_softmax_lse else 0
    p.scale = float(scale_value)
    p.key_rows = key.numel() // D

    if rows > 0:
        with torch.cuda.device(dev):
            nbytes = ctypes.c_size_t(0)
            _cabi.check(_cabi.lib.dsa_sfa_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)),
                        "sparse_flash_attention")
            ws = workspace(nbytes.value, dev)
            _cabi.check(_cabi.lib.dsa_sfa_forward(ctypes.byref(p), ws.data_ptr(), ws.numel(), current_stream(dev)),
                        "sparse_flash_attention")
            note_launch("sparse_flash_attention", ws, dev)
    if not return_softmax_lse:
        sm_max = torch.zeros(stat_shape, dtype=torch.float32, device=dev)
        sm_sum = torch.zeros(stat_shape, dtype=torch.float32, device=dev)
    return out, sm_max, sm_sum


class SparseFlashAttentionTriton(torch.nn.Module):
    """Attribute holder around sparse_flash_attention_triton
    (sparse_flash_attention_triton.py:1458-1509; unlike the reference Cell, `block_size` is
    forwarded)."""

    def __init__(self, scale_value=1.0, sparse_block_size=1, layout_query="BSND", layout_kv="BSND",
                 sparse_mode=0, attention_mode=2, return_softmax_lse=False, pre_tokens=INT64_MAX,
                 next_tokens=INT64_MAX, block_size=0):
        super().__init__()
        self.scale_value = scale_value
        self.sparse_block_size = sparse_block_size
        self.layout_query = layout_query
        self.layout_kv = layout_kv
        self.sparse_mode = sparse_mode
        self.attention_mode = attention_mode
        self.return_softmax_lse = return_softmax_lse
        self.pre_tokens = pre_tokens
        self.next_tokens = next_tokens
        self.block_size = block_size

    def forward(self, query, key, value, sparse_indices, query_rope=None, key_rope=None,
                actual_seq_lengths_query=None, actual_seq_lengths_kv=None, block_table=None):
        return sparse_flash_attention_triton(
            query, key, value, sparse_indices,
            scale_value=self.scale_value, block_table=block_table,
            actual_seq_lengths_query=actual_seq_lengths_query,
            actual_seq_lengths_kv=actual_seq_lengths_kv,
            query_rope=query_rope, key_rope=key_rope,
            sparse_block_size=self.sparse_block_size,
            layout_query=self.layout_query, layout_kv=self.layout_kv,
            sparse_mode=self.sparse_mode,
            pre_tokens=self.pre_tokens, next_tokens=self.next_tokens,
            attention_mode=self.attention_mode,
            return_softmax_lse=self.return_softmax_lse,
            block_size=self.block_size)

    construct = forward
