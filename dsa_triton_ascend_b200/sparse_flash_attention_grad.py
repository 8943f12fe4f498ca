"""sparse_flash_attention backward on B200: the reference's public operator, unchanged signature.

Mirrors `sparse_flash_attention_grad_triton` and `SparseFlashAttentionGradTriton`
(sparse_flash_attention_grad_triton.py:499-716): same argument names, defaults, ValueError
guards, layouts (BSND / TND) and the five outputs (d_query, d_key, d_value, d_query_rope,
d_key_rope), each with the shape and dtype of its forward input; d_key carries the QK path,
d_value the PV path.  Where the reference pads TND batches to dense BSND, concatenates
nope|rope copies, expands block-wise indices and computes delta = rowsum(dO * O) on the host
side before its kernel (:566-622), the kernel here reads the caller's tensors in place.
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
    """"auto" / "tensor" (mma.sync kernel) or "portable" (CUDA-core kernel)."""
    global _kernel
    _kernel = {"auto": _cabi.KERNEL_AUTO, "portable": _cabi.KERNEL_PORTABLE, "tensor": _cabi.KERNEL_TENSOR}[kind]


def sparse_flash_attention_grad_triton(
    query,
    key,
    value,
    sparse_indices,
    d_out,
    out,
    softmax_max,
    softmax_sum,
    scale_value: float = 1.0,
    query_rope=None,
    key_rope=None,
    actual_seq_lengths_query=None,
    actual_seq_lengths_kv=None,
    sparse_block_size: int = 1,
    layout: str = "BSND",
    sparse_mode: int = 3,
    pre_tokens: int = INT64_MAX,
    next_tokens: int = INT64_MAX,
    deterministic: bool = False,
):
    """Backward of the MLA-absorb sparse attention (one KV head).

    Args (as sparse_flash_attention_grad_triton.py:520-542):
        query: [B,S1,N1,D] BSND or [T1,N1,D] TND, fp16/bf16 (D in 128/256/512)
        key:   [B,S2,1,D] BSND / [T2,1,D] TND
        value: ignored (value = key[..., :D]); its gradient is still returned separately
        sparse_indices: [B,S1,1,K] or [T1,1,K] int32 block ids, -1 = unused
        d_out, out: gradient of / the forward attention output, shaped like query
        softmax_max / softmax_sum: fp32 forward statistics, [B,1,S1,N1] or [1,T1,N1]
        scale_value: softmax scale
        query_rope / key_rope: [..., 64], required
        actual_seq_lengths_query/kv: [B] int32 / list / None (cumulative for TND)
        sparse_block_size: power of two in [1, 128]
        layout: "BSND" / "TND" (query and key/value alike)
        sparse_mode: 0 full / 3 rightDownCausal
        pre_tokens / next_tokens: only the default INT64_MAX
        deterministic: only False (the scatter-add over keys uses atomics)

    Returns:
        (d_query, d_key, d_value, d_query_rope, d_key_rope)
    """
    if pre_tokens != INT64_MAX or next_tokens != INT64_MAX:
        raise ValueError("pre_tokens/next_tokens only support default INT64_MAX")
    if sparse_mode not in (0, 3):
        raise ValueError("Only sparse_mode 0 (full) / 3 (rightDownCausal) supported")
    if query_rope is None or key_rope is None:
        raise ValueError("query_rope and key_rope are required (no empty rope)")
    if deterministic:
        raise ValueError("deterministic=True is not supported (scatter-add path)")
    if sparse_block_size < 1 or (sparse_block_size & (sparse_block_size - 1)) != 0 or sparse_block_size > 128:
        raise ValueError("sparse_block_size must be a power of 2 in [1,128]")
    if layout not in ("BSND", "TND"):
        raise ValueError(f"layout must be BSND or TND, got {layout}")

    is_tnd = layout == "TND"
    dev = query.device
    if is_tnd:
        if actual_seq_lengths_query is None or actual_seq_lengths_kv is None:
            raise ValueError("TND requires cumulative actual_seq_lengths_query and actual_seq_lengths_kv")
        s1, N1, D = query.shape
        n2 = key.shape[1]
    else:
        B, s1, N1, D = query.shape
        s2, n2 = key.shape[1], key.shape[2]
    d_rope = query_rope.shape[-1]

    seq_q, _ = seq_tensor(actual_seq_lengths_query, dev)
    seq_k, host_k = seq_tensor(actual_seq_lengths_kv, dev)
    if is_tnd:
        B = seq_q.shape[0]
        s2 = max_len_from_cumulative(host_k, key.shape[0])

    if D not in _VALID_D:
        raise ValueError(f"D must be one of {_VALID_D}, got {D}")
    if d_rope != _D_ROPE or key_rope.shape[-1] != _D_ROPE:
        raise ValueError(f"rope dim must be {_D_ROPE}, got {d_rope}")
    if n2 != 1:
        raise ValueError("Only N2=1 (MQA) is supported")
    if N1 < 1:
        raise ValueError(f"N1 must be positive, got {N1}")
    if key.shape[-1] != D or d_out.shape != query.shape or out.shape != query.shape:
        raise ValueError("key, d_out and out must match query's head dim / shape")
    if not (query.dtype == key.dtype == query_rope.dtype == key_rope.dtype == d_out.dtype == out.dtype):
        raise ValueError("query, key, query_rope, key_rope, d_out and out must share a dtype")
    stat_shape = (1, s1, N1) if is_tnd else (B, 1, s1, N1)
    if tuple(softmax_max.shape) != stat_shape or tuple(softmax_sum.shape) != stat_shape:
        raise ValueError(f"softmax_max / softmax_sum must have shape {stat_shape}")
    require_cuda(query, key, sparse_indices, d_out, out, softmax_max, softmax_sum, query_rope, key_rope)

    query, query_rope = query.contiguous(), query_rope.contiguous()
    key, key_rope = key.contiguous(), key_rope.contiguous()
    d_out, out = d_out.contiguous(), out.contiguous()
    softmax_max = softmax_max.to(torch.float32).contiguous()
    softmax_sum = softmax_sum.to(torch.float32).contiguous()
    sparse_indices = sparse_indices.to(torch.int32).contiguous()

    d_query = torch.empty_like(query)
    d_query_rope = torch.empty_like(query_rope)
    d_key = torch.empty_like(key)
    d_key_rope = torch.empty_like(key_rope)
    d_value = torch.empty_like(key) if value is None else torch.empty(key.shape, dtype=value.dtype, device=dev)
    if d_value.dtype != key.dtype:
        raise ValueError("value must share key's dtype")

    p = _cabi.DsaSfaGradParams()
    p.struct_size = ctypes.sizeof(_cabi.DsaSfaGradParams)
    p.kernel = _kernel
    p.query, p.query_rope, p.key, p.key_rope = ptr(query), ptr(query_rope), ptr(key), ptr(key_rope)
    p.sparse_indices = ptr(sparse_indices)
    p.d_out, p.out = ptr(d_out), ptr(out)
    p.softmax_max, p.softmax_sum = ptr(softmax_max), ptr(softmax_sum)
    p.seq_q, p.seq_k = ptr(seq_q), ptr(seq_k)
    p.d_query, p.d_query_rope = ptr(d_query), ptr(d_query_rope)
    p.d_key, p.d_key_rope, p.d_value = ptr(d_key), ptr(d_key_rope), ptr(d_value)
    p.layout_q = p.layout_kv = _cabi.LAYOUTS[layout]
    p.dtype = dtype_code(query, (torch.bfloat16, torch.float16), "query")
    p.seq_q_cumulative = p.seq_k_cumulative = 1 if is_tnd else 0
    p.batch, p.s1, p.s2 = B, s1, s2
    p.n1, p.d, p.d_rope = N1, D, d_rope
    p.sparse_count, p.sparse_block_size = sparse_indices.shape[-1], sparse_block_size
    p.sparse_mode = sparse_mode
    p.scale = float(scale_value)
    p.key_rows = key.numel() // D

    with torch.cuda.device(dev):
        nbytes = ctypes.c_size_t(0)
        _cabi.check(_cabi.lib.dsa_sfa_grad_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)),
                    "sparse_flash_attention_grad")
        ws = workspace(nbytes.value, dev)
        _cabi.check(_cabi.lib.dsa_sfa_grad(ctypes.byref(p), ws.data_ptr(), ws.numel(), current_stream(dev)),
                    "sparse_flash_attention_grad")
        note_launch("sparse_flash_attention_grad", ws, dev)
    return d_query, d_key, d_value, d_query_rope, d_key_rope


class SparseFlashAttentionGradTriton(torch.nn.Module):
    """Attribute holder around sparse_flash_attention_grad_triton
    (sparse_flash_attention_grad_triton.py:683-716)."""

    def __init__(self, scale_value=1.0, sparse_block_size=1, layout="BSND", sparse_mode=3,
                 pre_tokens=INT64_MAX, next_tokens=INT64_MAX, deterministic=False):
        super().__init__()
        self.scale_value = scale_value
        self.sparse_block_size = sparse_block_size
        self.layout = layout
        self.sparse_mode = sparse_mode
        self.pre_tokens = pre_tokens
        self.next_tokens = next_tokens
        self.deterministic = deterministic

    def forward(self, query, key, value, sparse_indices, d_out, out, softmax_max, softmax_sum,
                query_rope=None, key_rope=None, actual_seq_lengths_query=None, actual_seq_lengths_kv=None):
        return sparse_flash_attention_grad_triton(
            query, key, value, sparse_indices, d_out, out, softmax_max, softmax_sum,
            scale_value=self.scale_value, query_rope=query_rope, key_rope=key_rope,
            actual_seq_lengths_query=actual_seq_lengths_query,
            actual_seq_lengths_kv=actual_seq_lengths_kv,
            sparse_block_size=self.sparse_block_size, layout=self.layout, sparse_mode=self.sparse_mode,
            pre_tokens=self.pre_tokens, next_tokens=self.next_tokens, deterministic=self.deterministic)

    construct = forward
