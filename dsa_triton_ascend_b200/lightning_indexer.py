"""lightning_indexer on B200: the reference's public operator with an unchanged signature.

Mirrors `lightning_indexer_triton` and `LightningIndexerTriton`
(lightning_indexer_triton.py:420-554): same argument names, defaults, layouts, output shapes,
-1 convention for unused slots and ValueError guards.  The work is done by the CUDA library
behind include/dsa_b200.h; TND inputs are consumed in place (no padded copies, no host syncs).

Differences from the reference wrapper, all additive:
  * `block_table` is accepted together with layout_key="PA_BSND" (the reference raises,
    :501-502); the key is then a paged cache [num_blocks, block_size, N2, D] and
    `actual_seq_lengths_key` holds per-batch lengths.
  * unused slots of `values` hold 0 as in the numpy golden (lightning_indexer_numpy.py:66-67);
    the reference device path leaves -inf there and its tests never read them.
  * ranking: by default scores are ranked after rounding to the q/k dtype, which reproduces the
    numpy golden position for position; `set_rank_mode("fp32")` ranks raw fp32 scores like the
    reference device path (`mint.topk` on fp32, :343-361).
"""
import ctypes
import os

import torch

from . import _cabi
from ._host import (INT64_MAX, current_stream, dtype_code, max_len_from_cumulative, note_launch, ptr,
                    require_cuda, seq_tensor, workspace)

_RANK_MODES = {"io_dtype": _cabi.RANK_IO_DTYPE, "fp32": _cabi.RANK_FP32}
_rank_mode = os.environ.get("DSA_LI_RANK_MODE", "io_dtype")
_kernel = _cabi.KERNEL_AUTO


def set_rank_mode(mode):
    """"io_dtype" (default; numpy-golden ranking) or "fp32" (reference device-path ranking)."""
    global _rank_mode
    if mode not in _RANK_MODES:
        raise ValueError(f"rank mode must be one of {sorted(_RANK_MODES)}")
    _rank_mode = mode


def set_kernel(kind):
    """"auto", "portable" (CUDA-core kernels) or "tensor" (tcgen05 path, error if not eligible)."""
    global _kernel
    _kernel = {"auto": _cabi.KERNEL_AUTO, "portable": _cabi.KERNEL_PORTABLE, "tensor": _cabi.KERNEL_TENSOR}[kind]


def _build_params(query, key, weights, actual_seq_lengths_query, actual_seq_lengths_key, block_table,
                  layout_query, layout_key, sparse_count, sparse_mode, return_value, max_seqlen_key=None):
    if layout_query not in ("BSND", "TND"):
        raise ValueError(f"layout_query must be BSND or TND, got {layout_query}")
    if layout_key not in ("BSND", "TND", "PA_BSND"):
        raise ValueError(f"layout_key must be BSND, TND or PA_BSND, got {layout_key}")
    if block_table is not None and layout_key != "PA_BSND":
        raise ValueError("block_table is only valid with layout_key='PA_BSND'")
    if layout_key == "PA_BSND" and block_table is None:
        raise ValueError("PA_BSND requires block_table")
    dev = query.device
    is_tnd = layout_query == "TND"

    if is_tnd:
        if query.dim() != 3:
            raise ValueError("TND query must be [T1, N1, D]")
        if actual_seq_lengths_query is None or actual_seq_lengths_key is None:
            raise ValueError("TND layout requires cumulative actual_seq_lengths_query/key")
        T1, N1, D = query.shape
        batch_dim, s1 = None, T1
    else:
        if query.dim() != 4:
            raise ValueError("BSND query must be [B, S1, N1, D]")
        batch_dim, s1, N1, D = query.shape

    seq_q, host_q = seq_tensor(actual_seq_lengths_query, dev)
    seq_k, host_k = seq_tensor(actual_seq_lengths_key, dev)
    # As in the reference, a TND query makes both length arguments cumulative
    # (lightning_indexer_triton.py:507-509) for BSND and TND keys.  A paged cache always takes
    # per-batch key lengths, like the attention operator (sparse_flash_attention_triton.py:1379).
    q_cum = 1 if is_tnd else 0
    k_cum = 1 if (is_tnd and layout_key != "PA_BSND") else 0
    B = seq_q.shape[0] if is_tnd else batch_dim

    block_size = max_blocks = 0
    if layout_key == "BSND":
        if key.dim() != 4:
            raise ValueError("BSND key must be [B, S2, N2, D]")
        s2, N2 = key.shape[1], key.shape[2]
    elif layout_key == "TND":
        if key.dim() != 3:
            raise ValueError("TND key must be [T2, N2, D]")
        if not is_tnd:
            if seq_k is None:
                raise ValueError("TND key requires cumulative actual_seq_lengths_key")
            k_cum = 1
        N2 = key.shape[1]
        # Longest key sequence: sizes the score scratch (rows x s2 fp32) and picks the top-k kernel.
        # With lengths on the device it is unknown without a sync, so the total token count stands
        # in unless the caller passes max_seqlen_key (as varlen attention interfaces do).
        s2 = int(max_seqlen_key) if max_seqlen_key is not None else max_len_from_cumulative(host_k, key.shape[0])
    else:
        if key.dim() != 4:
            raise ValueError("PA_BSND key must be [num_blocks, block_size, N2, D]")
        if seq_k is None:
            raise ValueError("PA_BSND requires actual_seq_lengths_key")
        block_size, N2 = key.shape[1], key.shape[2]
        block_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        max_blocks = block_table.shape[1]
        s2 = max_blocks * block_size

    if key.shape[-1] != D:
        raise ValueError(f"query and key head dims differ: {D} vs {key.shape[-1]}")
    if N1 % N2 != 0:
        raise ValueError(f"N1({N1}) must be divisible by N2({N2})")
    if key.dtype != query.dtype:
        raise ValueError("query and key must share a dtype")
    require_cuda(query, key, weights, block_table)

    query, key, weights = query.contiguous(), key.contiguous(), weights.contiguous()
    rows = s1 if is_tnd else B * s1
    idx = torch.empty((rows, N2, sparse_count), dtype=torch.int32, device=dev)
    val = torch.empty((rows, N2, sparse_count), dtype=query.dtype, device=dev) if return_value else None

    p = _cabi.DsaLiParams()
    p.struct_size = ctypes.sizeof(_cabi.DsaLiParams)
    p.kernel = _kernel
    p.query, p.key, p.weights = ptr(query), ptr(key), ptr(weights)
    p.seq_q, p.seq_k, p.block_table = ptr(seq_q), ptr(seq_k), ptr(block_table)
    p.out_indices, p.out_values = ptr(idx), ptr(val)
    p.layout_q, p.layout_k = _cabi.LAYOUTS[layout_query], _cabi.LAYOUTS[layout_key]
    p.dtype_qk = dtype_code(query, (torch.bfloat16, torch.float16), "query")
    p.dtype_w = dtype_code(weights, (torch.bfloat16, torch.float16, torch.float32), "weights")
    p.seq_q_cumulative, p.seq_k_cumulative = q_cum, k_cum
    p.batch, p.s1, p.s2 = B, s1, s2
    p.n1, p.n2, p.d = N1, N2, D
    p.block_size, p.max_blocks = block_size, max_blocks
    p.sparse_count, p.sparse_mode = int(sparse_count), int(sparse_mode)
    p.rank_mode = _RANK_MODES[_rank_mode]
    p.return_value = 1 if return_value else 0
    p.phases = _cabi.PHASE_ALL
    p.key_rows = key.numel() // (N2 * D)
    keep = (query, key, weights, seq_q, seq_k, block_table, idx, val)
    out_shape = (s1, N2, sparse_count) if is_tnd else (B, s1, N2, sparse_count)
    return p, keep, idx, val, out_shape


def lightning_indexer_triton(
    query,
    key,
    weights,
    actual_seq_lengths_query=None,
    actual_seq_lengths_key=None,
    block_table=None,
    layout_query="BSND",
    layout_key="BSND",
    sparse_count=2048,
    sparse_mode=3,
    pre_tokens=INT64_MAX,
    next_tokens=INT64_MAX,
    return_value=False,
    max_seqlen_key=None,
):
    """Top-`sparse_count` keys per query row of sum_g relu(q_g . k) * w_g.

    Args (as lightning_indexer_triton.py:481-499):
        query: [B,S1,N1,D] BSND or [T1,N1,D] TND, fp16/bf16 CUDA tensor
        key: [B,S2,N2,D] BSND, [T2,N2,D] TND or paged [blocks,block_size,N2,D], same dtype
        weights: [B,S1,N1] or [T1,N1], fp16/bf16/fp32
        actual_seq_lengths_query/key: [B] int32 tensor, list or None (full); cumulative for TND
        block_table: [B, max_blocks] int32, only with layout_key="PA_BSND"
        sparse_count: top-k count; sparse_mode: 0 full, 3 rightDownCausal
        pre_tokens / next_tokens: accepted and ignored, as in the reference
        return_value: also return the selected scores (else zeros)
        max_seqlen_key: (addition) upper bound of the per-sequence key length for a TND key whose
            cumulative lengths live on the device; without it the total key count T2 is used, which
            makes the score scratch rows x T2 fp32 and sends every row to the generic top-k kernel

    Returns:
        (indices int32, values in the query dtype), shape [B,S1,N2,sparse_count] or
        [T1,N2,sparse_count]; unused slots are -1 / 0.  Indices are positions inside the
        row's own key sequence.
    """
    if sparse_mode not in (0, 3):
        raise ValueError("Only sparse_mode 0 (full) / 3 (rightDownCausal) supported")
    p, keep, idx, val, out_shape = _build_params(
        query, key, weights, actual_seq_lengths_query, actual_seq_lengths_key, block_table,
        layout_query, layout_key, sparse_count, sparse_mode, return_value, max_seqlen_key)
    dev = query.device
    with torch.cuda.device(dev):
        nbytes = ctypes.c_size_t(0)
        _cabi.check(_cabi.lib.dsa_li_workspace_bytes(ctypes.byref(p), ctypes.byref(nbytes)), "lightning_indexer")
        ws = workspace(nbytes.value, dev)
        _cabi.check(_cabi.lib.dsa_li_forward(ctypes.byref(p), ws.data_ptr(), ws.numel(), current_stream(dev)),
                    "lightning_indexer")
        note_launch("lightning_indexer", ws, dev)
    del keep
    indices = idx.view(out_shape)
    values = val.view(out_shape) if val is not None else torch.zeros(out_shape, dtype=query.dtype, device=dev)
    return indices, values


class LightningIndexerTriton(torch.nn.Module):
    """Attribute holder around lightning_indexer_triton (lightning_indexer_triton.py:420-463)."""

    def __init__(self, sparse_count=2048, sparse_mode=3, layout_query="BSND", layout_key="BSND",
                 return_value=False, pre_tokens=INT64_MAX, next_tokens=INT64_MAX):
        super().__init__()
        self.sparse_count = sparse_count
        self.sparse_mode = sparse_mode
        self.layout_query = layout_query
        self.layout_key = layout_key
        self.return_value = return_value
        self.pre_tokens = pre_tokens
        self.next_tokens = next_tokens

    def forward(self, query, key, weights, actual_seq_lengths_query=None, actual_seq_lengths_key=None,
                block_table=None):
        return lightning_indexer_triton(
            query, key, weights,
            actual_seq_lengths_query=actual_seq_lengths_query,
            actual_seq_lengths_key=actual_seq_lengths_key,
            block_table=block_table,
            layout_query=self.layout_query, layout_key=self.layout_key,
            sparse_count=self.sparse_count, sparse_mode=self.sparse_mode,
            pre_tokens=self.pre_tokens, next_tokens=self.next_tokens,
            return_value=self.return_value)

    construct = forward
