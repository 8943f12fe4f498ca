"""Host-side helpers shared by the two operator wrappers: dtype/length handling, workspace
and stream plumbing.  torch is used for device memory and streams only."""
import functools
import os

import torch

from . import _cabi

INT64_MAX = 9223372036854775807

_DTYPES = {torch.bfloat16: _cabi.DTYPE_BF16, torch.float16: _cabi.DTYPE_FP16, torch.float32: _cabi.DTYPE_FP32}


def dtype_code(t, allowed, what):
    code = _DTYPES.get(t.dtype)
    if code is None or t.dtype not in allowed:
        raise ValueError(f"{what} dtype {t.dtype} is not supported")
    return code


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("dsa_triton_ascend_b200 runs on CUDA tensors only (there is no CPU path)")


@functools.lru_cache(maxsize=256)
def _cached_lengths(values, device):
    """Device copy of a tuple of lengths.  An upload from pageable host memory first waits for the
    stream's earlier work, and the GPU then idles while the host prepares the launch (about 0.1 ms per
    operator call); the same lengths (every layer and step of a fixed batch) are uploaded once.
    The tensors are never written; the one-time wait below makes a copy safe to read from any stream."""
    t = torch.tensor(values, dtype=torch.int32, device=device)
    if t.is_cuda:
        torch.cuda.current_stream(t.device).synchronize()
    return t


def seq_tensor(lengths, device):
    """None / list / tuple / tensor -> (int32 device tensor or None, host list or None)."""
    if lengths is None:
        return None, None
    if isinstance(lengths, (list, tuple)):
        host = [int(v) for v in lengths]
        return _cached_lengths(tuple(host), str(device)), host
    if isinstance(lengths, torch.Tensor):
        host = lengths.tolist() if not lengths.is_cuda else None
        return lengths.to(device=device, dtype=torch.int32).contiguous(), host
    raise ValueError("actual_seq_lengths must be None, a list/tuple or an int32 tensor")


def max_len_from_cumulative(host, fallback):
    """Largest per-sequence length of a cumulative list (upper bound `fallback` when unknown)."""
    if not host:
        return fallback
    prev, best = 0, 0
    for v in host:
        best = max(best, v - prev)
        prev = v
    return best


def ptr(t):
    return 0 if t is None else t.data_ptr()


def workspace(nbytes, device):
    # torch's caching allocator returns 512-byte aligned blocks; the library wants 256.
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def current_stream(device):
    return torch.cuda.current_stream(device).cuda_stream


# ---- device status ----------------------------------------------------------------------------------
# Every device-side wait of the tensor-core kernels is bounded; one that runs out leaves a non-zero
# status word at the start of the call's workspace and the outputs of that call are garbage.  The
# reference reports nothing from the device, so the operators stay asynchronous by default and
# remember the workspace of the latest call per (operator, device): `check_status()` reads those
# words (it synchronises) and raises.  DSA_CHECK_STATUS=1 makes every call check itself.
_last_ws = {}
_eager_check = os.environ.get("DSA_CHECK_STATUS", "0") not in ("", "0")


def note_launch(op, ws, device):
    _last_ws[(op, torch.device(device).index)] = ws
    if _eager_check:
        check_status()


def check_status():
    """Raise RuntimeError if the latest lightning_indexer / sparse_flash_attention call on any
    device recorded a failed device-side wait.  Synchronises the streams involved."""
    for (op, index), ws in list(_last_ws.items()):
        with torch.cuda.device(index):
            st = _cabi.lib.dsa_read_device_status(ws.data_ptr(), current_stream(ws.device))
        if st != 0:
            raise RuntimeError(f"{op} on cuda:{index}: {_cabi.status_string(st)}; the outputs of that call are invalid")
