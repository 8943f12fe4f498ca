"""ctypes binding of libdsa_b200.so (the C ABI declared in include/dsa_b200.h).

There is no fallback: importing this module fails loudly when the CUDA library has not been
built (`python dsa_triton_ascend_b200/csrc/build.py`).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# DSA_B200_LIB points at another build of the same library (e.g. one compiled with
# -DDSA_SFA_PROFILE for csrc/probes/sfa_role_cycles.py); there is still no fallback.
LIB_PATH = os.environ.get("DSA_B200_LIB") or os.path.join(_HERE, "csrc", "libdsa_b200.so")

LAYOUTS = {"BSND": 0, "TND": 1, "PA_BSND": 2}
DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
RANK_IO_DTYPE, RANK_FP32 = 0, 1
KERNEL_AUTO, KERNEL_PORTABLE, KERNEL_TENSOR = 0, 1, 2
PHASE_SCORE, PHASE_TOPK, PHASE_ALL = 1, 2, 3

ERR_VALUE = -3

_c = ctypes


class DsaLiParams(_c.Structure):
    _fields_ = [
        ("struct_size", _c.c_uint32), ("kernel", _c.c_int32),
        ("query", _c.c_void_p), ("key", _c.c_void_p), ("weights", _c.c_void_p),
        ("seq_q", _c.c_void_p), ("seq_k", _c.c_void_p), ("block_table", _c.c_void_p),
        ("out_indices", _c.c_void_p), ("out_values", _c.c_void_p),
        ("layout_q", _c.c_int32), ("layout_k", _c.c_int32),
        ("dtype_qk", _c.c_int32), ("dtype_w", _c.c_int32),
        ("seq_q_cumulative", _c.c_int32), ("seq_k_cumulative", _c.c_int32),
        ("batch", _c.c_int32), ("s1", _c.c_int32), ("s2", _c.c_int32),
        ("n1", _c.c_int32), ("n2", _c.c_int32), ("d", _c.c_int32),
        ("block_size", _c.c_int32), ("max_blocks", _c.c_int32),
        ("sparse_count", _c.c_int32), ("sparse_mode", _c.c_int32),
        ("rank_mode", _c.c_int32), ("return_value", _c.c_int32), ("phases", _c.c_int32),
        ("key_rows", _c.c_int64),
    ]


class DsaSfaParams(_c.Structure):
    _fields_ = [
        ("struct_size", _c.c_uint32), ("kernel", _c.c_int32),
        ("query", _c.c_void_p), ("query_rope", _c.c_void_p), ("key", _c.c_void_p), ("key_rope", _c.c_void_p),
        ("sparse_indices", _c.c_void_p),
        ("seq_q", _c.c_void_p), ("seq_k", _c.c_void_p), ("block_table", _c.c_void_p),
        ("out", _c.c_void_p), ("softmax_max", _c.c_void_p), ("softmax_sum", _c.c_void_p),
        ("layout_q", _c.c_int32), ("layout_kv", _c.c_int32), ("dtype", _c.c_int32),
        ("seq_q_cumulative", _c.c_int32), ("seq_k_cumulative", _c.c_int32),
        ("batch", _c.c_int32), ("s1", _c.c_int32), ("s2", _c.c_int32),
        ("n1", _c.c_int32), ("d", _c.c_int32), ("d_rope", _c.c_int32),
        ("block_size", _c.c_int32), ("max_blocks", _c.c_int32),
        ("sparse_count", _c.c_int32), ("sparse_block_size", _c.c_int32),
        ("sparse_mode", _c.c_int32), ("return_lse", _c.c_int32),
        ("scale", _c.c_float),
        ("key_rows", _c.c_int64),
    ]


class DsaSfaGradParams(_c.Structure):
    _fields_ = [
        ("struct_size", _c.c_uint32), ("kernel", _c.c_int32),
        ("query", _c.c_void_p), ("query_rope", _c.c_void_p), ("key", _c.c_void_p), ("key_rope", _c.c_void_p),
        ("sparse_indices", _c.c_void_p), ("d_out", _c.c_void_p), ("out", _c.c_void_p),
        ("softmax_max", _c.c_void_p), ("softmax_sum", _c.c_void_p),
        ("seq_q", _c.c_void_p), ("seq_k", _c.c_void_p),
        ("d_query", _c.c_void_p), ("d_query_rope", _c.c_void_p),
        ("d_key", _c.c_void_p), ("d_key_rope", _c.c_void_p), ("d_value", _c.c_void_p),
        ("layout_q", _c.c_int32), ("layout_kv", _c.c_int32), ("dtype", _c.c_int32),
        ("seq_q_cumulative", _c.c_int32), ("seq_k_cumulative", _c.c_int32),
        ("batch", _c.c_int32), ("s1", _c.c_int32), ("s2", _c.c_int32),
        ("n1", _c.c_int32), ("d", _c.c_int32), ("d_rope", _c.c_int32),
        ("sparse_count", _c.c_int32), ("sparse_block_size", _c.c_int32), ("sparse_mode", _c.c_int32),
        ("scale", _c.c_float),
        ("key_rows", _c.c_int64),
    ]

class DsaSliGradParams(_c.Structure):
    _fields_ = [
        ("struct_size", _c.c_uint32), ("kernel", _c.c_int32),
        ("query", _c.c_void_p), ("query_rope", _c.c_void_p), ("key", _c.c_void_p), ("key_rope", _c.c_void_p),
        ("query_index", _c.c_void_p), ("key_index", _c.c_void_p), ("weights", _c.c_void_p),
        ("sparse_indices", _c.c_void_p), ("softmax_max", _c.c_void_p), ("softmax_sum", _c.c_void_p),
        ("seq_q", _c.c_void_p), ("seq_k", _c.c_void_p),
        ("d_query_index", _c.c_void_p), ("d_key_index", _c.c_void_p), ("d_weights", _c.c_void_p),
        ("loss", _c.c_void_p),
        ("dtype", _c.c_int32), ("dtype_w", _c.c_int32),
        ("batch", _c.c_int32), ("s1", _c.c_int32), ("s2", _c.c_int32), ("n1", _c.c_int32),
        ("d", _c.c_int32), ("d_rope", _c.c_int32), ("g", _c.c_int32), ("d_idx", _c.c_int32),
        ("topk", _c.c_int32),
        ("scale", _c.c_float),
        ("dense", _c.c_int32), ("n2", _c.c_int32),
        ("softmax_max_index", _c.c_void_p), ("softmax_sum_index", _c.c_void_p),
    ]


class DsaDenseLseParams(_c.Structure):
    _fields_ = [
        ("struct_size", _c.c_uint32), ("reserved", _c.c_int32),
        ("query_index", _c.c_void_p), ("key_index", _c.c_void_p), ("weights", _c.c_void_p),
        ("seq_q", _c.c_void_p), ("seq_k", _c.c_void_p),
        ("softmax_max_index", _c.c_void_p), ("softmax_sum_index", _c.c_void_p),
        ("dtype", _c.c_int32), ("dtype_w", _c.c_int32),
        ("batch", _c.c_int32), ("s1", _c.c_int32), ("s2", _c.c_int32), ("g", _c.c_int32), ("d_idx", _c.c_int32),
    ]


EXPORTS = (
    "dsa_abi_version", "dsa_status_string", "dsa_read_device_status",
    "dsa_li_workspace_bytes", "dsa_li_forward", "dsa_li_uses_tensor_path",
    "dsa_sfa_workspace_bytes", "dsa_sfa_forward", "dsa_sfa_uses_tensor_path",
    "dsa_li_forward_static", "dsa_li_static_scratch_bytes", "dsa_selftest_wait_timeout",
    "dsa_kernel_launch_count", "dsa_sfa_grad_workspace_bytes", "dsa_sfa_grad",
    "dsa_sli_grad_workspace_bytes", "dsa_sli_grad", "dsa_dense_li_lse_workspace_bytes", "dsa_dense_li_lse",
)


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python dsa_triton_ascend_b200/csrc/build.py` "
            "(nvcc, sm_100a). There is no CPU or eager fallback.")
    lib = _c.CDLL(LIB_PATH)
    lib.dsa_abi_version.restype = _c.c_int
    lib.dsa_status_string.restype = _c.c_char_p
    lib.dsa_status_string.argtypes = [_c.c_int]
    lib.dsa_read_device_status.argtypes = [_c.c_void_p, _c.c_void_p]
    for name, ptype in (("li", DsaLiParams), ("sfa", DsaSfaParams)):
        f = getattr(lib, f"dsa_{name}_workspace_bytes")
        f.argtypes = [_c.POINTER(ptype), _c.POINTER(_c.c_size_t)]
        f.restype = _c.c_int
        f = getattr(lib, f"dsa_{name}_forward")
        f.argtypes = [_c.POINTER(ptype), _c.c_void_p, _c.c_size_t, _c.c_void_p]
        f.restype = _c.c_int
        f = getattr(lib, f"dsa_{name}_uses_tensor_path")
        f.argtypes = [_c.POINTER(ptype)]
        f.restype = _c.c_int
    lib.dsa_sfa_grad_workspace_bytes.argtypes = [_c.POINTER(DsaSfaGradParams), _c.POINTER(_c.c_size_t)]
    lib.dsa_sfa_grad_workspace_bytes.restype = _c.c_int
    lib.dsa_sfa_grad.argtypes = [_c.POINTER(DsaSfaGradParams), _c.c_void_p, _c.c_size_t, _c.c_void_p]
    lib.dsa_sfa_grad.restype = _c.c_int
    lib.dsa_sli_grad_workspace_bytes.argtypes = [_c.POINTER(DsaSliGradParams), _c.POINTER(_c.c_size_t)]
    lib.dsa_sli_grad_workspace_bytes.restype = _c.c_int
    lib.dsa_sli_grad.argtypes = [_c.POINTER(DsaSliGradParams), _c.c_void_p, _c.c_size_t, _c.c_void_p]
    lib.dsa_sli_grad.restype = _c.c_int
    lib.dsa_dense_li_lse_workspace_bytes.argtypes = [_c.POINTER(DsaDenseLseParams), _c.POINTER(_c.c_size_t)]
    lib.dsa_dense_li_lse_workspace_bytes.restype = _c.c_int
    lib.dsa_dense_li_lse.argtypes = [_c.POINTER(DsaDenseLseParams), _c.c_void_p, _c.c_size_t, _c.c_void_p]
    lib.dsa_dense_li_lse.restype = _c.c_int
    lib.dsa_li_forward_static.argtypes = [_c.POINTER(DsaLiParams), _c.c_void_p]
    lib.dsa_li_forward_static.restype = _c.c_int
    lib.dsa_li_static_scratch_bytes.restype = _c.c_size_t
    lib.dsa_selftest_wait_timeout.argtypes = [_c.c_void_p, _c.c_size_t, _c.c_void_p]
    lib.dsa_selftest_wait_timeout.restype = _c.c_int
    lib.dsa_kernel_launch_count.restype = _c.c_ulonglong
    return lib


lib = _load()


def status_string(code):
    return lib.dsa_status_string(int(code)).decode()


def check(code, what):
    """Raise for a non-zero status: ValueError for argument errors, RuntimeError otherwise."""
    if code == 0:
        return
    msg = f"{what}: {status_string(code)} (status {code})"
    if code == ERR_VALUE:
        raise ValueError(msg)
    raise RuntimeError(msg)
