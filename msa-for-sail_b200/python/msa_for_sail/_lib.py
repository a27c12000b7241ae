"""ctypes binding of libmsa_b200.so (the C ABI declared in include/msa_b200.h).

There is no fallback: if the shared library is missing or was built for another
ABI revision, importing this module raises.

``MSA_BOUNDS_CHECK=1`` in the environment loads ``libmsa_b200_check.so`` instead (build it with
``build.py --bounds-check``): same ABI, every index a kernel reads from a caller's table is
range-checked and a violation comes back in the status word as ``STATUS_BOUNDS`` (upstream:
``FMHA_GMEM_CHECK=1``, jit.py:67).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
BOUNDS_CHECK = os.environ.get("MSA_BOUNDS_CHECK", "0") not in ("", "0")
LIB_PATH = os.path.join(_HERE, "libmsa_b200_check.so" if BOUNDS_CHECK else "libmsa_b200.so")
STATUS_OK, STATUS_TIMEOUT, STATUS_BOUNDS = 0, 1, 2

MSA_DT_BF16, MSA_DT_E4M3, MSA_DT_F32 = 0, 1, 2
FLAG_OUT_O, FLAG_OUT_SCORE, FLAG_SPARSE = 1, 2, 4

_p = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_f32 = ctypes.c_float


class MsaWorkItem(ctypes.Structure):
    _fields_ = [("batch", _i32), ("head0", _i32), ("row0", _i32), ("kv_tile_begin", _i32),
                ("kv_tile_end", _i32), ("split", _i32), ("num_rows", _i32), ("reserved", _i32)]


class MsaFmhaParams(ctypes.Structure):
    _fields_ = [
        ("q", _p), ("k", _p), ("v", _p), ("out", _p), ("lse", _p), ("max_score", _p),
        ("partial_o", _p), ("partial_lse", _p),
        ("qo_start", _p), ("kv_start", _p), ("kv_len", _p), ("qo_offset", _p),
        ("kv_page_indptr", _p), ("kv_indices", _p), ("kv_block_indexes", _p), ("token_batch", _p),
        ("work", _p), ("k_scale_head", _p), ("v_scale_head", _p), ("status", _p),
        ("page_batch", _p), ("sparse_ws", _p), ("sparse_ws_bytes", _i64),
        ("q_stride_tok", _i64), ("q_stride_head", _i64),
        ("k_stride_page", _i64), ("k_stride_head", _i64), ("k_stride_tok", _i64),
        ("v_stride_page", _i64), ("v_stride_head", _i64), ("v_stride_tok", _i64),
        ("out_stride_tok", _i64), ("out_stride_head", _i64),
        ("kbi_stride_tok", _i64), ("kbi_stride_head", _i64), ("kv_extent", _i64),
        ("total_q", _i32), ("num_qo_heads", _i32), ("num_kv_heads", _i32), ("batch", _i32),
        ("num_work", _i32), ("block_m", _i32), ("pack", _i32), ("page_size", _i32),
        ("kv_block_num", _i32), ("num_splits", _i32), ("max_k_tiles", _i32), ("num_logical_pages", _i32), ("decode_rows", _i32),
        ("q_dtype", _i32), ("kv_dtype", _i32), ("max_score_dtype", _i32), ("flags", _i32),
        ("sm_scale", _f32), ("out_scale", _f32),
    ]


class MsaPlanArgs(ctypes.Structure):
    _fields_ = [("qo_len", _p), ("kv_len", _p), ("qo_offset", _p), ("batch", _i32),
                ("num_qo_heads", _i32), ("num_kv_heads", _i32), ("block_m", _i32), ("pack", _i32),
                ("num_splits", _i32), ("num_sms", _i32), ("reserved", _i32)]


class MsaPlanDeviceArgs(ctypes.Structure):
    _fields_ = [("qo_len", _p), ("kv_len", _p), ("qo_offset_in", _p), ("qo_start", _p), ("kv_start", _p),
                ("kv_len_out", _p), ("qo_offset_out", _p), ("kv_page_indptr", _p), ("token_batch", _p),
                ("splits_per_row", _p), ("work", _p), ("batch", _i32), ("num_qo_heads", _i32),
                ("num_kv_heads", _i32), ("block_m", _i32), ("pack", _i32), ("num_splits", _i32),
                ("page_size", _i32), ("causal", _i32), ("noncausal_offset", _i32), ("max_total_q", _i32),
                ("row_tiles", _i32)]


#: every symbol include/msa_b200.h declares
EXPORTS = ("msa_fmha_fwd", "msa_lse_merge", "msa_topk_select", "msa_plan_dense",
           "msa_status_string", "msa_build_arch", "msa_sizeof", "msa_fmha_fwd_split_static",
           "msa_sparse_workspace_bytes", "msa_plan_device", "msa_lse_merge_ex")


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python msa-for-sail_b200/build.py` "
            "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}")
    lib.msa_sizeof.argtypes = [ctypes.c_int]
    lib.msa_sizeof.restype = ctypes.c_int
    for which, st in ((0, MsaFmhaParams), (1, MsaWorkItem), (2, MsaPlanArgs)):
        if lib.msa_sizeof(which) != ctypes.sizeof(st):
            raise ImportError(
                f"ABI mismatch for {st.__name__}: library {lib.msa_sizeof(which)} bytes, "
                f"binding {ctypes.sizeof(st)} bytes; rebuild the library")
    lib.msa_fmha_fwd.argtypes = [ctypes.POINTER(MsaFmhaParams), _p]
    lib.msa_fmha_fwd.restype = ctypes.c_int
    lib.msa_lse_merge.argtypes = [_p, _i32, _p, _p, _p, _p, _i32, _i32, _i32, _i64, _i64, _f32, _p]
    lib.msa_lse_merge.restype = ctypes.c_int
    lib.msa_lse_merge_ex.argtypes = [_p, _i32, _p, _p, _p, _i32, _p, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _f32, _p]
    lib.msa_lse_merge_ex.restype = ctypes.c_int
    lib.msa_topk_select.argtypes = [_p, _i32, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _p]
    lib.msa_topk_select.restype = ctypes.c_int
    lib.msa_plan_dense.argtypes = [ctypes.POINTER(MsaPlanArgs), _p, _i32, _p, _p]
    lib.msa_plan_dense.restype = ctypes.c_int
    lib.msa_status_string.argtypes = [ctypes.c_int]
    lib.msa_status_string.restype = ctypes.c_char_p
    lib.msa_build_arch.restype = ctypes.c_int
    lib.msa_sparse_workspace_bytes.argtypes = [_i64, _i32, _i32, _i32, _i64]
    lib.msa_sparse_workspace_bytes.restype = _i64
    lib.msa_plan_device.argtypes = [ctypes.POINTER(MsaPlanDeviceArgs), _p]
    lib.msa_plan_device.restype = ctypes.c_int
    lib.msa_fmha_fwd_split_static.argtypes = [ctypes.POINTER(MsaFmhaParams), _p, _p]
    lib.msa_fmha_fwd_split_static.restype = ctypes.c_int
    return lib


lib = _load()


def check(code, what):
    """Turn a negative status into RuntimeError (upstream surfaces native failures the same
    way through TVM_FFI_THROW, csrc/fmha_sm80_plan.cu:89-91)."""
    if code < 0:
        raise RuntimeError(f"{what} failed: {lib.msa_status_string(code).decode()} ({code})")
    return code
