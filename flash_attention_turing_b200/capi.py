"""ctypes view of the C ABI declared in ``include/fa_b200.h``.

Used by the parity tests and the benchmark to call ``libfa_b200.so`` exactly as a non-Python host
would: raw device pointers, sizes and strides, an explicit stream, integer return codes.  The
struct layouts below must match the header field for field.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libfa_b200.so"

EXPORTED_SYMBOLS = (
    "fa_last_error",
    "fa_abi_version",
    "fa_device_status",
    "fa_fwd",
    "fa_bwd_workspace_bytes",
    "fa_bwd",
    "fa_kvcache_num_splits",
    "fa_kvcache_workspace_bytes",
    "fa_kvcache",
    "fa_combine",
)

_i64, _i32, _f32, _vp, _sz = C.c_int64, C.c_int32, C.c_float, C.c_void_p, C.c_size_t


def _strides(*names):
    return [(f"{n}_{s}_stride", _i64) for n in names for s in ("batch", "row", "head")]


class FaFwdParams(C.Structure):
    _fields_ = (
        [("q", _vp), ("k", _vp), ("v", _vp), ("o", _vp), ("lse", _vp)]
        + _strides("q", "k", "v", "o")
        + [("lse_row_stride", _i64), ("b", _i32), ("seqlen_q", _i32), ("seqlen_k", _i32), ("h", _i32),
           ("h_k", _i32), ("d", _i32), ("total_q", _i32), ("total_k", _i32), ("k_batch", _i32),
           ("softmax_scale", _f32), ("is_causal", _i32), ("cu_seqlens_q", _vp), ("cu_seqlens_k", _vp),
           ("seqused_k", _vp), ("cache_batch_idx", _vp), ("block_table", _vp),
           ("block_table_batch_stride", _i64), ("page_size", _i32), ("reserved0", _i32)]
    )


class FaBwdParams(C.Structure):
    _fields_ = (
        [("q", _vp), ("k", _vp), ("v", _vp), ("o", _vp), ("dout", _vp), ("lse", _vp), ("dq", _vp),
         ("dk", _vp), ("dv", _vp)]
        + _strides("q", "k", "v", "o", "do", "dq", "dk", "dv")
        + [("lse_row_stride", _i64), ("b", _i32), ("seqlen_q", _i32), ("seqlen_k", _i32), ("h", _i32),
           ("h_k", _i32), ("d", _i32), ("total_q", _i32), ("total_k", _i32), ("softmax_scale", _f32),
           ("is_causal", _i32), ("cu_seqlens_q", _vp), ("cu_seqlens_k", _vp), ("workspace", _vp),
           ("workspace_bytes", _sz)]
    )


class FaKvcacheParams(C.Structure):
    _fields_ = (
        [("q", _vp), ("k_cache", _vp), ("v_cache", _vp), ("k_new", _vp), ("v_new", _vp), ("o", _vp),
         ("lse", _vp)]
        + _strides("q", "kc", "vc", "kn", "vn", "o")
        + [("b", _i32), ("seqlen_q", _i32), ("seqlen_new", _i32), ("h", _i32), ("h_k", _i32), ("d", _i32),
           ("cache_batch", _i32), ("seqlen_cache", _i32), ("softmax_scale", _f32), ("is_causal", _i32),
           ("cache_seqlens", _vp), ("cache_batch_idx", _vp), ("block_table", _vp),
           ("block_table_batch_stride", _i64), ("max_blocks_per_seq", _i32), ("num_splits", _i32),
           ("workspace", _vp), ("workspace_bytes", _sz)]
    )


class FaCombineParams(C.Structure):
    _fields_ = [("o_accum", _vp), ("lse_accum", _vp), ("o", _vp), ("lse", _vp),
                ("o_batch_stride", _i64), ("o_row_stride", _i64), ("o_head_stride", _i64),
                ("num_splits", _i32), ("b", _i32), ("h", _i32), ("seqlen_q", _i32), ("d", _i32),
                ("reserved0", _i32)]


class FaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libfa_b200 error {code}: {message}")
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """dlopen ``libfa_b200.so`` (cached) and declare the prototypes."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} not found: run `python -m flash_attention_turing_b200._build`")
        l = C.CDLL(str(LIB_PATH))
        l.fa_last_error.restype = C.c_char_p
        l.fa_last_error.argtypes = []
        l.fa_abi_version.restype = C.c_int
        l.fa_device_status.restype = C.c_int
        l.fa_device_status.argtypes = [C.c_int]
        for name, struct in (("fa_fwd", FaFwdParams), ("fa_bwd", FaBwdParams),
                             ("fa_kvcache", FaKvcacheParams), ("fa_combine", FaCombineParams)):
            fn = getattr(l, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(struct), _vp]
        l.fa_bwd_workspace_bytes.restype = _sz
        l.fa_bwd_workspace_bytes.argtypes = [C.POINTER(FaBwdParams)]
        l.fa_kvcache_workspace_bytes.restype = _sz
        l.fa_kvcache_workspace_bytes.argtypes = [C.POINTER(FaKvcacheParams)]
        l.fa_kvcache_num_splits.restype = C.c_int
        l.fa_kvcache_num_splits.argtypes = [C.POINTER(FaKvcacheParams)]
        _lib = l
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise FaError(rc, lib().fa_last_error().decode())
