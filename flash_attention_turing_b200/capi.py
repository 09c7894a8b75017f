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
    "fa_selftest_wait_timeout",
    "fa_fwd",
    "fa_bwd_workspace_bytes",
    "fa_bwd",
    "fa_bwd_stages",
    "fa_kvcache_num_splits",
    "fa_kvcache_workspace_bytes",
    "fa_kvcache",
    "fa_kvcache_noalloc",
    "fa_combine",
    "fa_combine_gather",
    "fa_sum_gather",
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
           ("block_table_batch_stride", _i64), ("page_size", _i32), ("block_table_cols", _i32),
           ("causal_shift", _i32), ("reserved0", _i32)]
    )


class FaBwdParams(C.Structure):
    _fields_ = (
        [("q", _vp), ("k", _vp), ("v", _vp), ("o", _vp), ("dout", _vp), ("lse", _vp), ("dq", _vp),
         ("dk", _vp), ("dv", _vp)]
        + _strides("q", "k", "v", "o", "do", "dq", "dk", "dv")
        + [("lse_row_stride", _i64), ("b", _i32), ("seqlen_q", _i32), ("seqlen_k", _i32), ("h", _i32),
           ("h_k", _i32), ("d", _i32), ("total_q", _i32), ("total_k", _i32), ("softmax_scale", _f32),
           ("is_causal", _i32), ("cu_seqlens_q", _vp), ("cu_seqlens_k", _vp), ("workspace", _vp),
           ("workspace_bytes", _sz), ("flags", _i32), ("causal_shift", _i32)]
    )


FA_BWD_SINGLE_KERNEL = 1
FA_CAUSAL_SHIFT = 2


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


class FaCombineGatherParams(C.Structure):
    _fields_ = [("o_part", _vp * 16), ("lse_part", _vp * 16), ("o", _vp), ("lse", _vp), ("num_parts", _i32),
                ("b", _i32), ("h", _i32), ("seqlen_q", _i32), ("d", _i32), ("row_begin", _i32), ("rows", _i32),
                ("reserved0", _i32)]


class FaSumGatherParams(C.Structure):
    _fields_ = [("part", _vp * 16), ("out", _vp), ("num_parts", _i32), ("b", _i32), ("h", _i32), ("seqlen_q", _i32),
                ("d", _i32), ("row_begin", _i32), ("rows", _i32), ("reserved0", _i32), ("part_first_row", _i32 * 16)]


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
        l.fa_selftest_wait_timeout.restype = C.c_int
        l.fa_selftest_wait_timeout.argtypes = [C.c_uint32, _vp]
        for name, struct in (("fa_fwd", FaFwdParams), ("fa_bwd", FaBwdParams), ("fa_kvcache", FaKvcacheParams),
                             ("fa_kvcache_noalloc", FaKvcacheParams), ("fa_combine", FaCombineParams)):
            fn = getattr(l, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(struct), _vp]
        l.fa_combine_gather.restype = C.c_int
        l.fa_combine_gather.argtypes = [C.POINTER(FaCombineGatherParams), _vp]
        l.fa_sum_gather.restype = C.c_int
        l.fa_sum_gather.argtypes = [C.POINTER(FaSumGatherParams), _vp]
        l.fa_bwd_stages.restype = C.c_int
        l.fa_bwd_stages.argtypes = [C.POINTER(FaBwdParams), C.c_int, _vp]
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


# ------------------------------------------------------------------------------------------------
# helpers that fill the parameter structs from torch tensors (dense layouts); tests and the benchmark
# use them to call the C ABI with preallocated outputs
# ------------------------------------------------------------------------------------------------
def _set_strides(p, name, x):
    setattr(p, f"{name}_batch_stride", x.stride(0))
    setattr(p, f"{name}_row_stride", x.stride(1))
    setattr(p, f"{name}_head_stride", x.stride(2))


def fwd_params(q, k, v, o, lse, softmax_scale: float, causal: bool) -> FaFwdParams:
    """q (b, sq, h, d), k/v (b, sk, hk, d), o like q, lse (b, h, sq) fp32 -- all CUDA tensors."""
    p = FaFwdParams()
    p.q, p.k, p.v, p.o, p.lse = (x.data_ptr() for x in (q, k, v, o, lse))
    for name, x in (("q", q), ("k", k), ("v", v), ("o", o)):
        _set_strides(p, name, x)
    p.lse_row_stride = lse.shape[2]
    p.b, p.seqlen_q, p.h, p.d = q.shape
    p.seqlen_k, p.h_k, p.k_batch = k.shape[1], k.shape[2], k.shape[0]
    p.softmax_scale, p.is_causal = softmax_scale, int(causal)
    return p


def bwd_params(q, k, v, o, dout, lse, dq, dk, dv, workspace, softmax_scale: float, causal: bool) -> FaBwdParams:
    p = FaBwdParams()
    p.q, p.k, p.v, p.o, p.dout, p.lse, p.dq, p.dk, p.dv = (x.data_ptr() for x in (q, k, v, o, dout, lse, dq, dk, dv))
    for name, x in (("q", q), ("k", k), ("v", v), ("o", o), ("do", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
        _set_strides(p, name, x)
    p.lse_row_stride = lse.shape[2]
    p.b, p.seqlen_q, p.h, p.d = q.shape
    p.seqlen_k, p.h_k = k.shape[1], k.shape[2]
    p.softmax_scale, p.is_causal = softmax_scale, int(causal)
    if workspace is not None:
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    return p


def kvcache_params(q, k_cache, v_cache, k_new, v_new, o, lse, cache_seqlens, block_table, softmax_scale: float,
                   causal: bool, num_splits: int, cache_batch_idx=None) -> FaKvcacheParams:
    p = FaKvcacheParams()
    p.q, p.k_cache, p.v_cache, p.o, p.lse = (x.data_ptr() for x in (q, k_cache, v_cache, o, lse))
    for name, x in (("q", q), ("kc", k_cache), ("vc", v_cache), ("o", o)):
        _set_strides(p, name, x)
    p.seqlen_new = 0
    if k_new is not None:
        p.k_new, p.v_new = k_new.data_ptr(), v_new.data_ptr()
        _set_strides(p, "kn", k_new)
        _set_strides(p, "vn", v_new)
        p.seqlen_new = k_new.shape[1]
    p.b, p.seqlen_q, p.h, p.d = q.shape
    p.h_k = k_cache.shape[2]
    p.cache_batch, p.seqlen_cache = k_cache.shape[0], k_cache.shape[1]
    p.softmax_scale, p.is_causal = softmax_scale, int(causal)
    p.cache_seqlens = cache_seqlens.data_ptr()
    if cache_batch_idx is not None:
        p.cache_batch_idx = cache_batch_idx.data_ptr()
    if block_table is not None:
        p.block_table = block_table.data_ptr()
        p.block_table_batch_stride = block_table.stride(0)
        p.max_blocks_per_seq = block_table.shape[1]
    p.num_splits = num_splits
    return p
