"""ctypes bindings of libms_custom_ops_host.so (declared in include/ms_custom_ops_c.h)."""
from __future__ import annotations

import ctypes as C
import os

from . import _abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libms_custom_ops_host.so")

MS_MAX_DIMS = 8
KIND_NONE, KIND_VALUE, KIND_TYPE, KIND_RUNTIME, KIND_UNSUPPORTED = range(5)


class MsTensorDesc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * MS_MAX_DIMS), ("strides", C.c_int64 * MS_MAX_DIMS),
                ("on_host", C.c_int32), ("reserved", C.c_int32)]


_TP = C.POINTER(MsTensorDesc)


class MsPagedAttentionArgs(C.Structure):
    _fields_ = [(n, _TP) for n in (
        "query", "key_cache", "value_cache", "block_tables", "context_lens", "attn_mask", "batch_run_status",
        "k_descale", "k_offset", "v_descale", "v_offset", "razor_offset", "p_scale", "log_n", "q_seq_lens")] + [
        ("q_head_num", C.c_int64), ("qk_scale", C.c_double), ("kv_head_num", C.c_int64), ("mask_type", C.c_int64),
        ("batch_run_status_enable", C.c_int32), ("quant_type", C.c_int64), ("out_data_type", C.c_int64),
        ("has_quant_offset", C.c_int32), ("compress_type", C.c_int64), ("calc_type", C.c_int64),
        ("scale_type", C.c_int64), ("input_layout", C.c_int64), ("mla_v_dim", C.c_int64), ("input_format", C.c_int64)]


# every symbol include/ms_custom_ops_c.h declares
EXPORTS = (
    "ms_custom_ops_reshape_and_cache", "ms_custom_ops_reshape_and_cache_quant",
    "ms_custom_ops_paged_attention_infer", "ms_custom_ops_paged_attention_workspace_size",
    "ms_custom_ops_paged_attention", "ms_custom_ops_paged_attention_last_workspace_need",
    "ms_custom_ops_paged_attention_status", "ms_custom_ops_last_error",
    "ms_custom_ops_last_error_kind", "ms_custom_ops_num_ops", "ms_custom_ops_op_name",
    "ms_custom_ops_op_signature", "ms_custom_ops_plan_cache_stats", "ms_custom_ops_plan_cache_clear",
    "ms_custom_ops_paged_cache_load_infer", "ms_custom_ops_paged_cache_load_workspace_size",
    "ms_custom_ops_paged_cache_load", "ms_custom_ops_fa_update_infer", "ms_custom_ops_fa_update",
    "ms_custom_ops_paged_attention_with_lse", "ms_custom_ops_reshape_and_cache_infer",
    "ms_custom_ops_plan_cache_miss_stats", "ms_custom_ops_plan_arena_stats",
    "ms_custom_ops_reshape_and_cache_npd_infer", "ms_custom_ops_reshape_and_cache_npd",
)


class UnsupportedOnB200(NotImplementedError):
    """The reference operator accepts this combination; the B200 build does not implement it."""


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    _abi.lib()  # the kernel library first: clearer error when nothing is built
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m ms_custom_ops_b200.build`.")
    L = C.CDLL(LIB_PATH)
    vp, i64 = C.c_void_p, C.c_int64
    L.ms_custom_ops_reshape_and_cache.restype = C.c_int
    L.ms_custom_ops_reshape_and_cache.argtypes = [_TP] * 5 + [i64, i64, vp]
    L.ms_custom_ops_reshape_and_cache_quant.restype = C.c_int
    L.ms_custom_ops_reshape_and_cache_quant.argtypes = [_TP] * 9 + [vp]
    L.ms_custom_ops_reshape_and_cache_infer.restype = C.c_int
    L.ms_custom_ops_reshape_and_cache_infer.argtypes = [_TP] * 5 + [i64, i64, C.POINTER(C.c_int32),
                                                        C.POINTER(C.c_int32), C.POINTER(i64)]
    L.ms_custom_ops_reshape_and_cache_npd_infer.restype = C.c_int
    L.ms_custom_ops_reshape_and_cache_npd_infer.argtypes = [_TP] * 8 + [C.c_char_p, C.c_char_p] + [
        C.POINTER(C.c_int32)] * 3 + [C.POINTER(i64)] * 2
    L.ms_custom_ops_reshape_and_cache_npd.restype = C.c_int
    L.ms_custom_ops_reshape_and_cache_npd.argtypes = [_TP] * 8 + [C.c_char_p, C.c_char_p, _TP, _TP, vp]
    L.ms_custom_ops_plan_cache_miss_stats.restype = None
    L.ms_custom_ops_plan_cache_miss_stats.argtypes = [C.POINTER(i64)] * 2
    L.ms_custom_ops_plan_arena_stats.restype = None
    L.ms_custom_ops_plan_arena_stats.argtypes = [C.POINTER(i64)]
    ap = C.POINTER(MsPagedAttentionArgs)
    L.ms_custom_ops_paged_attention_infer.restype = C.c_int
    L.ms_custom_ops_paged_attention_infer.argtypes = [ap, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(i64)]
    L.ms_custom_ops_paged_attention_workspace_size.restype = C.c_int
    L.ms_custom_ops_paged_attention_workspace_size.argtypes = [ap, C.POINTER(C.c_size_t)]
    L.ms_custom_ops_paged_attention.restype = C.c_int
    L.ms_custom_ops_paged_attention.argtypes = [ap, _TP, vp, C.c_size_t, vp]
    L.ms_custom_ops_paged_attention_with_lse.restype = C.c_int
    L.ms_custom_ops_paged_attention_with_lse.argtypes = [ap, _TP, _TP, vp, C.c_size_t, vp]
    L.ms_custom_ops_paged_attention_last_workspace_need.restype = C.c_size_t
    L.ms_custom_ops_paged_attention_status.restype = C.c_int
    L.ms_custom_ops_paged_attention_status.argtypes = [vp]
    i32p, i64p = C.POINTER(C.c_int32), C.POINTER(i64)
    L.ms_custom_ops_paged_cache_load_infer.restype = C.c_int
    L.ms_custom_ops_paged_cache_load_infer.argtypes = [_TP] * 5 + [i64, C.c_int32, C.c_int32, i32p, i32p, i32p,
                                                       i64p, i64p]
    L.ms_custom_ops_paged_cache_load_workspace_size.restype = C.c_size_t
    L.ms_custom_ops_paged_cache_load_workspace_size.argtypes = [_TP]
    L.ms_custom_ops_paged_cache_load.restype = C.c_int
    L.ms_custom_ops_paged_cache_load.argtypes = [_TP] * 5 + [i64, C.c_int32, C.c_int32, _TP, _TP, vp, C.c_size_t, vp]
    L.ms_custom_ops_fa_update_infer.restype = C.c_int
    L.ms_custom_ops_fa_update_infer.argtypes = [_TP, _TP, i64, i64, i32p, i32p, i64p]
    L.ms_custom_ops_fa_update.restype = C.c_int
    L.ms_custom_ops_fa_update.argtypes = [_TP, _TP, i64, i64, _TP, vp]
    L.ms_custom_ops_last_error.restype = C.c_char_p
    L.ms_custom_ops_last_error_kind.restype = C.c_int
    L.ms_custom_ops_num_ops.restype = C.c_int
    L.ms_custom_ops_op_name.restype = C.c_char_p
    L.ms_custom_ops_op_name.argtypes = [C.c_int]
    L.ms_custom_ops_op_signature.restype = C.c_char_p
    L.ms_custom_ops_op_signature.argtypes = [C.c_int]
    L.ms_custom_ops_plan_cache_stats.restype = None
    L.ms_custom_ops_plan_cache_stats.argtypes = [C.POINTER(i64)] * 3
    L.ms_custom_ops_plan_cache_clear.restype = None
    _lib = L
    return L


def check(code):
    """Raise the exception the reference would have raised for this failure."""
    if code == 0:
        return
    L = lib()
    msg = L.ms_custom_ops_last_error().decode("utf-8", "replace")
    kind = L.ms_custom_ops_last_error_kind()
    if kind == KIND_VALUE:
        raise ValueError(msg)
    if kind == KIND_TYPE:
        raise TypeError(msg)
    if kind == KIND_UNSUPPORTED:
        raise UnsupportedOnB200(msg)
    raise _abi.MscoError(code, msg)


def registered_ops():
    L = lib()
    return {L.ms_custom_ops_op_name(i).decode(): L.ms_custom_ops_op_signature(i).decode()
            for i in range(L.ms_custom_ops_num_ops())}


def plan_cache_stats():
    h, m, e = C.c_int64(), C.c_int64(), C.c_int64()
    lib().ms_custom_ops_plan_cache_stats(C.byref(h), C.byref(m), C.byref(e))
    r, c = C.c_int64(), C.c_int64()
    lib().ms_custom_ops_plan_cache_miss_stats(C.byref(r), C.byref(c))
    return {"hits": h.value, "misses": m.value, "entries": e.value, "recycled": r.value, "created": c.value}


def plan_arena_stats():
    """Counters of the pinned memory pool the plans live in (no pinned allocation on the step path:
    `slabs` stops growing after start-up)."""
    buf = (C.c_int64 * 6)()
    lib().ms_custom_ops_plan_arena_stats(buf)
    names = ("slabs", "slab_bytes", "blocks_in_use", "block_allocs", "oversize_allocs", "pinned")
    return dict(zip(names, (int(v) for v in buf)))


def plan_cache_clear():
    lib().ms_custom_ops_plan_cache_clear()
