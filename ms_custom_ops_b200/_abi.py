"""ctypes bindings of libmsco_b200.so (declared in include/msco_b200.h).

Loading fails loudly: there is no CPU or PyTorch fallback for these operators.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmsco_b200.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_OOB, ERR_INTERNAL = range(7)
DTYPE_F16, DTYPE_BF16, DTYPE_I8, DTYPE_F32, DTYPE_I32, DTYPE_I64 = range(6)
STATIC_SCRATCH_BYTES = 16 << 20  # MSCO_STATIC_SCRATCH_BYTES
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_TMA = 0, 1, 2


class MscoPaDesc(C.Structure):
    _fields_ = [
        ("q_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("block_size", C.c_int32),
        ("num_blocks", C.c_int64), ("max_blocks_per_seq", C.c_int32), ("qk_scale", C.c_float),
        ("quant_type", C.c_int32), ("has_quant_offset", C.c_int32), ("mask_type", C.c_int32),
        ("mask_dtype", C.c_int32), ("mask_batch_stride", C.c_int64), ("mask_head_stride", C.c_int64),
        ("kernel", C.c_int32), ("cache_layout", C.c_int32),
    ]


class MscoPaPlanInfo(C.Structure):
    _fields_ = [
        ("kernel", C.c_int32), ("grid", C.c_int32), ("work_items", C.c_int32), ("partials", C.c_int32),
        ("max_splits", C.c_int32), ("rows_per_item", C.c_int32), ("workspace_bytes", C.c_int64),
        ("kv_tokens", C.c_int64),
    ]


MAX_PEERS = 8
IPC_HANDLE_BYTES = 64


class MscoGatherDesc(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("gathered", C.c_void_p * MAX_PEERS),
                ("flags", C.c_void_p * MAX_PEERS), ("slice_bytes", C.c_int64), ("ticket", C.c_void_p),
                ("status", C.c_void_p), ("wait_polls", C.c_uint32), ("reserved", C.c_uint32),
                ("packets", C.c_void_p * MAX_PEERS)]


class MscoError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"[msco error {code}] {message}")
        self.code = code
        self.message = message


_lib = None

# every symbol include/msco_b200.h declares
EXPORTS = (
    "msco_version", "msco_last_error", "msco_reshape_and_cache", "msco_reshape_and_cache_quant",
    "msco_paged_attention_split_tokens", "msco_paged_attention_split_tokens_for", "msco_paged_attention_plan", "msco_paged_attention_workspace_bytes",
    "msco_paged_attention_plan_info", "msco_paged_attention_plan_destroy", "msco_paged_attention_launch",
    "msco_paged_attention_status", "msco_paged_attention_profile_enable", "msco_paged_attention_profile_read",
    "msco_paged_attention_launch_static", "msco_paged_attention_status_static",
    "msco_ipc_export", "msco_ipc_import", "msco_ipc_release", "msco_peer_allgather", "msco_decode_step", "msco_decode_step_gather",
    "msco_paged_attention_launch_lse", "msco_expand_rows_i32", "msco_paged_attention_replan", "msco_plan_arena_stats",
    "msco_reshape_and_cache_bnsd", "msco_copy_device", "msco_paged_attention_plan_tokens",
    "msco_paged_attention_replan_tokens", "msco_paged_attention_tma_supported", "msco_paged_cache_load_workspace_bytes", "msco_paged_cache_load", "msco_fa_update", "msco_fa_update_strided",
)


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ms_custom_ops_b200.build` "
            "(nvcc, sm_100a). These operators have no fallback implementation.")
    L = C.CDLL(LIB_PATH)
    vp, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t
    L.msco_version.restype = C.c_int
    L.msco_last_error.restype = C.c_char_p
    L.msco_reshape_and_cache.restype = C.c_int
    L.msco_reshape_and_cache.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, vp]
    L.msco_reshape_and_cache_quant.restype = C.c_int
    L.msco_reshape_and_cache_quant.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32, vp, vp, vp, vp, i64, vp, vp]
    L.msco_reshape_and_cache_bnsd.restype = C.c_int
    L.msco_reshape_and_cache_bnsd.argtypes = [vp, vp, vp, vp, vp, i64, i32, i64, i64, i32, i64, vp, vp]
    L.msco_copy_device.restype = C.c_int
    L.msco_copy_device.argtypes = [vp, vp, sz, vp]
    L.msco_paged_cache_load_workspace_bytes.restype = sz
    L.msco_paged_cache_load_workspace_bytes.argtypes = [i32, i32]
    L.msco_paged_cache_load.restype = C.c_int
    L.msco_paged_cache_load.argtypes = [vp] * 7 + [i32] * 4 + [i64] * 3 + [i32, vp, sz, vp, vp]
    L.msco_fa_update.restype = C.c_int
    L.msco_fa_update.argtypes = [vp, vp, vp, i64, i32, i32, vp]
    L.msco_fa_update_strided.restype = C.c_int
    L.msco_fa_update_strided.argtypes = [vp, i64, vp, i64, i32, vp, i64, i32, i32, vp]
    L.msco_paged_attention_split_tokens.restype = i32
    L.msco_paged_attention_split_tokens.argtypes = [i32, i32]
    L.msco_paged_attention_split_tokens_for.restype = i32
    L.msco_paged_attention_split_tokens_for.argtypes = [i32, i32, i32]
    L.msco_paged_attention_plan.restype = C.c_int
    L.msco_paged_attention_plan.argtypes = [C.POINTER(MscoPaDesc), C.POINTER(i32), i32, C.POINTER(vp)]
    L.msco_paged_attention_replan.restype = C.c_int
    L.msco_paged_attention_replan.argtypes = [vp, C.POINTER(i32), i32]
    L.msco_paged_attention_plan_tokens.restype = C.c_int
    L.msco_paged_attention_plan_tokens.argtypes = [C.POINTER(MscoPaDesc), C.POINTER(i32), C.POINTER(i32), i32, C.POINTER(vp)]
    L.msco_paged_attention_replan_tokens.restype = C.c_int
    L.msco_paged_attention_replan_tokens.argtypes = [vp, C.POINTER(i32), C.POINTER(i32), i32]
    L.msco_paged_attention_tma_supported.restype = i32
    L.msco_paged_attention_tma_supported.argtypes = [C.POINTER(MscoPaDesc)]
    L.msco_plan_arena_stats.restype = None
    L.msco_plan_arena_stats.argtypes = [C.POINTER(i64)]
    L.msco_paged_attention_workspace_bytes.restype = sz
    L.msco_paged_attention_workspace_bytes.argtypes = [vp]
    L.msco_paged_attention_plan_info.restype = C.c_int
    L.msco_paged_attention_plan_info.argtypes = [vp, C.POINTER(MscoPaPlanInfo)]
    L.msco_paged_attention_plan_destroy.restype = None
    L.msco_paged_attention_plan_destroy.argtypes = [vp]
    L.msco_paged_attention_launch.restype = C.c_int
    L.msco_paged_attention_launch.argtypes = [vp] * 12 + [sz, vp]
    L.msco_expand_rows_i32.restype = C.c_int
    L.msco_expand_rows_i32.argtypes = [vp, i32, i32, C.POINTER(i32), i32, vp, vp, vp]
    L.msco_paged_attention_launch_lse.restype = C.c_int
    L.msco_paged_attention_launch_lse.argtypes = [vp] * 13 + [sz, vp]
    L.msco_paged_attention_status.restype = C.c_int
    L.msco_paged_attention_status.argtypes = [vp, vp]
    L.msco_paged_attention_launch_static.restype = C.c_int
    L.msco_paged_attention_launch_static.argtypes = [vp] * 12
    L.msco_paged_attention_status_static.restype = C.c_int
    L.msco_paged_attention_status_static.argtypes = [vp]
    L.msco_decode_step.restype = C.c_int
    L.msco_decode_step.argtypes = [vp] * 6 + [i64] + [vp] * 9 + [sz, vp]
    L.msco_decode_step_gather.restype = C.c_int
    L.msco_decode_step_gather.argtypes = [vp] * 6 + [i64] + [vp] * 9 + [sz, vp, C.POINTER(MscoGatherDesc), C.c_uint32]
    L.msco_ipc_export.restype = C.c_int
    L.msco_ipc_export.argtypes = [vp, C.c_char_p, C.POINTER(i64)]
    L.msco_ipc_import.restype = C.c_int
    L.msco_ipc_import.argtypes = [C.c_char_p, i64, C.POINTER(vp)]
    L.msco_ipc_release.restype = C.c_int
    L.msco_ipc_release.argtypes = [vp, i64]
    L.msco_peer_allgather.restype = C.c_int
    L.msco_peer_allgather.argtypes = [C.POINTER(MscoGatherDesc), vp, C.c_uint32, vp]
    L.msco_paged_attention_profile_enable.restype = C.c_int
    L.msco_paged_attention_profile_enable.argtypes = [vp, i32]
    L.msco_paged_attention_profile_read.restype = C.c_int
    L.msco_paged_attention_profile_read.argtypes = [vp, C.POINTER(C.c_float), i32, C.POINTER(i32)]
    _lib = L
    return L


def check(code):
    if code != OK:
        raise MscoError(code, lib().msco_last_error().decode("utf-8", "replace"))


def plan_arena_stats():
    """Counters of the pinned plan arena (see msco_plan_arena_stats)."""
    buf = (C.c_int64 * 6)()
    lib().msco_plan_arena_stats(buf)
    names = ("slabs", "slab_bytes", "blocks_in_use", "block_allocs", "oversize_allocs", "pinned")
    return dict(zip(names, (int(v) for v in buf)))


class PaPlan:
    """Owner of one MscoPaPlan (host-side launch plan for a vector of context lengths)."""

    def __init__(self, desc: MscoPaDesc, context_lens, q_seq_lens=None):
        """`q_seq_lens` (one entry per sequence): multi-token queries, stacked into the q rows of the items."""
        L = lib()
        lens = (C.c_int32 * len(context_lens))(*[int(x) for x in context_lens])
        h = C.c_void_p()
        if q_seq_lens is None:
            check(L.msco_paged_attention_plan(C.byref(desc), lens, len(context_lens), C.byref(h)))
        else:
            ql = (C.c_int32 * len(q_seq_lens))(*[int(x) for x in q_seq_lens])
            check(L.msco_paged_attention_plan_tokens(C.byref(desc), lens, ql, len(context_lens), C.byref(h)))
        self._h = h
        self.desc = desc
        self.batch = len(context_lens)

    @property
    def handle(self):
        return self._h

    def replan(self, context_lens):
        """Re-plan in place for new lengths (same descriptor); `context_lens` is a list or an int32
        numpy array.  Keeps the plan's pinned block and tensor maps: no allocation."""
        if hasattr(context_lens, "ctypes"):
            ptr, n = context_lens.ctypes.data_as(C.POINTER(C.c_int32)), int(context_lens.size)
        else:
            n = len(context_lens)
            ptr = (C.c_int32 * n)(*[int(x) for x in context_lens])
        check(lib().msco_paged_attention_replan(self._h, ptr, n))
        self.batch = n

    @property
    def workspace_bytes(self) -> int:
        return int(lib().msco_paged_attention_workspace_bytes(self._h))

    def info(self) -> MscoPaPlanInfo:
        out = MscoPaPlanInfo()
        check(lib().msco_paged_attention_plan_info(self._h, C.byref(out)))
        return out

    def profile_enable(self, enable=True):
        check(lib().msco_paged_attention_profile_enable(self._h, int(enable)))

    def profile_read(self):
        """Attention-kernel durations (ms) of the launches since the last read (at most 64)."""
        buf = (C.c_float * 64)()
        n = C.c_int32()
        check(lib().msco_paged_attention_profile_read(self._h, buf, 64, C.byref(n)))
        return [float(buf[i]) for i in range(n.value)]

    def close(self):
        if self._h:
            lib().msco_paged_attention_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
