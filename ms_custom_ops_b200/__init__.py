"""B200-native paged-KV decode operators: ``reshape_and_cache`` and ``paged_attention``, with the
two operators either side of them, ``paged_cache_load`` and ``fa_update``.

Drop-in for the operators of the same names in ``ms_custom_ops``
(python/ms_custom_ops/__init__.py:76 re-exports them from the plugin module;
pybind definitions at ops/c_api/reshape_and_cache/reshape_and_cache.cc:212-217
and ops/c_api/paged_attention/paged_attention_pynative.cc:763-777): the same
argument names, order, defaults, layouts, dtypes and attribute values.

Call path: this module -> libms_custom_ops_host.so (C++ operator layer:
validation, plan cache) -> libmsco_b200.so (hand-written sm_100a kernels).
Tensors are torch CUDA tensors, used purely as handles to device memory; the
launch goes to torch's current stream.  ``context_lens`` must live on the host
(a CPU int32 tensor, a numpy array or a list), exactly as the reference
requires.  There is no CPU or PyTorch fallback: without the built libraries
the operators raise ImportError.
"""
from __future__ import annotations

import ctypes as C
import math
import threading
import weakref

import numpy as np

from . import _abi, _host
from ._abi import MscoError  # noqa: F401
from ._host import (UnsupportedOnB200, plan_arena_stats, plan_cache_clear, plan_cache_stats,  # noqa: F401
                    registered_ops)

__all__ = ["reshape_and_cache", "reshape_and_cache_infer", "reshape_and_cache_npd", "reshape_and_cache_npd_infer",
           "reshape_and_cache_quant", "paged_attention",
           "paged_attention_infer", "plan_arena_stats",
           "paged_cache_load", "paged_cache_load_infer", "fa_update", "fa_update_infer", "paged_attention_with_lse",
           "paged_attention_workspace_size", "paged_attention_check_status", "TensorSpec", "MscoError",
           "UnsupportedOnB200", "registered_ops", "plan_cache_stats", "plan_cache_clear"]

_DT = {"float16": _abi.DTYPE_F16, "bfloat16": _abi.DTYPE_BF16, "int8": _abi.DTYPE_I8,
       "float32": _abi.DTYPE_F32, "int32": _abi.DTYPE_I32, "int64": _abi.DTYPE_I64}
_DT_NAMES = {v: k for k, v in _DT.items()}


class TensorSpec:
    """Shape / dtype of a tensor without data: enough for shape inference and workspace sizing."""

    def __init__(self, shape, dtype, on_host=False, data=0):
        self.shape = tuple(int(s) for s in shape)
        self.dtype = dtype if isinstance(dtype, str) else str(dtype).replace("torch.", "")
        self.on_host = on_host
        self.data = data


def _dtype_code(dt) -> int:
    name = dt if isinstance(dt, str) else str(dt).replace("torch.", "")
    if name not in _DT:
        raise TypeError(f"unsupported dtype {dt}")
    return _DT[name]


def _contig_strides(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= max(int(s), 1)
    return list(reversed(st))


# id(tensor) -> (weak reference, data_ptr, shape, MsTensorDesc, pointer).  A decode loop passes the same
# tensor objects step after step; a descriptor is reused while the object is alive and still has the
# address and shape it was built from (strides only change together with one of those or through a
# view, which is another object).
_desc_cache = {}


class _Descs:
    """Builds MsTensorDesc structs and keeps the Python objects behind them alive."""

    def __init__(self):
        self.keep = []

    def __call__(self, t, host_ok=False):
        if t is None:
            return None
        d = _host.MsTensorDesc()
        if isinstance(t, TensorSpec):
            shape, strides = t.shape, _contig_strides(t.shape)
            d.data, d.dtype, d.on_host = t.data, _dtype_code(t.dtype), int(t.on_host)
        elif isinstance(t, (list, tuple, np.ndarray)):
            if not host_ok:
                raise TypeError("device tensors must be torch CUDA tensors")
            a = np.ascontiguousarray(np.asarray(t))
            if a.dtype == np.int64 and isinstance(t, (list, tuple)):
                a = a.astype(np.int32)
            self.keep.append(a)
            shape, strides = a.shape, [s // max(a.itemsize, 1) for s in a.strides]
            d.data, d.dtype, d.on_host = a.ctypes.data, _dtype_code(str(a.dtype)), 1
        else:  # torch tensor
            hit = _desc_cache.get(id(t))
            ptr = t.data_ptr()
            if hit is not None and hit[0]() is t and hit[1] == ptr and hit[2] == t.shape:
                return hit[4]
            self.keep.append(t)
            shape, strides = tuple(t.shape), tuple(t.stride())
            d.data, d.dtype, d.on_host = ptr, _dtype_code(t.dtype), 0 if t.is_cuda else 1
            if len(_desc_cache) > 4096:
                _desc_cache.clear()
            _desc_cache[id(t)] = (weakref.ref(t), ptr, t.shape, d, C.pointer(d))
        if len(shape) > _host.MS_MAX_DIMS:
            raise ValueError("tensors of more than 8 dimensions are not supported")
        d.ndim = len(shape)
        for i, (s, st) in enumerate(zip(shape, strides)):
            d.shape[i], d.strides[i] = int(s), int(st)
        self.keep.append(d)
        return C.pointer(d)


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


# --------------------------------------------------------------------------
# reshape_and_cache
# --------------------------------------------------------------------------
def reshape_and_cache(key, value=None, key_cache=None, value_cache=None, slot_mapping=None, cache_mode=0,
                      head_num=0):
    """Scatter the token rows of `key` / `value` into the paged caches, in place.

    key / value   [tokens, kv_heads * head_dim] or [batch, seq, kv_heads * head_dim]; fp16 / bf16 / int8
    key_cache / value_cache  [num_blocks, block_size, kv_heads, head_dim], same dtype as key / value
    slot_mapping  int32 [tokens]; token i goes to block slot // block_size, offset slot % block_size;
                  negative slots are skipped
    cache_mode    0 = ND (1 = FRACTAL_NZ is Ascend-only and raises UnsupportedOnB200)
    head_num      only used by the NZ layout

    Returns None, like the reference's eager entry point (it registers no output:
    ops/c_api/reshape_and_cache/reshape_and_cache.cc:204-210); the placeholder output a graph-mode
    framework sees is described by ``reshape_and_cache_infer``.
    """
    D = _Descs()
    rc = _host.lib().ms_custom_ops_reshape_and_cache(
        D(key), D(value), D(key_cache), D(value_cache), D(slot_mapping), int(cache_mode), int(head_num), _stream())
    if rc:
        _host.check(rc)
    return None


def reshape_and_cache_infer(key, value=None, key_cache=None, value_cache=None, slot_mapping=None, cache_mode=0,
                            head_num=0):
    """Shape / dtype of the operator's placeholder output (key's) after the operator's checks, without
    touching a GPU.  Accepts TensorSpec or real tensors; returns (shape tuple, dtype name)."""
    D = _Descs()
    dt, nd = C.c_int32(), C.c_int32()
    shp = (C.c_int64 * _host.MS_MAX_DIMS)()
    _host.check(_host.lib().ms_custom_ops_reshape_and_cache_infer(
        D(key), D(value), D(key_cache), D(value_cache), D(slot_mapping), int(cache_mode), int(head_num),
        C.byref(dt), C.byref(nd), shp))
    return tuple(shp[i] for i in range(nd.value)), _DT_NAMES[dt.value]


def reshape_and_cache_npd(key, value, key_cache, value_cache, slot_mapping, actual_seq_qlen, actual_seq_kvlen,
                          block_tbl, kv_cache_layout='BNSD', key_value_layout='NPD'):
    """Cache write in either block layout; returns ``(out_key, out_value)``.

    key / value   [tokens, heads * head_dim] (or [batch, seq, heads * head_dim]); fp16 / bf16 / int8
    key_cache / value_cache  kv_cache_layout 'BNSD': [num_blocks, heads, block_size, head_dim] (head-major, the
                  layout ``paged_attention(input_layout=1)`` reads); 'BSND': [num_blocks, block_size, heads, head_dim]
    slot_mapping  int32 [tokens]; negative slots are skipped
    key_value_layout  'TH': the outputs are the current key / value, (tokens, heads * head_dim).  The default
                  'NPD' (outputs re-blocked per page together with the cached history, an input format of the
                  Ascend attention kernels) raises UnsupportedOnB200; so does nothing else of the argument list.
    actual_seq_qlen / actual_seq_kvlen / block_tbl only serve the 'NPD' outputs and may be None.
    """
    import torch
    D = _Descs()
    out_key, out_value = torch.empty_like(key), torch.empty_like(value)
    rc = _host.lib().ms_custom_ops_reshape_and_cache_npd(
        D(key), D(value), D(key_cache), D(value_cache), D(slot_mapping), D(actual_seq_qlen, host_ok=True),
        D(actual_seq_kvlen, host_ok=True), D(block_tbl), str(kv_cache_layout).encode(), str(key_value_layout).encode(),
        D(out_key), D(out_value), _stream())
    if rc:
        _host.check(rc)
    return out_key, out_value


def reshape_and_cache_npd_infer(key, value, key_cache, value_cache, slot_mapping, actual_seq_qlen=None,
                                actual_seq_kvlen=None, block_tbl=None, kv_cache_layout='BNSD', key_value_layout='NPD'):
    """Shapes and dtypes of (out_key, out_value) after the operator's checks; TensorSpec or real tensors."""
    D = _Descs()
    kd, vd, nd = C.c_int32(), C.c_int32(), C.c_int32()
    ks, vs = (C.c_int64 * _host.MS_MAX_DIMS)(), (C.c_int64 * _host.MS_MAX_DIMS)()
    _host.check(_host.lib().ms_custom_ops_reshape_and_cache_npd_infer(
        D(key), D(value), D(key_cache), D(value_cache), D(slot_mapping), D(actual_seq_qlen, host_ok=True),
        D(actual_seq_kvlen, host_ok=True), D(block_tbl), str(kv_cache_layout).encode(), str(key_value_layout).encode(),
        C.byref(kd), C.byref(vd), C.byref(nd), ks, vs))
    return ((tuple(ks[i] for i in range(nd.value)), _DT_NAMES[kd.value]),
            (tuple(vs[i] for i in range(nd.value)), _DT_NAMES[vd.value]))


def reshape_and_cache_quant(key, value, key_cache, value_cache, slot_mapping, k_descale, v_descale,
                            k_offset=None, v_offset=None):
    """Extension: quantise fp16 / bf16 rows to the int8 caches while scattering them.

    Per channel c = (kv_head, head_dim): ``q = saturate_int8(rint(float32(x) / descale[c]) - offset[c])``
    with IEEE division and round-half-to-even -- the inverse of the ``(q + offset) * descale``
    de-quantisation of ``paged_attention(quant_type=1)``.  The reference operator has no such mode.
    """
    D = _Descs()
    _host.check(_host.lib().ms_custom_ops_reshape_and_cache_quant(
        D(key), D(value), D(key_cache), D(value_cache), D(slot_mapping), D(k_descale), D(v_descale),
        D(k_offset), D(v_offset), _stream()))
    return None


# --------------------------------------------------------------------------
# paged_attention
# --------------------------------------------------------------------------
def _pa_args(D, query, key_cache, value_cache, block_tables, context_lens, attn_mask, batch_run_status,
             k_descale, k_offset, v_descale, v_offset, razor_offset, p_scale, log_n, q_seq_lens, q_head_num,
             qk_scale, kv_head_num, mask_type, batch_run_status_enable, quant_type, out_data_type,
             has_quant_offset, compress_type, calc_type, scale_type, input_layout, mla_v_dim, input_format):
    # one argument block per thread and attribute set: the scalar fields are written once
    attrs = (q_head_num, qk_scale, kv_head_num, mask_type, batch_run_status_enable, quant_type, out_data_type,
             has_quant_offset, compress_type, calc_type, scale_type, input_layout, mla_v_dim, input_format)
    cache = _tls.__dict__.setdefault("pa_args", {})
    a = cache.get(attrs)
    fresh = a is None
    if fresh:
        if len(cache) > 64:
            cache.clear()
        a = cache[attrs] = _host.MsPagedAttentionArgs()
    a.query, a.key_cache, a.value_cache, a.block_tables = D(query), D(key_cache), D(value_cache), D(block_tables)
    a.context_lens = D(context_lens, host_ok=True)
    # optional tensors: most are absent in most calls; a field is only touched when it is, or was, set
    opt = (attn_mask, batch_run_status, k_descale, k_offset, v_descale, v_offset, razor_offset, p_scale, log_n,
           q_seq_lens)
    was = a._msco_optional_set if not fresh else ()
    now = []
    for name, t in zip(_PA_OPTIONAL, opt):
        if t is not None:
            setattr(a, name, D(t, host_ok=name in ("batch_run_status", "q_seq_lens")))
            now.append(name)
        elif name in was:
            setattr(a, name, None)
    a._msco_optional_set = now
    if not fresh:
        return a
    a.q_head_num, a.qk_scale, a.kv_head_num = int(q_head_num), float(qk_scale), int(kv_head_num)
    a.mask_type, a.batch_run_status_enable = int(mask_type), int(bool(batch_run_status_enable))
    a.quant_type, a.out_data_type, a.has_quant_offset = int(quant_type), int(out_data_type), int(bool(has_quant_offset))
    a.compress_type, a.calc_type, a.scale_type = int(compress_type), int(calc_type), int(scale_type)
    a.input_layout, a.mla_v_dim, a.input_format = int(input_layout), int(mla_v_dim), int(input_format)
    return a


_tls = threading.local()
_workspaces = {}  # (device index, stream handle) -> grow-only uint8 buffer


def _workspace(device, nbytes, stream_handle=None):
    import torch
    if stream_handle is None:
        stream_handle = torch.cuda.current_stream(device).cuda_stream
    key = (device.index, stream_handle)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes * 1.25), 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def paged_attention(query, key_cache, value_cache, block_tables, context_lens, attn_mask=None,
                    batch_run_status=None, k_descale=None, k_offset=None, v_descale=None, v_offset=None,
                    razor_offset=None, p_scale=None, log_n=None, q_seq_lens=None, q_head_num=0, qk_scale=1.0,
                    kv_head_num=0, mask_type=0, batch_run_status_enable=False, quant_type=0, out_data_type=-1,
                    has_quant_offset=False, compress_type=0, calc_type=0, scale_type=0, input_layout=0,
                    mla_v_dim=0, input_format=0):
    """Decode attention over the paged KV cache; returns ``attention_out`` shaped like `query`.

    query        [batch, q_head_num, head_dim] fp16 / bf16 (one token per sequence)
    key_cache / value_cache  [num_blocks, block_size, kv_heads, head_dim]; query's dtype, or int8
                 with quant_type = 1.  With input_layout = 1 (BNSD) the caches are head-major,
                 [num_blocks, kv_heads, block_size, head_dim], as reshape_and_cache_npd writes them
    block_tables int32 [batch, max_blocks]; context_lens int32 [batch] on the HOST
    attn_mask    additive: mask_type 1 (NORM) [batch, 1, max_ctx], 2 (ALIBI) [batch, heads, 1, max_ctx]
    k_descale / v_descale float32, k_offset / v_offset int32, [kv_heads * head_dim] (quant_type = 1):
                 K = (int8 + offset) * descale per channel
    Attribute values are the reference's (mask_type, quant_type, ... enums).  Combinations that the
    reference accepts but this build does not implement raise UnsupportedOnB200; invalid
    combinations raise ValueError as in the reference.
    """
    return _paged_attention(False, query, key_cache, value_cache, block_tables, context_lens, attn_mask,
                            batch_run_status, k_descale, k_offset, v_descale, v_offset, razor_offset, p_scale, log_n,
                            q_seq_lens, q_head_num, qk_scale, kv_head_num, mask_type, batch_run_status_enable,
                            quant_type, out_data_type, has_quant_offset, compress_type, calc_type, scale_type,
                            input_layout, mla_v_dim, input_format)


def paged_attention_with_lse(query, key_cache, value_cache, block_tables, context_lens, **kw):
    """Extension (no reference counterpart): ``paged_attention`` that also returns the log-sum-exp.

    Same arguments as ``paged_attention`` (optional ones by keyword).  Returns ``(attention_out, lse)``
    with ``lse`` float32 [batch, q_head_num] = log(sum over the context of exp(qk_scale * q.k + mask)),
    -inf for an empty context: attention outputs computed over different parts of a context are merged
    exactly by ``fa_update(stack(lse), stack(out.float()))``.
    """
    return _paged_attention(True, query, key_cache, value_cache, block_tables, context_lens, *_kw_to_positional(kw))


def _paged_attention(with_lse, query, *rest):
    import torch
    D = _Descs()
    a = _pa_args(D, query, *rest)
    L = _host.lib()
    out = torch.empty_like(query)
    dev = query.device
    sh = torch.cuda.current_stream(dev).cuda_stream
    stream = C.c_void_p(sh)
    # the output has query's shape, strides and dtype: its descriptor is a copy of query's with another address
    od = _tls.__dict__.get("out_desc")
    if od is None:
        od = _tls.out_desc = _host.MsTensorDesc()
        _tls.out_desc_ptr = C.pointer(od)
    if query.is_contiguous() and a.query:
        C.memmove(C.byref(od), a.query, C.sizeof(od))
        od.data = out.data_ptr()
        out_ptr = _tls.out_desc_ptr
    else:
        out_ptr = D(out)
    if with_lse:
        lse = torch.empty(query.shape[:2], dtype=torch.float32, device=dev)

        def launch(ws):
            return L.ms_custom_ops_paged_attention_with_lse(C.byref(a), out_ptr, D(lse), C.c_void_p(ws.data_ptr()),
                                                            ws.numel(), stream)
    else:
        def launch(ws):
            return L.ms_custom_ops_paged_attention(C.byref(a), out_ptr, C.c_void_p(ws.data_ptr()), ws.numel(), stream)
    # launch with the workspace at hand; if it is too small nothing was launched and the library
    # tells how much is needed (one validation + plan lookup per call in the steady state)
    ws = _workspace(dev, 0, sh)
    rc = launch(ws)
    if rc != 0:
        need = L.ms_custom_ops_paged_attention_last_workspace_need()
        if need <= ws.numel():
            _host.check(rc)
        _host.check(launch(_workspace(dev, need, sh)))
    return (out, lse) if with_lse else out


def paged_attention_infer(query, key_cache, value_cache, block_tables, context_lens, **kw):
    """Shape / dtype inference (and full argument validation) without touching a GPU.

    Accepts TensorSpec or real tensors; returns (shape tuple, dtype name).
    """
    D = _Descs()
    a = _pa_args(D, query, key_cache, value_cache, block_tables, context_lens, *_kw_to_positional(kw))
    dt, nd = C.c_int32(), C.c_int32()
    shp = (C.c_int64 * _host.MS_MAX_DIMS)()
    _host.check(_host.lib().ms_custom_ops_paged_attention_infer(C.byref(a), C.byref(dt), C.byref(nd), shp))
    return tuple(shp[i] for i in range(nd.value)), _DT_NAMES[dt.value]


def paged_attention_workspace_size(query, key_cache, value_cache, block_tables, context_lens, **kw) -> int:
    """Bytes of device workspace a launch with these arguments needs (planning only, no GPU work)."""
    D = _Descs()
    a = _pa_args(D, query, key_cache, value_cache, block_tables, context_lens, *_kw_to_positional(kw))
    n = C.c_size_t()
    _host.check(_host.lib().ms_custom_ops_paged_attention_workspace_size(C.byref(a), C.byref(n)))
    return int(n.value)


_PA_OPTIONAL = ("attn_mask", "batch_run_status", "k_descale", "k_offset", "v_descale", "v_offset", "razor_offset",
                "p_scale", "log_n", "q_seq_lens")
_PA_ATTRS = (("q_head_num", 0), ("qk_scale", 1.0), ("kv_head_num", 0), ("mask_type", 0),
             ("batch_run_status_enable", False), ("quant_type", 0), ("out_data_type", -1),
             ("has_quant_offset", False), ("compress_type", 0), ("calc_type", 0), ("scale_type", 0),
             ("input_layout", 0), ("mla_v_dim", 0), ("input_format", 0))


def _kw_to_positional(kw):
    unknown = set(kw) - set(_PA_OPTIONAL) - {n for n, _ in _PA_ATTRS}
    if unknown:
        raise TypeError(f"paged_attention got unexpected arguments {sorted(unknown)}")
    return [kw.get(n) for n in _PA_OPTIONAL] + [kw.get(n, d) for n, d in _PA_ATTRS]


# --------------------------------------------------------------------------
# paged_cache_load
# --------------------------------------------------------------------------
_load_workspaces = {}  # (device index, stream handle) -> grow-only uint8 buffer (row offsets of the gather)


def _host_int32(t):
    """Host copy of an int32 vector given as a torch tensor (either side), numpy array or list."""
    if isinstance(t, (list, tuple, np.ndarray)):
        return np.ascontiguousarray(np.asarray(t))
    return t.detach().cpu().numpy()  # a device tensor: synchronises, as the reference does


def paged_cache_load_infer(key_cache, value_cache, block_tables, seq_lens, seq_starts=None, kv_cache_cfg=0,
                           is_seq_lens_cumsum_type=False, has_seq_starts=False):
    """Shapes and dtypes of (key_out, value_out) after the operator's checks, without touching a GPU.

    Accepts TensorSpec or real tensors.  The row count is -1 when `seq_lens` carries no host values.
    """
    D = _Descs()
    kd, vd, nd = C.c_int32(), C.c_int32(), C.c_int32()
    ks, vs = (C.c_int64 * _host.MS_MAX_DIMS)(), (C.c_int64 * _host.MS_MAX_DIMS)()
    _host.check(_host.lib().ms_custom_ops_paged_cache_load_infer(
        D(key_cache), D(value_cache), D(block_tables), D(seq_lens, host_ok=True), D(seq_starts, host_ok=True),
        int(kv_cache_cfg), int(bool(is_seq_lens_cumsum_type)), int(bool(has_seq_starts)), C.byref(kd), C.byref(vd),
        C.byref(nd), ks, vs))
    return ((tuple(ks[i] for i in range(nd.value)), _DT_NAMES[kd.value]),
            (tuple(vs[i] for i in range(nd.value)), _DT_NAMES[vd.value]))


def paged_cache_load(key_cache, value_cache, block_tables, seq_lens, seq_starts=None, kv_cache_cfg=0,
                     is_seq_lens_cumsum_type=False, has_seq_starts=False):
    """Gather the token rows of every sequence from the paged caches; returns ``(key_out, value_out)``.

    key_cache / value_cache  [num_blocks, block_size, num_heads, head_size_k / head_size_v];
                 fp16 / bf16 / int8, the two may differ
    block_tables int32 [batch, block_indices]
    seq_lens     int32 [batch] lengths, or [batch + 1] running sums with is_seq_lens_cumsum_type
    seq_starts   int32 [batch] (has_seq_starts): sequence i is read from block-table column
                 seq_starts[i] // block_size on
    key_out / value_out  [sum of lengths, num_heads, head_size], cache dtypes
    The row count is the sum of `seq_lens`, which is therefore read on the host as in the reference:
    pass `seq_lens` as a CPU tensor / numpy array to avoid the device synchronisation.
    """
    import torch
    lens_host = _host_int32(seq_lens)
    (kshape, _), (vshape, _) = paged_cache_load_infer(
        key_cache, value_cache, block_tables, lens_host, seq_starts, kv_cache_cfg, is_seq_lens_cumsum_type,
        has_seq_starts)
    dev = key_cache.device

    def on_device(t):
        if t is None or (hasattr(t, "is_cuda") and t.is_cuda):
            return t
        return torch.as_tensor(np.asarray(t) if not hasattr(t, "is_cuda") else t).to(dev, non_blocking=True)
    block_tables, seq_lens, seq_starts = on_device(block_tables), on_device(seq_lens), on_device(seq_starts)
    key_out = torch.empty(kshape, dtype=key_cache.dtype, device=dev)
    value_out = torch.empty(vshape, dtype=value_cache.dtype, device=dev)
    D = _Descs()
    L = _host.lib()
    need = L.ms_custom_ops_paged_cache_load_workspace_size(D(block_tables))
    wkey = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    ws = _load_workspaces.get(wkey)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(int(need * 1.25), 1 << 16), dtype=torch.uint8, device=dev)
        _load_workspaces[wkey] = ws
    _host.check(L.ms_custom_ops_paged_cache_load(
        D(key_cache), D(value_cache), D(block_tables), D(seq_lens), D(seq_starts), int(kv_cache_cfg),
        int(bool(is_seq_lens_cumsum_type)), int(bool(has_seq_starts)), D(key_out), D(value_out),
        C.c_void_p(ws.data_ptr()), ws.numel(), _stream()))
    return key_out, value_out


# --------------------------------------------------------------------------
# fa_update
# --------------------------------------------------------------------------
def fa_update_infer(lse, local_out, fa_update_type=0, sp=1):
    """Shape / dtype of the merged output after the operator's checks; TensorSpec or real tensors."""
    D = _Descs()
    dt, nd = C.c_int32(), C.c_int32()
    shp = (C.c_int64 * _host.MS_MAX_DIMS)()
    _host.check(_host.lib().ms_custom_ops_fa_update_infer(D(lse), D(local_out), int(fa_update_type), int(sp),
                                                          C.byref(dt), C.byref(nd), shp))
    return tuple(shp[i] for i in range(nd.value)), _DT_NAMES[dt.value]


def fa_update(lse, local_out, fa_update_type=0, sp=1):
    """Merge `sp` partial attention outputs by their log-sum-exps (DECODE_UPDATE).

    lse        float32 [sp, rows]  (rows = batch * seq_len * head_num), natural logarithm
    local_out  float32 [sp, rows, head_size], head_size a multiple of 8 in [8, 512]
    returns    float32 [rows, head_size] = sum_s softmax_s(lse)[s, row] * local_out[s, row, :]
    """
    import torch
    shape, _ = fa_update_infer(lse, local_out, fa_update_type, sp)
    out = torch.empty(shape, dtype=torch.float32, device=local_out.device)
    D = _Descs()
    _host.check(_host.lib().ms_custom_ops_fa_update(D(lse), D(local_out), int(fa_update_type), int(sp), D(out),
                                                    _stream()))
    return out


def paged_attention_check_status(device=None):
    """Synchronise the current stream and raise if the last paged_attention launch on it reported
    an expired bounded wait (MSCO_ERR_TIMEOUT) or a block id outside the cache (MSCO_ERR_OOB)."""
    import torch
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    stream = torch.cuda.current_stream(device)
    ws = _workspaces.get((device.index, stream.cuda_stream))
    stream.synchronize()
    if ws is not None:
        _host.check(_host.lib().ms_custom_ops_paged_attention_status(C.c_void_p(ws.data_ptr())))
