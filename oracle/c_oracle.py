"""ctypes loader for the compiled C restatement (oracle/paged_kv_oracle.c).

TEST INFRASTRUCTURE ONLY.  Used where the numpy restatement would be too slow
(large cases) and as the timed multi-threaded CPU baseline.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpaged_kv_oracle.so")
_lib = None

_CODES = {"float16": 0, "bfloat16": 1, "int8": 2, "float32": 3}


def build(force=False):
    src = os.path.join(_HERE, "paged_kv_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libpaged_kv_oracle.so"], check=True, stdout=subprocess.DEVNULL)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        L.pko_paged_attention.restype = C.c_int
        L.pko_max_threads.restype = C.c_int
        L.pko_reshape_and_cache.restype = None
        L.pko_reshape_and_cache_quant.restype = None
        L.pko_paged_cache_load.restype = C.c_int64
        L.pko_fa_update.restype = None
        _lib = L
    return _lib


def _code(a):
    name = str(a.dtype)
    if name not in _CODES:
        raise TypeError(name)
    return _CODES[name]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def max_threads() -> int:
    return int(lib().pko_max_threads())


def paged_attention(query, key_cache, value_cache, block_tables, context_lens, scale, k_descale=None,
                    v_descale=None, k_offset=None, v_offset=None, mask=None, mask_type=0, threads=0):
    """float32 [batch, q_heads, head_dim]; same contract as paged_kv_numpy.paged_attention_golden."""
    q = np.ascontiguousarray(query)
    kc, vc = np.ascontiguousarray(key_cache), np.ascontiguousarray(value_cache)
    bt = np.ascontiguousarray(block_tables, dtype=np.int32)
    lens = np.ascontiguousarray(context_lens, dtype=np.int32).reshape(-1)
    batch, hq, d = q.shape
    nb, bs, hkv, _ = kc.shape
    f32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
    i32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.int32)
    kd, vd, ko, vo = f32(k_descale), f32(v_descale), i32(k_offset), i32(v_offset)
    m = f32(mask)
    mbs = mhs = 0
    if m is not None:
        if mask_type == 2:
            mbs, mhs = m.shape[1] * m.shape[3], m.shape[3]
        else:
            mbs, mhs = m.shape[2], 0
    out = np.empty((batch, hq, d), dtype=np.float32)
    rc = lib().pko_paged_attention(
        _p(q), _code(q), _p(kc), _p(vc), _code(kc), _p(bt), _p(lens), C.c_int(batch), C.c_int(hq), C.c_int(hkv),
        C.c_int(d), C.c_int(bs), C.c_int64(nb), C.c_int(bt.shape[1]), C.c_float(scale), _p(kd), _p(ko), _p(vd),
        _p(vo), _p(m), C.c_int64(mbs), C.c_int64(mhs), _p(out), C.c_int(threads))
    if rc != 0:
        raise RuntimeError(f"pko_paged_attention failed ({rc})")
    return out


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, threads=0, inplace=False):
    """Returns the updated caches (bit copy of rows, negative slots skipped): copies, or the
    given arrays themselves with inplace=True (contiguous arrays only)."""
    kc = key_cache if inplace else np.array(key_cache, copy=True)
    vc = None if value_cache is None else (value_cache if inplace else np.array(value_cache, copy=True))
    k = np.ascontiguousarray(key)
    v = None if value is None else np.ascontiguousarray(value)
    slot = np.ascontiguousarray(slot_mapping, dtype=np.int32).reshape(-1)
    t = slot.size
    lib().pko_reshape_and_cache(_p(k), _p(v), _p(kc), _p(vc), _p(slot), C.c_int64(t),
                                C.c_int64(k.nbytes // max(t, 1)), C.c_int64(0 if v is None else v.nbytes // max(t, 1)),
                                C.c_int(threads))
    return kc, vc


def reshape_and_cache_quant(key, value, key_cache, value_cache, slot_mapping, k_descale, v_descale,
                            k_offset=None, v_offset=None, threads=0, inplace=False):
    kc = key_cache if inplace else np.array(key_cache, copy=True)
    vc = None if value_cache is None else (value_cache if inplace else np.array(value_cache, copy=True))
    k = np.ascontiguousarray(key)
    v = None if value is None else np.ascontiguousarray(value)
    slot = np.ascontiguousarray(slot_mapping, dtype=np.int32).reshape(-1)
    t = slot.size
    f32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.float32)
    i32 = lambda a: None if a is None else np.ascontiguousarray(a, dtype=np.int32)
    kd, vd, ko, vo = f32(k_descale), f32(v_descale), i32(k_offset), i32(v_offset)
    lib().pko_reshape_and_cache_quant(_p(k), _p(v), C.c_int(_code(k)), _p(kc), _p(vc), _p(slot), C.c_int64(t),
                                      C.c_int64(k.size // max(t, 1)), C.c_int64(0 if v is None else v.size // max(t, 1)),
                                      _p(kd), _p(ko), _p(vd), _p(vo), C.c_int(threads))
    return kc, vc


def paged_cache_load(key_cache, value_cache, block_tables, seq_lens, seq_starts=None, seq_lens_cumsum=False,
                     threads=0):
    """Same contract as paged_kv_numpy.paged_cache_load_golden (ND layout), sequences over threads."""
    kc, vc = np.ascontiguousarray(key_cache), np.ascontiguousarray(value_cache)
    bt = np.ascontiguousarray(block_tables, dtype=np.int32)
    lens = np.ascontiguousarray(seq_lens, dtype=np.int32).reshape(-1)
    st = None if seq_starts is None else np.ascontiguousarray(seq_starts, dtype=np.int32)
    total = int(lens[-1]) if seq_lens_cumsum else int(lens.sum())
    ko = np.empty((total,) + kc.shape[2:], dtype=kc.dtype)
    vo = np.empty((total,) + vc.shape[2:], dtype=vc.dtype)
    rc = lib().pko_paged_cache_load(
        _p(kc), _p(vc), _p(bt), _p(lens), _p(st), _p(ko), _p(vo), C.c_int(bt.shape[0]), C.c_int(bt.shape[1]),
        C.c_int(kc.shape[1]), C.c_int64(kc[0, 0].nbytes), C.c_int64(vc[0, 0].nbytes), C.c_int64(total),
        C.c_int(1 if seq_lens_cumsum else 0), C.c_int(threads))
    if rc < 0:
        raise RuntimeError("pko_paged_cache_load failed")
    return ko, vo


def fa_update(lse, local_out, threads=0):
    """Same contract as paged_kv_numpy.fa_update_golden: float32 [rows, head_size]."""
    l = np.ascontiguousarray(lse, dtype=np.float32)
    x = np.ascontiguousarray(local_out, dtype=np.float32)
    sp, rows, hd = x.shape
    out = np.empty((rows, hd), dtype=np.float32)
    lib().pko_fa_update(_p(l), _p(x), _p(out), C.c_int64(rows), C.c_int(hd), C.c_int(sp), C.c_int(threads))
    return out

