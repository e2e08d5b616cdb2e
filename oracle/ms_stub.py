"""Minimal stand-in for the `mindspore` and `ms_custom_ops` modules.

TEST INFRASTRUCTURE ONLY.  Lets the reference's own system-test modules
(tests/st/test_custom_paged_attention.py, tests/st/test_custom_reshape_and_cache.py)
be *imported* on a machine without MindSpore so that their numpy golden
functions can be called to produce fixtures.  Nothing here computes anything:
dtype sentinels, a `Tensor` that round-trips numpy arrays (bf16 through
ml_dtypes), and empty shells for the names the modules touch at import time.
"""
from __future__ import annotations

import sys
import types

import ml_dtypes
import numpy as np


class _DType:
    def __init__(self, name, np_dtype):
        self.name = name
        self.np_dtype = np_dtype

    def __repr__(self):
        return f"mindspore.{self.name}"


def install():
    """Register the fake modules in sys.modules (idempotent)."""
    if "mindspore" in sys.modules and getattr(sys.modules["mindspore"], "_is_stub", False):
        return sys.modules["mindspore"]

    ms = types.ModuleType("mindspore")
    ms._is_stub = True
    ms.float16 = _DType("float16", np.float16)
    ms.bfloat16 = _DType("bfloat16", ml_dtypes.bfloat16)
    ms.float32 = _DType("float32", np.float32)
    ms.int8 = _DType("int8", np.int8)
    ms.int32 = _DType("int32", np.int32)
    ms.int64 = _DType("int64", np.int64)
    ms.bool_ = _DType("bool_", np.bool_)
    ms.dtype = _DType

    class Tensor:
        def __init__(self, data, dtype=None):
            arr = np.asarray(data)
            if dtype is not None:
                arr = arr.astype(dtype.np_dtype)
            self._a = arr
            self.dtype = dtype
            self.shape = arr.shape

        def asnumpy(self):
            # MindSpore returns float32 values on the bf16 grid for bf16 tensors
            if self._a.dtype == ml_dtypes.bfloat16:
                return self._a.astype(np.float32)
            return self._a

        def float(self):
            return Tensor(self._a.astype(np.float32), ms.float32)

        def astype(self, dtype):
            return Tensor(self._a, dtype)

    ms.Tensor = Tensor

    ctx = types.ModuleType("mindspore.context")
    ctx.GRAPH_MODE, ctx.PYNATIVE_MODE = 0, 1
    ctx._state = {"mode": 1}
    ctx.set_context = lambda **kw: ctx._state.update(kw)
    ctx.get_context = lambda k: ctx._state.get(k)
    ms.context = ctx
    ms.set_context = ctx.set_context
    ms.get_context = ctx.get_context
    ms.GRAPH_MODE, ms.PYNATIVE_MODE = 0, 1
    ms.set_seed = lambda s: None
    ms.set_device = lambda *a, **k: None

    nn = types.ModuleType("mindspore.nn")

    class Cell:
        def __init__(self, *a, **k):
            pass

        def __call__(self, *a, **k):
            return self.construct(*a, **k)

        def set_inputs(self, *a, **k):
            pass

    nn.Cell = Cell
    ms.nn = nn
    ops = types.ModuleType("mindspore.ops")
    ms.ops = ops
    ms.mint = types.ModuleType("mindspore.mint")
    ms.jit = lambda fn=None, **k: fn if fn is not None else (lambda f: f)

    common = types.ModuleType("mindspore.common")
    api = types.ModuleType("mindspore.common.api")
    api.jit = lambda fn=None, **k: fn if fn is not None else (lambda f: f)
    npd = types.ModuleType("mindspore.common.np_dtype")
    npd.bfloat16 = ml_dtypes.bfloat16
    common.api, common.np_dtype = api, npd
    ms.common = common

    mods = {
        "mindspore": ms, "mindspore.context": ctx, "mindspore.nn": nn, "mindspore.ops": ops,
        "mindspore.mint": ms.mint, "mindspore.common": common,
        "mindspore.common.api": api, "mindspore.common.np_dtype": npd,
        "ms_custom_ops": types.ModuleType("ms_custom_ops"),
    }
    sys.modules.update(mods)
    return ms
