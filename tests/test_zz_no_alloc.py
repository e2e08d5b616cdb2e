"""GPU: the scratch-free launch (msco_paged_attention_launch_static) gives the same result as the
ordinary launch.

Some users of this library cannot allocate device memory at the moment they launch: a custom-op
callback inside a framework may only touch the tensors it was handed, a serving loop may have
frozen all allocation after start-up, a thin foreign-language binding may have no allocator at
all.  For them the library carries a fixed scratch array in its device image.  This test calls
that entry point through the C ABI, twice in a row (the array is shared by all calls and keeps
the previous call's contents, so the second call also proves nothing stale is read), and
compares with the caller-workspace entry point.  It lives in a file that pytest collects last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from ms_custom_ops_b200 import _abi, kernels, workloads
from oracle import paged_kv_numpy as oracle
from tests.helpers import assert_close, to_dev, to_np

pytestmark = pytest.mark.gpu


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _case(spec_n, scale, seed_shift=0):
    spec = workloads.config_spec(spec_n, scale)
    if spec.kv_int8:  # long enough for several int8 splits (contexts of up to 4096 int8 tokens are one item)
        spec.batch, spec.len_lo, spec.len_hi = 10, 3000, 9000
    spec.seed += seed_shift
    c = workloads.decode_case(spec)
    dev = {k: to_dev(c[k]) for k in ("query", "key_cache", "value_cache", "block_tables")}
    dev["k_descale"], dev["v_descale"] = to_dev(c["k_descale"]), to_dev(c["v_descale"])
    return spec, c, dev


def _launch_static(plan, d, out):
    L = _abi.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _abi.check(L.msco_paged_attention_launch_static(
        plan.handle, _p(d["query"]), _p(d["key_cache"]), _p(d["value_cache"]), _p(d["block_tables"]),
        _p(d["k_descale"]), None, _p(d["v_descale"]), None, None, _p(out), stream))
    torch.cuda.current_stream().synchronize()
    _abi.check(L.msco_paged_attention_status_static(plan.handle))


@pytest.mark.parametrize("n,scale", [(2, 0.125), (3, 0.4)])
def test_static_scratch_launch_matches_workspace_launch_twice(n, scale):
    results = []
    for rep in range(2):  # two different problems back to back through the same built-in scratch
        spec, c, d = _case(n, scale, seed_shift=rep)
        lens = [int(x) for x in c["context_lens"]]
        quant = 1 if spec.kv_int8 else 0
        desc = kernels.make_pa_desc(d["query"], d["key_cache"], d["block_tables"], c["qk_scale"], quant)
        plan = _abi.PaPlan(desc, lens)
        assert plan.info().partials > 0, "the case must exercise the split partials in the scratch"
        assert plan.workspace_bytes <= _abi.STATIC_SCRATCH_BYTES
        # existing entry point, caller-provided workspace
        ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
        ref = torch.empty_like(d["query"])
        kernels.pa_launch(plan, d["query"], d["key_cache"], d["value_cache"], d["block_tables"], ref, ws,
                          d["k_descale"], None, d["v_descale"], None)
        kernels.pa_status(plan, ws)
        # new entry point, no workspace argument at all
        out = torch.full_like(d["query"], float("nan"))
        _launch_static(plan, d, out)
        a, b = to_np(out).astype(np.float32), to_np(ref).astype(np.float32)
        assert np.all(np.isfinite(a))
        tol = 2e-2 if spec.kv_int8 else 1e-2
        assert np.all(np.abs(a - b) <= tol + tol * np.abs(b))
        # same kernels, same plan, same split order: the two results are in fact identical
        assert np.array_equal(to_np(out).view(np.uint16), to_np(ref).view(np.uint16))
        # and, directly, against the oracle of the reference's golden
        g = oracle.paged_attention_golden(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                          c["context_lens"], c["qk_scale"], c["k_descale"], c["v_descale"])
        assert_close(a, g, tol, f"static-scratch launch, {spec.name}")
        results.append(a)
        plan.close()
    assert not np.array_equal(results[0], results[1])


def test_static_scratch_rejects_plans_that_do_not_fit():
    # 40 sequences of 64K tokens at 64 q heads need far more than the built-in 16 MiB
    desc = _abi.MscoPaDesc()
    desc.q_dtype = desc.kv_dtype = _abi.DTYPE_BF16
    desc.num_q_heads, desc.num_kv_heads, desc.head_dim, desc.block_size = 64, 8, 128, 128
    desc.num_blocks, desc.max_blocks_per_seq, desc.qk_scale = 1 << 16, 512, 0.1
    plan = _abi.PaPlan(desc, [65536] * 40)
    assert plan.workspace_bytes > _abi.STATIC_SCRATCH_BYTES
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = _abi.lib().msco_paged_attention_launch_static(
        plan.handle, _p(dummy), _p(dummy), _p(dummy), _p(dummy), None, None, None, None, None, _p(dummy), None)
    assert rc == _abi.ERR_INVALID_ARG
    msg = _abi.lib().msco_last_error().decode()
    assert str(plan.workspace_bytes) in msg and str(_abi.STATIC_SCRATCH_BYTES) in msg
    plan.close()
