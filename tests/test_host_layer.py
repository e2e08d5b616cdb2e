"""CPU: the C-ABI libraries load and export every declared symbol; the operator layer
validates like the reference; planning is a pure function of each sequence's length."""
import ctypes
import os
import re

import numpy as np
import pytest
import yaml

import ms_custom_ops_b200 as ops
from ms_custom_ops_b200 import TensorSpec as T
from ms_custom_ops_b200 import _abi, _host

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:msco|ms_custom_ops)_[a-z0-9_]+)\s*\(", text)))


@pytest.mark.parametrize("header,loader,listed", [("msco_b200.h", _abi.lib, _abi.EXPORTS),
                                                  ("ms_custom_ops_c.h", _host.lib, _host.EXPORTS)])
def test_library_exports_every_declared_symbol(header, loader, listed):
    names = _declared(header)
    assert sorted(listed) == names, "the Python binding list and the header disagree"
    lib = loader()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/{header} but not exported"
    assert _abi.lib().msco_version() == 1


def test_registered_signatures_match_the_yaml_definitions():
    reg = ops.registered_ops()
    for op, sub in (("reshape_and_cache", "reshape_and_cache"), ("paged_attention", "paged_attention"),
                    ("paged_cache_load", "paged_cache_load"), ("fa_update", "fa_update"),
                    ("reshape_and_cache_npd", "reshape_and_cache_npd")):
        y = yaml.safe_load(open(os.path.join(ROOT, "ms_custom_ops_b200", "ops", "c_api", sub, op + "_op.yaml")))
        parts = []
        for name, spec in y[op]["args"].items():
            default = spec.get("default")
            default = {"false": False, "true": True}.get(default, default) if isinstance(default, str) else default
            parts.append(name if "default" not in spec else f"{name}={default}")
        assert reg[op] == f"{op}({', '.join(parts)})"
    # and the Python functions expose the same names, order and defaults
    import inspect
    for op in ("reshape_and_cache", "paged_attention", "paged_cache_load", "fa_update", "reshape_and_cache_npd"):
        sig = inspect.signature(getattr(ops, op))
        got = ", ".join(n if p.default is inspect._empty else
                        f"{n}={p.default!r}" if isinstance(p.default, str) else f"{n}={p.default}"
                        for n, p in sig.parameters.items())
        assert reg[op] == f"{op}({got})"


Q = T((4, 32, 128), "float16")
KC = T((64, 128, 8, 128), "float16")
KC8 = T((64, 128, 8, 128), "int8")
BT = T((4, 8), "int32")
LENS = [100, 200, 1024, 5]
OKW = dict(q_head_num=32, kv_head_num=8, qk_scale=0.088)


def test_infer_returns_query_shape_and_dtype():
    assert ops.paged_attention_infer(Q, KC, KC, BT, LENS, **OKW) == ((4, 32, 128), "float16")
    qb = T((4, 32, 128), "bfloat16")
    sc, of = T((1024,), "float32"), T((1024,), "int32")
    assert ops.paged_attention_infer(qb, KC8, KC8, BT, LENS, quant_type=1, k_descale=sc, v_descale=sc, k_offset=of,
                                     v_offset=of, has_quant_offset=True, **OKW)[1] == "bfloat16"


@pytest.mark.parametrize("kw,exc,frag", [
    (dict(q_head_num=0), ValueError, "q_head_num should be greater than 0"),
    (dict(q_head_num=32, kv_head_num=-1), ValueError, "kv_head_num should be greater than or equal to 0"),
    (dict(q_head_num=32, kv_head_num=5), ValueError, "must be divisible by kv_head_num"),
    (dict(q_head_num=32, kv_head_num=8, scale_type=2), ValueError, "scale_type is invalid"),
    (dict(q_head_num=32, kv_head_num=8, scale_type=1, quant_type=1), ValueError, "scale type logn"),
    (dict(q_head_num=32, kv_head_num=8, mla_v_dim=577), ValueError, "[0, 576]"),
    (dict(q_head_num=32, kv_head_num=8, input_layout=2), ValueError, "input layout should be"),
    (dict(q_head_num=32, kv_head_num=8, calc_type=2), ValueError, "calc_type should be"),
    (dict(q_head_num=32, kv_head_num=8, calc_type=1, quant_type=1), ValueError, "MTP scene"),
    (dict(q_head_num=32, kv_head_num=8, input_layout=1, scale_type=1), ValueError, "BNSD"),
    (dict(q_head_num=32, kv_head_num=8, compress_type=3), ValueError, "compress type should not be 3"),
    (dict(q_head_num=32, kv_head_num=8, compress_type=2), ValueError, "mask type should not be"),
    (dict(q_head_num=32, kv_head_num=8, quant_type=2), ValueError, "out_data_type must be"),
    (dict(q_head_num=32, kv_head_num=8, quant_type=3, out_data_type=1, has_quant_offset=True), ValueError,
     "has_quant_offset must be false"),
    (dict(q_head_num=32, kv_head_num=8, mla_v_dim=64), ValueError, "kv_head_num should be 1"),
    (dict(q_head_num=32, kv_head_num=8, quant_type=1), ValueError, "key cache dtype must be int8"),
    (dict(q_head_num=16, kv_head_num=8), ValueError, "must equal query's head dimension"),
    (dict(q_head_num=32, kv_head_num=4), ValueError, "must equal the head_num of key_cache"),
    (dict(q_head_num=32, kv_head_num=8, mask_type=4), ValueError, "MASK_FREE is only supported on 310P"),
    (dict(q_head_num=32, kv_head_num=8, mask_type=1), ValueError, "attn_mask must be provided"),
    # accepted by the reference, not built here
    (dict(q_head_num=32, kv_head_num=8, calc_type=1), ops.MscoError, "q_seq_lens must be provided"),
    (dict(q_head_num=32, kv_head_num=8, calc_type=1, q_seq_lens=[1, 1, 1, 1], mask_type=1,
          attn_mask=T((4, 1, 1024), "float16")), ops.UnsupportedOnB200, "prefill-shaped"),
    (dict(q_head_num=32, kv_head_num=8, mask_type=3), ops.UnsupportedOnB200, "mask_type=3"),
    (dict(q_head_num=32, kv_head_num=8, scale_type=1), ops.UnsupportedOnB200, "LogN"),
    (dict(q_head_num=32, kv_head_num=8, input_layout=1, quant_type=1), ValueError, "BNSD"),
    (dict(q_head_num=32, kv_head_num=8, compress_type=1), ops.UnsupportedOnB200, "compress_type"),
    (dict(q_head_num=32, kv_head_num=8, batch_run_status_enable=True), ops.UnsupportedOnB200, "batch_run_status"),
])
def test_parameter_rules_raise_like_the_reference(kw, exc, frag):
    with pytest.raises(exc) as e:
        ops.paged_attention_infer(Q, KC, KC, BT, LENS, **kw)
    assert frag in str(e.value)


def test_shape_and_type_rules():
    bad_rank = T((4, 32 * 128), "float16")
    with pytest.raises(ValueError, match="rank of query must be 3"):
        ops.paged_attention_infer(bad_rank, KC, KC, BT, LENS, **OKW)
    with pytest.raises(ValueError, match="rank of key_cache must be 4"):
        ops.paged_attention_infer(Q, T((64, 128, 1024), "float16"), KC, BT, LENS, **OKW)
    with pytest.raises(ValueError, match="rank of block table must be 2"):
        ops.paged_attention_infer(Q, KC, KC, T((32,), "int32"), LENS, **OKW)
    with pytest.raises(ValueError, match="num_blocks of key_cache and value_cache must be same"):
        ops.paged_attention_infer(Q, KC, T((32, 128, 8, 128), "float16"), BT, LENS, **OKW)
    with pytest.raises(ValueError, match="head_size of key_cache and query must be same"):
        ops.paged_attention_infer(T((4, 32, 64), "float16"), KC, KC, BT, LENS, **OKW)
    with pytest.raises(ValueError, match=r"block_size \* head_size must be <= 128 \* 128"):
        big = T((64, 256, 8, 128), "float16")
        ops.paged_attention_infer(Q, big, big, BT, LENS, **OKW)
    with pytest.raises(ValueError, match="query dtype must be float16/bfloat16"):
        ops.paged_attention_infer(T((4, 32, 128), "float32"), KC, KC, BT, LENS, **OKW)
    with pytest.raises(ValueError, match="cache dtype must equal the query dtype"):
        ops.paged_attention_infer(Q, T((64, 128, 8, 128), "bfloat16"), T((64, 128, 8, 128), "bfloat16"), BT, LENS, **OKW)
    with pytest.raises(ValueError, match="context_lens has 3 entries"):
        ops.paged_attention_infer(Q, KC, KC, BT, [1, 2, 3], **OKW)
    with pytest.raises(ValueError, match="exceeds the block table"):
        ops.paged_attention_workspace_size(Q, KC, KC, BT, [1, 2, 3, 1025], **OKW)
    with pytest.raises(ops.UnsupportedOnB200, match="FRACTAL_NZ"):
        ops.paged_attention_infer(T((4, 4096), "float16"), T((64, 128, 1024), "float16"),
                                  T((64, 128, 1024), "float16"), BT, LENS, input_format=1, **OKW)
    # context_lens must live on the host, as in the reference
    with pytest.raises(ops.MscoError, match="must be a CPU tensor"):
        ops.paged_attention_infer(Q, KC, KC, BT, T((4,), "int32", on_host=False), **OKW)
    with pytest.raises(ops.MscoError, match="must be Int32"):
        ops.paged_attention_infer(Q, KC, KC, BT, np.array([1, 2, 3, 4], dtype=np.int64), **OKW)


def test_multi_token_queries_infer_and_validation():
    # calc_type = 1: query holds sum(q_seq_lens) tokens, block tables / context_lens one row per sequence
    q6 = T((6, 32, 128), "float16")
    mtp = dict(OKW, calc_type=1, q_seq_lens=[2, 1, 3, 0])
    assert ops.paged_attention_infer(q6, KC, KC, BT, LENS, **mtp) == ((6, 32, 128), "float16")
    spec = dict(mtp, mask_type=3, attn_mask=T((6, 1024), "float16"))
    assert ops.paged_attention_infer(q6, KC, KC, BT, LENS, **spec)[0] == (6, 32, 128)
    with pytest.raises(ValueError, match="sum to 6 but query holds 4"):
        ops.paged_attention_infer(Q, KC, KC, BT, LENS, **mtp)
    with pytest.raises(ValueError, match="q_seq_lens has 3 entries"):
        ops.paged_attention_infer(q6, KC, KC, BT, LENS, **dict(mtp, q_seq_lens=[2, 2, 2]))
    with pytest.raises(ValueError, match="must not be negative"):
        ops.paged_attention_infer(q6, KC, KC, BT, LENS, **dict(mtp, q_seq_lens=[7, -1, 0, 0]))
    with pytest.raises(ValueError, match="SPEC mask must have shape"):
        ops.paged_attention_infer(q6, KC, KC, BT, LENS, **dict(spec, attn_mask=T((4, 1024), "float16")))
    with pytest.raises(ValueError, match="the mask covers 512"):
        ops.paged_attention_infer(q6, KC, KC, BT, LENS, **dict(spec, attn_mask=T((6, 512), "float16")))
    with pytest.raises(ValueError, match="block_tables has 5 rows"):
        ops.paged_attention_infer(q6, KC, KC, T((5, 8), "int32"), LENS, **mtp)
    # head_dim 128: the tokens of a sequence are stacked into the q rows of the work items, the plan of one
    # token per sequence is the decode plan
    plain = ops.paged_attention_workspace_size(Q, KC, KC, BT, LENS, **OKW)
    one_each = ops.paged_attention_workspace_size(Q, KC, KC, BT, LENS, **dict(OKW, calc_type=1, q_seq_lens=[1] * 4))
    assert one_each == plain
    # a head_dim the TMA kernel does not serve: one decode row per token, and the workspace also holds one
    # block-table row and one index per query token
    q40, kc40 = T((4, 32, 40), "float16"), T((64, 128, 8, 40), "float16")
    plain = ops.paged_attention_workspace_size(q40, kc40, kc40, BT, LENS, **OKW)
    one_each = ops.paged_attention_workspace_size(q40, kc40, kc40, BT, LENS, **dict(OKW, calc_type=1, q_seq_lens=[1] * 4))
    assert one_each == (plain + 255) // 256 * 256 + 256 + 256


def test_paged_cache_load_infer_and_validation_without_a_gpu():
    kc, vc, bt = T((128, 128, 16, 144), "bfloat16"), T((128, 128, 16, 128), "int8"), T((16, 12), "int32")
    lens = np.arange(1, 17, dtype=np.int32)
    # row count = sum of the lengths, or the last running sum; -1 when the lengths are not on the host
    assert ops.paged_cache_load_infer(kc, vc, bt, lens) == (((136, 16, 144), "bfloat16"), ((136, 16, 128), "int8"))
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    starts = T((16,), "int32")
    assert ops.paged_cache_load_infer(kc, vc, bt, cu, starts, 0, True, True)[0] == ((136, 16, 144), "bfloat16")
    assert ops.paged_cache_load_infer(kc, vc, bt, T((16,), "int32"))[0][0][0] == -1
    with pytest.raises(ops.MscoError, match="seq_lens dtype must be int32"):
        ops.paged_cache_load_infer(kc, vc, bt, lens.astype(np.int64))
    with pytest.raises(ops.UnsupportedOnB200, match="FRACTAL_NZ"):
        ops.paged_cache_load_infer(kc, vc, bt, lens, None, 1)
    with pytest.raises(ValueError, match="kv_cache_cfg must be 0"):
        ops.paged_cache_load_infer(kc, vc, bt, lens, None, 5)
    with pytest.raises(ValueError, match="exactly when has_seq_starts"):
        ops.paged_cache_load_infer(kc, vc, bt, lens, starts, 0, False, False)
    with pytest.raises(ValueError, match="17 elements"):
        ops.paged_cache_load_infer(kc, vc, bt, lens, None, 0, True, False)
    with pytest.raises(ValueError, match="batch = 16"):
        ops.paged_cache_load_infer(kc, vc, bt, lens, T((15,), "int32"), 0, False, True)
    with pytest.raises(ValueError, match="rank 4"):
        ops.paged_cache_load_infer(T((128, 128, 2304), "bfloat16"), vc, bt, lens)
    with pytest.raises(ValueError, match="agree in num_blocks"):
        ops.paged_cache_load_infer(kc, T((128, 64, 16, 128), "int8"), bt, lens)
    with pytest.raises(TypeError, match="Float16/BFloat16/Int8"):
        ops.paged_cache_load_infer(T((128, 128, 16, 144), "float32"), vc, bt, lens)
    with pytest.raises(TypeError, match="block_tables must be Int32"):
        ops.paged_cache_load_infer(kc, vc, T((16, 12), "int64"), lens)
    # the workspace holds one row offset per (sequence, block) pair plus one per sequence
    L, D = _host.lib(), ops._Descs()
    assert L.ms_custom_ops_paged_cache_load_workspace_size(D(bt)) == (16 + 16 + 16 * 12) * 4
    assert _abi.lib().msco_paged_cache_load_workspace_bytes(16, 12) == (16 + 16 + 16 * 12) * 4
    # zero-sized inputs are a successful no-op (no CUDA call is made)
    assert L.ms_custom_ops_paged_cache_load(D(kc), D(vc), D(T((0, 12), "int32")), D(T((0,), "int32")), None, 0, 0, 0,
                                            D(T((0, 16, 144), "bfloat16")), D(T((0, 16, 128), "int8")), None, 0,
                                            None) == 0


def test_fa_update_infer_and_validation_without_a_gpu():
    assert ops.fa_update_infer(T((3, 13000), "float32"), T((3, 13000, 128), "float32"), 0, 3) == ((13000, 128), "float32")
    with pytest.raises(ValueError, match="local_out dim must be 3, but got : 2"):
        ops.fa_update_infer(T((3, 10), "float32"), T((3, 80), "float32"), 0, 3)
    for hd in (4, 12, 520):
        with pytest.raises(ValueError, match="head_size must be in range \\[8, 512\\] and be the multiple of 8"):
            ops.fa_update_infer(T((3, 10), "float32"), T((3, 10, hd), "float32"), 0, 3)
    with pytest.raises(ValueError, match="fa_update_type must be 0"):
        ops.fa_update_infer(T((3, 10), "float32"), T((3, 10, 8), "float32"), 2, 3)
    with pytest.raises(ValueError, match="sp must be in range"):
        ops.fa_update_infer(T((9, 10), "float32"), T((9, 10, 8), "float32"), 0, 9)
    with pytest.raises(ValueError, match="3 partitions but sp is 2"):
        ops.fa_update_infer(T((3, 10), "float32"), T((3, 10, 8), "float32"), 0, 2)
    with pytest.raises(ValueError, match="lse must be"):
        ops.fa_update_infer(T((3, 11), "float32"), T((3, 10, 8), "float32"), 0, 3)
    with pytest.raises(TypeError, match="must be Float32"):
        ops.fa_update_infer(T((3, 10), "float16"), T((3, 10, 8), "float32"), 0, 3)


def test_reshape_and_cache_validation_without_a_gpu():
    L = _host.lib()
    D = ops._Descs()
    key, cache, slot = T((39, 512), "float16"), T((20, 64, 16, 32), "float16"), T((39,), "int32")

    def call(*a, mode=0):
        return L.ms_custom_ops_reshape_and_cache(*[D(x) for x in a], mode, 0, None)
    with pytest.raises(ops.UnsupportedOnB200, match="FRACTAL_NZ"):
        _host.check(call(key, None, cache, None, slot, mode=1))
    with pytest.raises(ValueError, match="cache_mode must be 0"):
        _host.check(call(key, None, cache, None, slot, mode=7))
    with pytest.raises(TypeError, match="same dtype"):
        _host.check(call(key, None, T((20, 64, 16, 32), "bfloat16"), None, slot))
    with pytest.raises(ValueError, match="provided together"):
        _host.check(call(key, key, cache, None, slot))
    with pytest.raises(ValueError, match="slot_mapping has"):
        _host.check(call(key, None, cache, None, T((40,), "int32")))
    with pytest.raises(ValueError, match="hidden size"):
        _host.check(call(T((39, 256), "float16"), None, cache, None, slot))
    with pytest.raises(TypeError, match="slot_mapping must be Int32"):
        _host.check(call(key, None, cache, None, T((39,), "int64")))
    # zero-sized inputs are a successful no-op (no CUDA call is made)
    assert call(T((0, 512), "float16"), None, cache, None, T((0,), "int32")) == 0


def _plan(lens, hq=32, hkv=8, d=128, bs=128, kv="bfloat16", kernel=0, mask=0, max_blocks=None):
    desc = _abi.MscoPaDesc()
    desc.q_dtype = _abi.DTYPE_BF16
    desc.kv_dtype = {"bfloat16": _abi.DTYPE_BF16, "int8": _abi.DTYPE_I8}[kv]
    desc.quant_type = 1 if kv == "int8" else 0
    desc.num_q_heads, desc.num_kv_heads, desc.head_dim, desc.block_size = hq, hkv, d, bs
    desc.num_blocks = 1 << 20
    desc.max_blocks_per_seq = max_blocks or (max(list(lens) + [1]) + bs - 1) // bs
    desc.qk_scale = 0.1
    desc.kernel = kernel
    desc.mask_type = mask
    desc.mask_dtype = _abi.DTYPE_F32
    return _abi.PaPlan(desc, lens)


def test_split_rule_depends_on_the_sequence_only():
    g = _abi.lib().msco_paged_attention_split_tokens
    f = lambda n: g(n, _abi.DTYPE_BF16)
    assert [f(n) for n in (1, 512, 513, 16384, 16385, 65536, 65537, 131072)] == [512] * 4 + [1024] * 2 + [2048] * 2
    assert [g(n, _abi.DTYPE_I8) for n in (1, 4096, 4097, 16384, 16385, 65537)] == [4096] * 2 + [2048] * 4
    lens = [5000, 300, 0, 70000, 512, 513]
    info = _plan(lens).info()
    splits = [(n + f(n) - 1) // f(n) if n else 0 for n in lens]
    assert info.max_splits == max(splits) == 35
    assert info.partials == sum(s for s in splits if s > 1)
    assert info.work_items == sum(splits) * 8
    assert info.kv_tokens == sum(lens)
    assert info.kernel == 2 and info.rows_per_item == 8 and info.grid == 148
    # per-sequence split counts do not change with the batch they are planned in
    alone = _plan([5000]).info()
    assert alone.partials == splits[0] and alone.work_items == splits[0] * 8


def test_kernel_selection_and_workspace():
    assert _plan([100], hq=64, hkv=8).info().rows_per_item == 8
    assert _plan([100], hq=128, hkv=8).info().rows_per_item == 16
    wide = _plan([100], hq=24 * 8, hkv=8).info()      # 24 q rows per kv head -> two 16-row items
    assert wide.rows_per_item == 16 and wide.work_items == 16
    assert _plan([100], d=64).info().kernel == 2       # head_dim 64 / 128 / 256 (16-bit cache): TMA kernel
    assert _plan([100], d=256, bs=64).info().kernel == 2
    assert _plan([100], d=256, bs=64, hq=128).info().rows_per_item == 8   # head_dim 256: 8 q rows per item
    assert _plan([100], d=256, bs=128).info().kernel == 1   # a tile of the head_dim 256 variant holds 64 tokens
    assert _plan([100], d=32).info().kernel == 1       # every other head_dim -> general kernel
    assert _plan([100], d=64, kv="int8").info().kernel == 1   # int8 cache: head_dim 128 only
    assert _plan([100], bs=48).info().kernel == 1
    assert _plan([100], mask=1).info().kernel == 2      # additive masks run in the TMA kernel too
    assert _plan([100], d=64, mask=2).info().kernel == 2
    assert _plan([100], kv="int8").info().kernel == 2
    with pytest.raises(_abi.MscoError):
        _plan([100], d=32, kernel=2)
    p = _plan([1000, 3000])
    parts = 2 + 6
    assert p.workspace_bytes >= parts * 32 * (128 + 2) * 4
    assert p.workspace_bytes % 256 == 0
    empty = _plan([0, 0])
    assert empty.info().work_items == 0 and empty.workspace_bytes % 256 == 0
    with pytest.raises(_abi.MscoError, match="negative"):
        _plan([-1])


def test_plan_cache_hits_on_repeated_lengths():
    ops.plan_cache_clear()
    for _ in range(3):
        ops.paged_attention_workspace_size(Q, KC, KC, BT, LENS, **OKW)
    ops.paged_attention_workspace_size(Q, KC, KC, BT, [100, 200, 1024, 6], **OKW)
    st = ops.plan_cache_stats()
    assert st["misses"] == 2 and st["hits"] == 2 and st["entries"] == 2
    ops.plan_cache_clear()
    assert ops.plan_cache_stats()["entries"] == 0


def test_plan_cache_entries_follow_the_misses_until_recycling_starts():
    ops.plan_cache_clear()
    for i in range(3):
        ops.paged_attention_workspace_size(Q, KC, KC, BT, [100 + i, 200, 1024, 5], **OKW)
    st = ops.plan_cache_stats()
    assert st["misses"] == 3 and st["created"] == 3 and st["recycled"] == 0
    ops.plan_cache_clear()


def test_decode_loop_replans_in_place_without_pinned_allocations():
    """Every decode step grows every length, so every step is a plan-cache miss.  After the first few
    plans of a descriptor exist, a miss re-plans one of them in place: no plan is created, no block of
    the pinned arena is requested, no slab is added (the role of the reference's TilingMemMgr,
    ops/framework/ms_kernels_internal/tiling_mem_mgr.cc:82-137)."""
    ops.plan_cache_clear()
    q, kc, bt = T((64, 32, 128), "bfloat16"), T((4096, 128, 8, 128), "bfloat16"), T((64, 80), "int32")
    rng = np.random.default_rng(0)
    lens = rng.integers(2048, 8192, 64).astype(np.int32)
    kw = dict(q_head_num=32, kv_head_num=8, qk_scale=0.088)
    for _ in range(8):   # warm-up: the first plans of this descriptor are built
        lens += 1
        ops.paged_attention_workspace_size(q, kc, kc, bt, lens, **kw)
    c0, a0 = ops.plan_cache_stats(), ops.plan_arena_stats()
    sizes = []
    for _ in range(200):
        lens += 1
        sizes.append(ops.paged_attention_workspace_size(q, kc, kc, bt, lens, **kw))
    c1, a1 = ops.plan_cache_stats(), ops.plan_arena_stats()
    assert c1["misses"] - c0["misses"] == 200 and c1["hits"] == c0["hits"]
    assert c1["recycled"] - c0["recycled"] == 200 and c1["created"] == c0["created"]
    assert a1["slabs"] == a0["slabs"] and a1["block_allocs"] == a0["block_allocs"]
    assert a1["blocks_in_use"] == a0["blocks_in_use"] and c1["entries"] == c0["entries"]
    assert sizes[-1] >= sizes[0]
    ops.plan_cache_clear()


def test_replan_equals_a_fresh_plan():
    rng = np.random.default_rng(1)
    base = rng.integers(1, 9000, 37).astype(np.int32)
    plan = _plan([int(x) for x in base], hq=32, hkv=8, max_blocks=(20000 + 127) // 128)
    for _ in range(5):
        lens = rng.integers(0, 20000, int(rng.integers(1, 300))).astype(np.int32)
        plan.replan(lens)
        fresh = _plan([int(x) for x in lens], hq=32, hkv=8, max_blocks=(20000 + 127) // 128)
        a, b = plan.info(), fresh.info()
        for f in ("kernel", "grid", "work_items", "partials", "max_splits", "rows_per_item", "kv_tokens"):
            assert getattr(a, f) == getattr(b, f), f
        assert plan.workspace_bytes == fresh.workspace_bytes
    with pytest.raises(_abi.MscoError, match="exceeds the block table"):
        plan.replan([10 ** 7])


def test_plan_arena_recycles_blocks():
    a0 = _abi.plan_arena_stats()
    plans = [_plan([100 + i] * 16) for i in range(50)]
    a1 = _abi.plan_arena_stats()
    assert a1["blocks_in_use"] - a0["blocks_in_use"] == 50
    for p in plans:
        p.close()
    again = [_plan([100 + i] * 16) for i in range(50)]
    a2 = _abi.plan_arena_stats()
    assert a2["slabs"] == a1["slabs"] and a2["blocks_in_use"] == a1["blocks_in_use"]
    for p in again:
        p.close()
    assert _abi.plan_arena_stats()["blocks_in_use"] == a0["blocks_in_use"]


def test_reshape_and_cache_infer_returns_the_placeholder_of_the_reference():
    # CustomReshapeAndCacheOpFuncImpl: the (never written) output has key's shape and dtype
    k2, c = T((4, 1024), "float16"), T((8, 128, 8, 128), "float16")
    assert ops.reshape_and_cache_infer(k2, k2, c, c, T((4,), "int32")) == ((4, 1024), "float16")
    k3 = T((2, 3, 1024), "bfloat16")
    cb = T((8, 128, 8, 128), "bfloat16")
    assert ops.reshape_and_cache_infer(k3, None, cb, None, T((6,), "int32")) == ((2, 3, 1024), "bfloat16")
    with pytest.raises(ops.UnsupportedOnB200):
        ops.reshape_and_cache_infer(k2, k2, c, c, T((4,), "int32"), cache_mode=1)
    with pytest.raises(ValueError):
        ops.reshape_and_cache_infer(k2, k2, c, c, T((5,), "int32"))


def test_bnsd_layout_is_accepted_under_the_reference_rules():
    # input_layout = 1: caches are (num_blocks, kv_heads, block_size, head_size); same checks on the same
    # quantities (reference: paged_attention_pynative.cc:119-145 for what may be combined with it)
    kc = T((64, 8, 128, 128), "float16")
    assert ops.paged_attention_infer(Q, kc, kc, BT, LENS, input_layout=1, **OKW) == ((4, 32, 128), "float16")
    assert ops.paged_attention_workspace_size(Q, kc, kc, BT, LENS, input_layout=1, **OKW) > 0
    with pytest.raises(ValueError, match="kv_head_num"):   # read as BNSD, a BSND-shaped cache has 128 heads
        ops.paged_attention_infer(Q, KC, KC, BT, LENS, input_layout=1, **OKW)
    for kw in (dict(calc_type=1), dict(compress_type=1), dict(scale_type=1)):
        with pytest.raises(ValueError, match="BNSD"):
            ops.paged_attention_infer(Q, kc, kc, BT, LENS, input_layout=1, **OKW, **kw)


def test_reshape_and_cache_npd_checks():
    k, c = T((32, 1024), "float16"), T((4, 8, 16, 128), "float16")
    sm = T((32,), "int32")
    assert ops.reshape_and_cache_npd_infer(k, k, c, c, sm, key_value_layout="TH") == (((32, 1024), "float16"),) * 2
    cb = T((4, 16, 8, 128), "float16")
    assert ops.reshape_and_cache_npd_infer(k, k, cb, cb, sm, kv_cache_layout="BSND", key_value_layout="TH")[0][0] == (32, 1024)
    with pytest.raises(ops.UnsupportedOnB200, match="NPD"):
        ops.reshape_and_cache_npd_infer(k, k, c, c, sm)    # the reference's default output layout
    with pytest.raises(ValueError, match="kv_cache_layout"):
        ops.reshape_and_cache_npd_infer(k, k, c, c, sm, kv_cache_layout="NHWC", key_value_layout="TH")
    with pytest.raises(ValueError, match="hidden sizes"):
        ops.reshape_and_cache_npd_infer(k, k, cb, cb, sm, key_value_layout="TH")  # BSND-shaped cache read as BNSD
    with pytest.raises(TypeError):
        ops.reshape_and_cache_npd_infer(k, k, c, c, T((32,), "int64"), key_value_layout="TH")


def test_stacked_query_tokens_plan():
    # 4 q heads per kv head: up to 4 consecutive tokens of a sequence share one work item (16 q rows)
    def plan(ql, lens, hq=32, hkv=8, **kw):
        desc = _plan(lens, hq=hq, hkv=hkv, **kw).desc
        return _abi.PaPlan(desc, lens, ql)
    one = _plan([3000, 100]).info()
    st = plan([4, 1], [3000, 100]).info()
    assert st.rows_per_item == 16 and st.work_items == one.work_items and st.kv_tokens == one.kv_tokens
    st = plan([9, 0], [3000, 100]).info()            # 9 tokens -> runs of 4, 4, 1; the second sequence has no query
    assert st.work_items == 3 * 6 * 8 and st.partials == (4 + 4 + 1) * 6
    st = plan([2, 2], [600, 0]).info()               # an empty context: its rows are zero-filled, no items
    assert st.work_items == 2 * 8
    assert plan([3, 3], [100, 200], hq=64, hkv=8).info().work_items == 2 * 2 * 8   # 8 q heads per kv head: 2 tokens per item
    assert plan([3], [100], hq=128, hkv=8).info().work_items == 3 * 8              # 16 per kv head: one token per item
    with pytest.raises(_abi.MscoError, match="TMA kernel"):
        plan([2], [100], d=40)


def test_decode_step_gather_validates_before_anything_is_launched():
    # the fused decode step with the exchange folded in: a NULL plan, an empty batch and a malformed
    # gather descriptor are refused on the host, before any CUDA call
    import ctypes as C
    L = _abi.lib()
    nul = C.c_void_p(None)

    def call(plan, desc):
        return L.msco_decode_step_gather(plan, *([nul] * 5), 0, *([nul] * 9), 0, nul, desc, C.c_uint32(1))

    def last_error():
        return L.msco_last_error().decode()

    d = _abi.MscoGatherDesc()
    assert call(nul, C.byref(d)) == _abi.ERR_INVALID_ARG
    empty = _plan([])
    assert call(empty.handle, C.byref(d)) == _abi.ERR_INVALID_ARG
    assert "nothing to gather" in last_error()
    plan = _plan([100, 2000])
    assert call(plan.handle, None) == _abi.ERR_INVALID_ARG
    assert "NULL gather descriptor" in last_error()
    d.world, d.rank, d.slice_bytes = 2, 2, 4096           # rank out of range
    assert call(plan.handle, C.byref(d)) == _abi.ERR_INVALID_ARG
    assert "bad rank" in last_error()
    d.rank, d.slice_bytes = 1, 4090                        # not a multiple of 16
    assert call(plan.handle, C.byref(d)) == _abi.ERR_INVALID_ARG
    d.slice_bytes = 4096                                   # ticket / status words missing
    assert call(plan.handle, C.byref(d)) == _abi.ERR_INVALID_ARG
    assert "ticket / status" in last_error()
    for p in (empty, plan):
        p.close()
