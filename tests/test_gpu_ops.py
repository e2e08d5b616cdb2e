"""GPU parity through the operator-level API (the call a user of the plugin makes)."""
import os

import numpy as np
import pytest
import torch

import ms_custom_ops_b200 as ops
from ms_custom_ops_b200 import workloads
from oracle import c_oracle
from oracle import paged_kv_numpy as oracle
from tests.golden import cases, st_inputs
from tests.helpers import assert_close, to_dev, to_np, tol_for

pytestmark = pytest.mark.gpu
GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_config1_exact_against_reference_fixture():
    """Benchmark configuration 1: cache scatter bit-exact, attention within fp16 tolerance of the
    stored output of the reference's golden."""
    fx = np.load(os.path.join(GOLDEN_DIR, "config1.npz"))
    spec = workloads.config_spec(1)
    c = workloads.decode_case(spec)
    kc, vc = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    assert ops.reshape_and_cache(to_dev(c["key"]), to_dev(c["value"]), kc, vc, to_dev(c["slot_mapping"]), 0, 0) is None
    assert cases.digest(to_np(kc)) == str(fx["sha_key_cache"])
    assert cases.digest(to_np(vc)) == str(fx["sha_value_cache"])
    out = ops.paged_attention(to_dev(c["query"]), kc, vc, to_dev(c["block_tables"]),
                              torch.from_numpy(c["context_lens"]), q_head_num=32, kv_head_num=8,
                              qk_scale=c["qk_scale"])
    ops.paged_attention_check_status()
    assert out.shape == (4, 32, 128) and out.dtype == torch.float16
    g = fx["golden"]
    assert_close(to_np(out), g, 5e-3, "config1")
    ok, detail = oracle.reference_accuracy_verdict(to_np(out), g, "float16", 32, int(c["context_lens"].max()))
    assert ok, detail
    rel_max, rel_l2 = oracle.scale_free_error(to_np(out), g)
    assert rel_l2 < 3e-3, (rel_max, rel_l2)


@pytest.mark.parametrize("name", sorted(cases.RAC_CASES))
def test_reshape_and_cache_reference_fixtures_bit_exact(name):
    c = cases.rac_case(name)
    fx = np.load(os.path.join(GOLDEN_DIR, f"rac_{name}.npz"))
    kc, vc = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    ops.reshape_and_cache(to_dev(c["key"]), to_dev(c["value"]), kc, vc, to_dev(c["slot_mapping"]), 0)
    assert cases.digest(to_np(kc)) == str(fx["sha_key_cache"])
    assert cases.digest(to_np(vc)) == str(fx["sha_value_cache"])


def test_reshape_and_cache_key_only_keyword_form():
    c = cases.rac_case("fp16_rank3")
    g, _ = oracle.reshape_and_cache_golden(c["key"], None, c["key_cache"], None, c["slot_mapping"])
    kc = to_dev(c["key_cache"])
    ops.reshape_and_cache(to_dev(c["key"]), key_cache=kc, slot_mapping=to_dev(c["slot_mapping"]), cache_mode=0)
    assert np.array_equal(to_np(kc), g)


@pytest.mark.parametrize("name", ["basic_bf16", "norm_mask_bf16", "alibi_fp16", "gqa_32to8_alibi",
                                  "int8_kv_offset", "gqa_int8_bf16", "bf16_int8_head33", "head_256_block_16"])
def test_paged_attention_operator_on_reference_cases(name):
    case = cases.st_case(name)
    v = st_inputs.operator_view(case)
    out = ops.paged_attention(
        to_dev(v["query"]), to_dev(v["key_cache"]), to_dev(v["value_cache"]), to_dev(v["block_tables"]),
        v["context_lens"], to_dev(v["mask"]), None, to_dev(v["k_descale"]), to_dev(v["k_offset"]),
        to_dev(v["v_descale"]), to_dev(v["v_offset"]), None, None, None, None, v["num_heads"], v["qk_scale"],
        v["kv_heads"], v["mask_type"], False, v["quant_type"], -1, v["has_quant_offset"])
    ops.paged_attention_check_status()
    fx = np.load(os.path.join(GOLDEN_DIR, f"pa_{name}.npz"))
    ok, detail = oracle.reference_accuracy_verdict(to_np(out), fx["golden"], case["q_dtype"], case["num_heads"],
                                                   int(max(case["context_lens"])), case["quant_type"] != 0)
    assert ok, (name, detail)


def test_decode_step_config5_scaled_scatter_then_attention():
    """Prefill-heavy scatter (5% padding slots) in both variants, then mixed decode."""
    for quant in (False, True):
        sc = workloads.scatter_case(4096, 512, dtype="bfloat16", pad_frac=0.05, seed=5, quant=quant)
        kc, vc = to_dev(sc["key_cache"]), to_dev(sc["value_cache"])
        if quant:
            gk, gv = c_oracle.reshape_and_cache_quant(sc["key"], sc["value"], sc["key_cache"], sc["value_cache"],
                                                      sc["slot_mapping"], sc["k_descale"], sc["v_descale"])
            ops.reshape_and_cache_quant(to_dev(sc["key"]), to_dev(sc["value"]), kc, vc, to_dev(sc["slot_mapping"]),
                                        to_dev(sc["k_descale"]), to_dev(sc["v_descale"]))
        else:
            gk, gv = c_oracle.reshape_and_cache(sc["key"], sc["value"], sc["key_cache"], sc["value_cache"],
                                                sc["slot_mapping"])
            ops.reshape_and_cache(to_dev(sc["key"]), to_dev(sc["value"]), kc, vc, to_dev(sc["slot_mapping"]))
        assert np.array_equal(to_np(kc).view(np.uint8), gk.view(np.uint8))
        assert np.array_equal(to_np(vc).view(np.uint8), gv.view(np.uint8))
    spec = workloads.config_spec(5, 0.25)
    c = workloads.decode_case(spec)
    kc, vc = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    ops.reshape_and_cache(to_dev(c["key"]), to_dev(c["value"]), kc, vc, to_dev(c["slot_mapping"]))
    out = ops.paged_attention(to_dev(c["query"]), kc, vc, to_dev(c["block_tables"]), c["context_lens"],
                              q_head_num=32, kv_head_num=8, qk_scale=c["qk_scale"])
    gk, gv = c_oracle.reshape_and_cache(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
    g = c_oracle.paged_attention(c["query"], gk, gv, c["block_tables"], c["context_lens"], c["qk_scale"])
    assert_close(to_np(out), g, 1e-2, "config5")
    assert oracle.scale_free_error(to_np(out), g)[1] < 1e-2


def test_operator_errors_on_the_gpu_box():
    c = cases.st_case("basic_fp16")
    q, kc, vc, bt = (to_dev(c[k]) for k in ("query", "key_cache", "value_cache", "block_tables"))
    with pytest.raises(ops.MscoError, match="must be a CPU tensor"):
        ops.paged_attention(q, kc, vc, bt, to_dev(c["context_lens"]), q_head_num=32, kv_head_num=1)
    with pytest.raises(ops.MscoError, match="must be contiguous"):
        strided = torch.zeros((4, 32, 256), dtype=q.dtype, device=q.device)[:, :, :128]
        ops.paged_attention(strided, kc, vc, bt, c["context_lens"], q_head_num=32, kv_head_num=1)
    with pytest.raises(ValueError, match="q_head_num should be greater than 0"):
        ops.paged_attention(q, kc, vc, bt, c["context_lens"])
    # a block id outside the cache is reported through the status word; the GPU stays usable
    bad = c["block_tables"].copy()
    bad[1, 0] = 64
    ops.paged_attention(q, kc, vc, to_dev(bad), c["context_lens"], q_head_num=32, kv_head_num=1, qk_scale=1.0)
    with pytest.raises(ops.MscoError) as e:
        ops.paged_attention_check_status()
    assert e.value.code == 5
    out = ops.paged_attention(q, kc, vc, bt, c["context_lens"], q_head_num=32, kv_head_num=1, qk_scale=1.0)
    ops.paged_attention_check_status()
    assert torch.isfinite(out.float()).all()


def test_plan_cache_and_length_change_between_steps():
    spec = workloads.config_spec(2, 0.06)
    c = workloads.decode_case(spec)
    q, kc, vc, bt = (to_dev(c[k]) for k in ("query", "key_cache", "value_cache", "block_tables"))
    ops.plan_cache_clear()
    lens = c["context_lens"].copy()
    outs = []
    for step in range(3):  # the same lengths twice, then one sequence one token shorter
        if step == 2:
            lens[0] -= 1
        outs.append(to_np(ops.paged_attention(q, kc, vc, bt, lens, q_head_num=32, kv_head_num=8,
                                              qk_scale=c["qk_scale"])))
    st = ops.plan_cache_stats()
    assert st["entries"] == 2 and st["hits"] >= 1
    assert np.array_equal(outs[0].view(np.uint16), outs[1].view(np.uint16))
    g = oracle.paged_attention_golden(c["query"], c["key_cache"], c["value_cache"], c["block_tables"], lens,
                                      c["qk_scale"])
    assert_close(outs[2], g, 1e-2, "after length change")


# ----------------------------------------------------------------------------
# head-major ("BNSD") cache blocks: reshape_and_cache_npd writes them, paged_attention(input_layout=1) reads them
# ----------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(cases.RACNPD_CASES))
def test_reshape_and_cache_npd_bit_exact(name):
    c = cases.racnpd_case(name)
    fx = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"racnpd_{name}.npz"))
    kc, vc = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    ok, ov = ops.reshape_and_cache_npd(to_dev(c["key"]), to_dev(c["value"]), kc, vc, to_dev(c["slot_mapping"]), None,
                                       None, None, kv_cache_layout="BNSD", key_value_layout="TH")
    assert cases.digest(to_np(kc)) == str(fx["sha_key_cache"]) and cases.digest(to_np(vc)) == str(fx["sha_value_cache"])
    assert np.array_equal(to_np(ok).view(np.uint8), c["key"].view(np.uint8))       # "TH" outputs: key / value
    assert np.array_equal(to_np(ov).view(np.uint8), c["value"].view(np.uint8))
    # the other block layout through the same operator equals reshape_and_cache
    bk, bv = oracle.reshape_and_cache_golden(c["key"], c["value"], oracle.bnsd_to_bsnd(c["key_cache"]),
                                             oracle.bnsd_to_bsnd(c["value_cache"]), c["slot_mapping"])
    kc2, vc2 = to_dev(oracle.bnsd_to_bsnd(c["key_cache"])), to_dev(oracle.bnsd_to_bsnd(c["value_cache"]))
    ops.reshape_and_cache_npd(to_dev(c["key"]), to_dev(c["value"]), kc2, vc2, to_dev(c["slot_mapping"]), None, None,
                              None, kv_cache_layout="BSND", key_value_layout="TH")
    assert np.array_equal(to_np(kc2).view(np.uint8), bk.view(np.uint8))
    assert np.array_equal(to_np(vc2).view(np.uint8), bv.view(np.uint8))
    with pytest.raises(ops.UnsupportedOnB200):
        ops.reshape_and_cache_npd(to_dev(c["key"]), to_dev(c["value"]), kc, vc, to_dev(c["slot_mapping"]), None, None, None)


@pytest.mark.parametrize("n,scale,hd,bs", [(2, 0.1, 128, 128), (1, 1.0, 128, 128), (4, 0.05, 128, 128),
                                           (2, 0.1, 64, 32), (2, 0.05, 256, 64), (2, 0.05, 80, 16)])
def test_decode_over_head_major_caches(n, scale, hd, bs):
    # one decode step on head-major caches: reshape_and_cache_npd('BNSD') then paged_attention(input_layout=1);
    # the output must equal, bit for bit, the step on the same data in the block-size-major layout
    spec = workloads.config_spec(n, scale)
    spec.head_size, spec.block_size = hd, bs
    c = workloads.decode_case(spec)
    kw = dict(q_head_num=spec.num_heads, kv_head_num=spec.kv_heads, qk_scale=c["qk_scale"])
    q, key, val = to_dev(c["query"]), to_dev(c["key"]), to_dev(c["value"])
    bt, slot = to_dev(c["block_tables"]), to_dev(c["slot_mapping"])
    kc, vc = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    ops.reshape_and_cache(key, val, kc, vc, slot)
    ref = ops.paged_attention(q, kc, vc, bt, c["context_lens"], **kw)
    hk = to_dev(np.ascontiguousarray(np.transpose(c["key_cache"], (0, 2, 1, 3))))
    hv = to_dev(np.ascontiguousarray(np.transpose(c["value_cache"], (0, 2, 1, 3))))
    ops.reshape_and_cache_npd(key, val, hk, hv, slot, None, None, None, kv_cache_layout="BNSD", key_value_layout="TH")
    out = ops.paged_attention(q, hk, hv, bt, c["context_lens"], input_layout=1, **kw)
    ops.paged_attention_check_status()
    assert torch.equal(hk.permute(0, 2, 1, 3), kc) and torch.equal(hv.permute(0, 2, 1, 3), vc)
    assert np.array_equal(to_np(out).view(np.uint16), to_np(ref).view(np.uint16))
    gk, gv = oracle.reshape_and_cache_golden(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
    g = oracle.paged_attention_golden(c["query"], gk, gv, c["block_tables"], c["context_lens"], c["qk_scale"])
    assert_close(to_np(out), g, tol_for(spec.dtype, False), f"{spec.name} head-major")
