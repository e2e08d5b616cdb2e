"""GPU parity of the CUDA kernels, called through the thin C ABI, against the CPU oracle.

reshape_and_cache is bit-exact; paged attention is checked at the decode
path's tolerances (rtol = atol = 1e-2 bf16, 5e-3 fp16, 2e-2 with int8 KV), by
the reference's own acceptance rule, and by a scale-free error bound so that a
wrong kernel cannot pass on small magnitudes alone.
"""
import os

import numpy as np
import pytest
import torch

from ms_custom_ops_b200 import _abi, kernels, workloads
from oracle import paged_kv_numpy as oracle
from tests.golden import cases, st_inputs
from tests.helpers import BF16, assert_close, to_dev, to_np, tol_for

pytestmark = pytest.mark.gpu

NP = {"float16": np.float16, "bfloat16": BF16, "int8": np.int8}


# ----------------------------------------------------------------------------
# reshape_and_cache
# ----------------------------------------------------------------------------
def _rac_inputs(dtype, kv_dim, t=39, nb=20, bs=64, heads=16, hd=32, seed=0, vhd=None):
    rng = np.random.default_rng(seed)
    vhd = vhd or hd

    def rnd(shape):
        if dtype == "int8":
            return rng.integers(-128, 128, shape, dtype=np.int8)
        return rng.random(shape, dtype=np.float32).astype(NP[dtype])
    kshape = (t, heads * hd) if kv_dim == 2 else (13, t // 13, heads * hd)
    vshape = (t, heads * vhd) if kv_dim == 2 else (13, t // 13, heads * vhd)
    slot = rng.permutation(nb * bs)[:t].astype(np.int32)
    return rnd(kshape), rnd(vshape), rnd((nb, bs, heads, hd)), rnd((nb, bs, heads, vhd)), slot


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "int8"])
@pytest.mark.parametrize("kv_dim", [2, 3])
def test_rac_reference_shapes_bit_exact(dtype, kv_dim):
    # shapes of tests/st/test_custom_reshape_and_cache.py:50-56,345-347
    k, v, kc, vc, slot = _rac_inputs(dtype, kv_dim)
    gk, gv = oracle.reshape_and_cache_golden(k, v, kc, vc, slot)
    dkc, dvc = to_dev(kc), to_dev(vc)
    kernels.rac_scatter(to_dev(k), to_dev(v), dkc, dvc, to_dev(slot))
    torch.cuda.synchronize()
    assert np.array_equal(to_np(dkc).view(np.uint8), gk.view(np.uint8))
    assert np.array_equal(to_np(dvc).view(np.uint8), gv.view(np.uint8))


def test_rac_key_only_and_different_head_dims():
    k, v, kc, vc, slot = _rac_inputs("float16", 2, vhd=48)
    gk, gv = oracle.reshape_and_cache_golden(k, v, kc, vc, slot)
    dkc, dvc = to_dev(kc), to_dev(vc)
    kernels.rac_scatter(to_dev(k), to_dev(v), dkc, dvc, to_dev(slot))
    assert np.array_equal(to_np(dkc), gk) and np.array_equal(to_np(dvc), gv)
    dkc2 = to_dev(kc)
    kernels.rac_scatter(to_dev(k), None, dkc2, None, to_dev(slot))
    assert np.array_equal(to_np(dkc2), gk)


def test_rac_unaligned_rows_use_scalar_path():
    # 7 heads x 9 dims = 63 elements: neither 16-byte rows (fp16) nor even bytes (int8)
    for dtype in ("float16", "int8"):
        k, v, kc, vc, slot = _rac_inputs(dtype, 2, heads=7, hd=9)
        gk, gv = oracle.reshape_and_cache_golden(k, v, kc, vc, slot)
        dkc, dvc = to_dev(kc), to_dev(vc)
        kernels.rac_scatter(to_dev(k), to_dev(v), dkc, dvc, to_dev(slot))
        assert np.array_equal(to_np(dkc), gk) and np.array_equal(to_np(dvc), gv)


@pytest.mark.parametrize("dtype", ["bfloat16", "int8"])
def test_rac_negative_slots_skipped_and_oob_counted(dtype):
    case = workloads.scatter_case(2048, 64, dtype="bfloat16", pad_frac=0.05, seed=11)
    k, v, kc, vc = case["key"], case["value"], case["key_cache"], case["value_cache"]
    if dtype == "int8":
        k, v, kc, vc = (a.view(np.int8)[..., ::2].copy() for a in (k, v, kc, vc))
    slot = case["slot_mapping"].copy()
    assert (slot < 0).any()
    gk, gv = oracle.reshape_and_cache_golden(k, v, kc, vc, slot)
    dkc, dvc = to_dev(kc), to_dev(vc)
    oob = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.rac_scatter(to_dev(k), to_dev(v), dkc, dvc, to_dev(slot), oob)
    assert np.array_equal(to_np(dkc).view(np.uint8), gk.view(np.uint8))
    assert np.array_equal(to_np(dvc).view(np.uint8), gv.view(np.uint8))
    assert int(oob.item()) == 0
    # slots beyond the cache are dropped and counted, never written
    slot2 = slot.copy()
    slot2[:3] = 64 * 128 + np.arange(3)
    keep = slot2.copy()
    keep[:3] = -1
    gk2, gv2 = oracle.reshape_and_cache_golden(k, v, kc, vc, keep)
    dkc, dvc = to_dev(kc), to_dev(vc)
    kernels.rac_scatter(to_dev(k), to_dev(v), dkc, dvc, to_dev(slot2), oob)
    assert np.array_equal(to_np(dkc).view(np.uint8), gk2.view(np.uint8))
    assert int(oob.item()) == 3


def test_rac_empty_inputs_are_a_no_op():
    k, v, kc, vc, slot = _rac_inputs("float16", 2)
    dkc = to_dev(kc)
    empty = torch.empty((0, k.shape[1]), dtype=torch.float16, device="cuda")
    kernels.rac_scatter(empty, empty, dkc, to_dev(vc), torch.empty(0, dtype=torch.int32, device="cuda"))
    assert np.array_equal(to_np(dkc), kc)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("offsets", [False, True])
def test_rac_quant_bit_exact(dtype, offsets):
    case = workloads.scatter_case(1500, 32, dtype=dtype, pad_frac=0.05, seed=7, quant=True)
    rng = np.random.default_rng(1)
    c = case["key"].shape[1]
    ko = rng.integers(-20, 20, c).astype(np.int32) if offsets else None
    vo = rng.integers(-20, 20, c).astype(np.int32) if offsets else None
    # exercise saturation, exact .5 ties and zeros
    case["key"][0, :8] = np.array([1e4, -1e4, 0.0, 0.5, 1.5, 2.5, -0.5, -1.5], dtype=np.float32).astype(NP[dtype])
    case["k_descale"][:8] = np.array([0.01, 0.01, 0.02, 1.0, 1.0, 1.0, 1.0, 1.0], dtype=np.float32)
    gk, gv = oracle.reshape_and_cache_quant_golden(case["key"], case["value"], case["key_cache"],
                                                   case["value_cache"], case["slot_mapping"],
                                                   case["k_descale"], case["v_descale"], ko, vo)
    dkc, dvc = to_dev(case["key_cache"]), to_dev(case["value_cache"])
    kernels.rac_scatter_quant(to_dev(case["key"]), to_dev(case["value"]), dkc, dvc, to_dev(case["slot_mapping"]),
                              to_dev(case["k_descale"]), to_dev(case["v_descale"]), to_dev(ko), to_dev(vo))
    assert np.array_equal(to_np(dkc), gk)
    assert np.array_equal(to_np(dvc), gv)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("offsets", [False, True])
def test_rac_quant_adversarial_scales_ties_and_offsets(dtype, offsets):
    # every 16-bit input value (NaN and infinities included) against scales chosen per element to land
    # the quotient on or next to a tie or an integer, scales that are zero, denormal, huge, infinite, NaN
    # or negative, powers of two, and offsets up to far beyond the int8 range: bit-exact against the
    # division of the oracle wherever the kernel's division-free test accepts and wherever it does not
    c, tokens = 1024, 512
    rng = np.random.default_rng(11)
    allv = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32) if dtype == "float16" else \
        (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)
    key = rng.choice(allv, (tokens, c)).astype(np.float32)
    val = rng.choice(allv, (tokens, c)).astype(np.float32)
    with np.errstate(all="ignore"):
        x0 = np.abs(key[0]) + 1e-3
        kd = np.empty(c, np.float32)
        kd[0::4] = x0[0::4] / (rng.integers(0, 300, c // 4) + 0.5) * (1 + rng.integers(-3, 4, c // 4) * 2.0 ** -23)
        kd[1::4] = x0[1::4] / rng.integers(1, 30000, c // 4) * (1 + rng.integers(-3, 4, c // 4) * 2.0 ** -23)
        kd[2::4] = 2.0 ** rng.integers(-20, 8, c // 4)
        kd[3::4] = rng.random(c // 4) * 0.04 + 0.01
        vd = np.exp(rng.uniform(-60, 60, c)).astype(np.float32) * rng.choice([-1.0, 1.0], c).astype(np.float32)
        odd = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, 1e-39, 3e38, 1.7e38, 1.2e-38], dtype=np.float32)
        vd[:64] = rng.choice(odd, 64)
    kd = np.nan_to_num(kd, nan=1.0, posinf=1.0, neginf=1.0).astype(np.float32)
    kd[kd == 0] = 1.0
    ko = rng.choice([0, 1, -7, 127, -128, 129, 8192, -8192, 8193, 1 << 20], c).astype(np.int32) if offsets else None
    vo = rng.integers(-200, 200, c).astype(np.int32) if offsets else None
    key, val = key.astype(NP[dtype]), val.astype(NP[dtype])
    slots = rng.permutation(tokens).astype(np.int32)
    zero = np.zeros((tokens // 128, 128, 8, 128), np.int8)
    gk, gv = oracle.reshape_and_cache_quant_golden(key, val, zero, zero.copy(), slots, kd, vd, ko, vo)
    dkc, dvc = to_dev(zero), to_dev(zero)
    kernels.rac_scatter_quant(to_dev(key), to_dev(val), dkc, dvc, to_dev(slots), to_dev(kd), to_dev(vd),
                              to_dev(ko), to_dev(vo))
    assert np.array_equal(to_np(dkc), gk)
    assert np.array_equal(to_np(dvc), gv)


# ----------------------------------------------------------------------------
# paged attention
# ----------------------------------------------------------------------------
def _run_pa(case, kernel=_abi.KERNEL_AUTO):
    v = st_inputs.operator_view(case)
    out, info = kernels.paged_attention_raw(
        to_dev(v["query"]), to_dev(v["key_cache"]), to_dev(v["value_cache"]), to_dev(v["block_tables"]),
        [int(x) for x in v["context_lens"]], v["qk_scale"], v["quant_type"],
        to_dev(v["k_descale"]), to_dev(v["k_offset"]), to_dev(v["v_descale"]), to_dev(v["v_offset"]),
        to_dev(v["mask"]), v.get("mask_type", 0), kernel)
    return to_np(out), info


def _golden(case):
    return oracle.paged_attention_golden(
        case["query"], case["key_cache"], case["value_cache"], case["block_tables"], case["context_lens"],
        case["qk_scale"], case["k_descale"], case["v_descale"], case["k_offset"], case["v_offset"],
        case["mask"], case.get("mask_type", 0))


def _check(case, out, what):
    quant = case["quant_type"] != 0
    # (1) the reference's own rule against the reference's own golden, which for bf16 is computed
    #     from the un-rounded float32 draws (tests/st/test_custom_paged_attention.py:1005-1099)
    g_ref = _golden(case)
    ok, detail = oracle.reference_accuracy_verdict(out, g_ref, case["q_dtype"], case["num_heads"],
                                                   int(max(case["context_lens"])), quant)
    assert ok, (what, detail)
    # (2) the decode path's tolerance against the float32 golden of the tensors the operator
    #     actually received (bf16 caches and masks rounded to bf16)
    g = _golden(st_inputs.operator_view(case))
    assert_close(out, g, tol_for(case["q_dtype"], quant), what)
    rel_max, rel_l2 = oracle.scale_free_error(out, g)
    assert rel_l2 < 1e-2, (what, rel_max, rel_l2)


ST_CASES = cases.ST_CASES
_st_case = cases.st_case
GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _fixture(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


@pytest.mark.parametrize("name", sorted(ST_CASES))
def test_pa_reference_case_matrix(name):
    case = _st_case(name)
    out, info = _run_pa(case)
    _check(case, out, name)
    # and against the stored output of the reference's own golden function for these inputs
    fx = _fixture("pa_" + name)
    assert str(fx["sha_query"]) == cases.digest(case["query"])
    quant = case["quant_type"] != 0
    ok, detail = oracle.reference_accuracy_verdict(out, fx["golden"], case["q_dtype"], case["num_heads"],
                                                   int(max(case["context_lens"])), quant)
    assert ok, (name, detail)


@pytest.mark.parametrize("name", ["basic_fp16", "basic_bf16", "gqa_32to8_alibi", "block_16", "varied_seqlens",
                                  "int8_kv_offset", "gqa_int8_bf16", "bf16_int8_gqa_24to2",
                                  "bf16_int8_gqa_64to32", "bf16_int8_head128", "odd_heads", "large_seqlen_bf16"])
def test_pa_both_kernels_agree_with_oracle(name):
    # the reference's shapes without the mask: both kernels against the oracle
    case = _st_case(name, mask_free=True)
    out_g, info_g = _run_pa(case, _abi.KERNEL_GENERIC)
    out_t, info_t = _run_pa(case, _abi.KERNEL_TMA)
    assert info_g.kernel == 1 and info_t.kernel == 2
    _check(case, out_g, name + "/generic")
    _check(case, out_t, name + "/tma")


@pytest.mark.parametrize("name", ["norm_mask_fp16", "norm_mask_bf16", "alibi_fp16", "alibi_bf16", "gqa_8to1_alibi",
                                  "gqa_32to8_alibi", "odd_heads", "varied_seqlens", "gqa_int8_offset",
                                  "bf16_int8_gqa_24to2", "bf16_int8_head128", "large_seqlen_bf16"])
def test_pa_masked_cases_in_both_kernels(name):
    # NORM / ALIBI additive masks: the general kernel and the TMA kernel against the oracle
    case = _st_case(name)
    assert case["mask_type"] in (1, 2)
    out_g, info_g = _run_pa(case, _abi.KERNEL_GENERIC)
    out_t, info_t = _run_pa(case, _abi.KERNEL_TMA)
    assert info_g.kernel == 1 and info_t.kernel == 2
    _check(case, out_g, name + "/generic")
    _check(case, out_t, name + "/tma")


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5])
def test_pa_benchmark_configs_scaled(n):
    # the five benchmark configurations at reduced batch / length, reshape_and_cache first
    scale = {1: 1.0, 2: 0.125, 3: 0.125, 4: 0.06, 5: 0.125}[n]
    spec = workloads.config_spec(n, scale)
    case = workloads.decode_case(spec)
    dkc, dvc = to_dev(case["key_cache"]), to_dev(case["value_cache"])
    slot = case["slot_mapping"]
    if spec.kv_int8:
        gk, gv = oracle.reshape_and_cache_quant_golden(case["key"], case["value"], case["key_cache"],
                                                       case["value_cache"], slot, case["k_descale"], case["v_descale"])
        kernels.rac_scatter_quant(to_dev(case["key"]), to_dev(case["value"]), dkc, dvc, to_dev(slot),
                                  to_dev(case["k_descale"]), to_dev(case["v_descale"]))
    else:
        gk, gv = oracle.reshape_and_cache_golden(case["key"], case["value"], case["key_cache"],
                                                 case["value_cache"], slot)
        kernels.rac_scatter(to_dev(case["key"]), to_dev(case["value"]), dkc, dvc, to_dev(slot))
    assert np.array_equal(to_np(dkc).view(np.uint8), gk.view(np.uint8))
    assert np.array_equal(to_np(dvc).view(np.uint8), gv.view(np.uint8))
    out, info = kernels.paged_attention_raw(
        to_dev(case["query"]), dkc, dvc, to_dev(case["block_tables"]), list(case["context_lens"]),
        case["qk_scale"], 1 if spec.kv_int8 else 0, to_dev(case["k_descale"]), None, to_dev(case["v_descale"]), None)
    assert info.kernel == 2
    g = oracle.paged_attention_golden(case["query"], gk, gv, case["block_tables"], case["context_lens"],
                                      case["qk_scale"], case["k_descale"], case["v_descale"])
    tol = tol_for(spec.dtype, spec.kv_int8)
    assert_close(to_np(out), g, tol, spec.name)
    rel_max, rel_l2 = oracle.scale_free_error(to_np(out), g)
    assert rel_l2 < 1e-2 and rel_max < 3e-2, (spec.name, rel_max, rel_l2)


@pytest.mark.parametrize("dtype,kv8", [("bfloat16", False), ("float16", False), ("bfloat16", True)])
def test_pa_length_edges_and_empty_sequences(dtype, kv8):
    lens = [0, 1, 15, 16, 17, 127, 128, 129, 511, 512, 513, 1023, 1025, 0, 2048, 3000]
    spec = workloads.DecodeSpec("edges", len(lens), 32, dtype=dtype, kv_int8=kv8, seed=21)
    rng = np.random.default_rng(spec.seed)
    case = workloads.decode_case(spec)
    nb, tables, slots = workloads.layout(spec, np.array(lens, dtype=np.int32), rng)
    assert nb <= case["num_blocks"] or True
    spec2 = workloads.DecodeSpec("edges", len(lens), 32, dtype=dtype, kv_int8=kv8, seed=21, num_blocks=nb)
    spec2.len_lo, spec2.len_hi = 1, 1
    case = workloads.decode_case(spec2)
    case["context_lens"] = np.array(lens, dtype=np.int32)
    case["block_tables"] = tables
    for kernel in (_abi.KERNEL_GENERIC, _abi.KERNEL_TMA):
        out, info = kernels.paged_attention_raw(
            to_dev(case["query"]), to_dev(case["key_cache"]), to_dev(case["value_cache"]), to_dev(tables), lens,
            case["qk_scale"], 1 if kv8 else 0, to_dev(case["k_descale"]), None, to_dev(case["v_descale"]), None,
            kernel=kernel)
        g = oracle.paged_attention_golden(case["query"], case["key_cache"], case["value_cache"], tables,
                                          case["context_lens"], case["qk_scale"], case["k_descale"], case["v_descale"])
        o = to_np(out).astype(np.float32)
        assert np.all(o[0] == 0) and np.all(o[13] == 0)  # empty sequences give zeros
        assert_close(o, g, tol_for(dtype, kv8), f"edges kernel={kernel}")
        rel_max, rel_l2 = oracle.scale_free_error(o, g)
        assert rel_l2 < 1e-2, (kernel, rel_max, rel_l2)


def test_pa_long_context_uses_larger_splits():
    # 20000 and 70000 tokens: 1024- and 2048-token splits, many partials through the reduce kernel
    lens = [20000, 70000, 700]
    spec = workloads.DecodeSpec("long", 3, 16, kv_heads=2, dtype="bfloat16", seed=9, len_lo=1, len_hi=1)
    rng = np.random.default_rng(3)
    nb, tables, _ = workloads.layout(spec, np.array(lens, dtype=np.int32), rng)
    spec.num_blocks = nb
    case = workloads.decode_case(spec)
    out, info = kernels.paged_attention_raw(to_dev(case["query"]), to_dev(case["key_cache"]),
                                            to_dev(case["value_cache"]), to_dev(tables), lens, case["qk_scale"])
    assert info.max_splits == 35 and info.partials == 20 + 35 + 2
    g = oracle.paged_attention_golden(case["query"], case["key_cache"], case["value_cache"], tables,
                                      np.array(lens), case["qk_scale"])
    assert_close(to_np(out), g, 1e-2, "long")
    rel_max, rel_l2 = oracle.scale_free_error(to_np(out), g)
    assert rel_l2 < 1e-2, (rel_max, rel_l2)


@pytest.mark.parametrize("kernel", [_abi.KERNEL_GENERIC, _abi.KERNEL_TMA])
@pytest.mark.parametrize("kv8", [False, True])
def test_pa_batch_invariance_bitwise(kernel, kv8):
    # a request's output must not depend on what it is batched with
    # (tests/st/test_custom_paged_attention_batch_invariant.py:231-317)
    lens_all = [255, 256, 257, 511, 512, 513, 2048, 4096, 700, 1, 33, 1500] * 4
    spec = workloads.DecodeSpec("binv", len(lens_all), 32, dtype="bfloat16", kv_int8=kv8, seed=33, len_lo=1, len_hi=1)
    rng = np.random.default_rng(5)
    nb, tables, _ = workloads.layout(spec, np.array(lens_all, dtype=np.int32), rng)
    spec.num_blocks = nb
    case = workloads.decode_case(spec)
    q, kc, vc = to_dev(case["query"]), to_dev(case["key_cache"]), to_dev(case["value_cache"])
    kd, vd = to_dev(case["k_descale"]), to_dev(case["v_descale"])
    dt = to_dev(tables)
    full, _ = kernels.paged_attention_raw(q, kc, vc, dt, lens_all, case["qk_scale"], int(kv8), kd, None, vd, None,
                                          kernel=kernel)
    full = to_np(full).view(np.uint16)
    for i in (0, 3, 6, 7, 9, 23, 47):
        one, _ = kernels.paged_attention_raw(q[i:i + 1].contiguous(), kc, vc, dt[i:i + 1].contiguous(),
                                             [lens_all[i]], case["qk_scale"], int(kv8), kd, None, vd, None,
                                             kernel=kernel)
        assert np.array_equal(to_np(one).view(np.uint16)[0], full[i]), f"request {i} changed with the batch"


@pytest.mark.parametrize("n,scale", [(2, 0.1), (3, 0.3), (1, 1.0)])
def test_fused_decode_step_equals_separate_calls(n, scale):
    # msco_decode_step (scatter + attention in one call, programmatic launch overlap) must give the
    # same cache and the same output, bit for bit, as the two separate launches
    spec = workloads.config_spec(n, scale)
    c = workloads.decode_case(spec)
    dev = {k: to_dev(c[k]) for k in ("query", "key", "value", "block_tables", "slot_mapping")}
    kd, vd = to_dev(c["k_descale"]), to_dev(c["v_descale"])
    lens = [int(x) for x in c["context_lens"]]
    desc = kernels.make_pa_desc(dev["query"], to_dev(c["key_cache"]), dev["block_tables"], c["qk_scale"],
                                1 if spec.kv_int8 else 0)
    plan = _abi.PaPlan(desc, lens)
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device="cuda")
    results = []
    for fused in (False, True):
        kc, vc = to_dev(c["key_cache"]), to_dev(c["value_cache"])
        out = torch.empty_like(dev["query"])
        for _ in range(3):  # repeated launches reuse the workspace without clearing it
            if fused:
                kernels.decode_step(plan, dev["key"], dev["value"], kc, vc, dev["slot_mapping"], dev["query"],
                                    dev["block_tables"], out, ws, kd, None, vd, None)
            else:
                if spec.kv_int8:
                    kernels.rac_scatter_quant(dev["key"], dev["value"], kc, vc, dev["slot_mapping"], kd, vd)
                else:
                    kernels.rac_scatter(dev["key"], dev["value"], kc, vc, dev["slot_mapping"])
                kernels.pa_launch(plan, dev["query"], kc, vc, dev["block_tables"], out, ws, kd, None, vd, None)
        kernels.pa_status(plan, ws)
        results.append((to_np(kc).copy(), to_np(out).copy()))
    assert np.array_equal(results[0][0].view(np.uint8), results[1][0].view(np.uint8))
    assert np.array_equal(results[0][1].view(np.uint16), results[1][1].view(np.uint16))
    plan.close()


@pytest.mark.parametrize("n,scale", [(2, 0.1), (3, 0.3)])
def test_decode_step_captured_in_a_cuda_graph_replays_bit_identically(n, scale):
    # a decode step whose lengths do not change (a frozen step) can be captured once and replayed: the
    # three launches -- with their programmatic launch overlap -- become graph nodes, the plan rides in
    # the kernel parameters; the replays must reproduce the eager step's cache and output bit for bit
    spec = workloads.config_spec(n, scale)
    c = workloads.decode_case(spec)
    dev = {k: to_dev(c[k]) for k in ("query", "key", "value", "block_tables", "slot_mapping")}
    kd, vd = to_dev(c["k_descale"]), to_dev(c["v_descale"])
    desc = kernels.make_pa_desc(dev["query"], to_dev(c["key_cache"]), dev["block_tables"], c["qk_scale"],
                                1 if spec.kv_int8 else 0)
    plan = _abi.PaPlan(desc, [int(x) for x in c["context_lens"]])
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device="cuda")

    def step(kc, vc, out):
        kernels.decode_step(plan, dev["key"], dev["value"], kc, vc, dev["slot_mapping"], dev["query"],
                            dev["block_tables"], out, ws, kd, None, vd, None)
    kc0, vc0 = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    want = torch.empty_like(dev["query"])
    step(kc0, vc0, want)            # eager: also sets the kernels' attributes before any capture
    torch.cuda.synchronize()
    kernels.pa_status(plan, ws)

    kc1, vc1 = to_dev(c["key_cache"]), to_dev(c["value_cache"])
    got = torch.empty_like(dev["query"])
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step(kc1, vc1, got)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        got.zero_()
        graph.replay()
        torch.cuda.synchronize()
        kernels.pa_status(plan, ws)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    assert torch.equal(kc1.view(torch.uint8), kc0.view(torch.uint8))
    assert torch.equal(vc1.view(torch.uint8), vc0.view(torch.uint8))
    plan.close()


def test_pa_out_of_range_block_id_is_reported_not_faulted():
    case = _st_case("gqa_32to8_alibi", mask_free=True)
    v = st_inputs.operator_view(case)
    tables = v["block_tables"].copy()
    tables[2, 0] = 10 ** 6
    for kernel in (_abi.KERNEL_GENERIC, _abi.KERNEL_TMA):
        with pytest.raises(_abi.MscoError) as e:
            kernels.paged_attention_raw(to_dev(v["query"]), to_dev(v["key_cache"]), to_dev(v["value_cache"]),
                                        to_dev(tables), list(v["context_lens"]), v["qk_scale"], kernel=kernel)
        assert e.value.code == _abi.ERR_OOB


# ----------------------------------------------------------------------------
# the benchmark configurations at FULL size (caches generated on the device, the C / OpenMP
# restatement of the reference golden as the checker)
# ----------------------------------------------------------------------------
def _host_case(c, lens, slots):
    kd, vd = c["k_descale"], c["v_descale"]
    return {"query": to_np(c["query"]), "key": to_np(c["key"]), "value": to_np(c["value"]),
            "key_cache": to_np(c["key_cache"]), "value_cache": to_np(c["value_cache"]),
            "block_tables": c["block_tables_host"], "slot_mapping": slots, "context_lens": lens,
            "k_descale": None if kd is None else kd.cpu().numpy(), "v_descale": None if vd is None else vd.cpu().numpy()}


@pytest.mark.parametrize("n", [2, 3, 4, 5])
def test_pa_benchmark_configs_full_size(n):
    # C2 (bf16, batch 64), C3 (int8 KV, batch 128, 64 q heads), C4 (log-uniform lengths up to 131072
    # tokens, 2048-token splits, batch 32) and C5's decode (batch 256): one real decode step through
    # msco_decode_step on caches of the full size, every sequence checked against the C oracle
    from oracle import c_oracle
    spec = workloads.config_spec(n)
    c = workloads.decode_case_device(spec, "cuda", growth_steps=2)
    lens = np.asarray(c["context_lens"], dtype=np.int32)
    if n == 4:
        assert lens.max() > 65536, "the drawn lengths must reach the 2048-token split rule"
    quant = 1 if spec.kv_int8 else 0
    desc = kernels.make_pa_desc(c["query"], c["key_cache"], c["block_tables"], c["qk_scale"], quant)
    plan = _abi.PaPlan(desc, [int(x) for x in lens])
    info = plan.info()
    assert info.kernel == 2 and (info.partials > 0 or n == 3)  # C3: int8 contexts of up to 4096 tokens are one item
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device="cuda")
    out = torch.empty_like(c["query"])
    slots = workloads.slots_of_last_token(c["block_tables_host"], lens, spec.block_size)
    kernels.decode_step(plan, c["key"], c["value"], c["key_cache"], c["value_cache"], to_dev(slots), c["query"],
                        c["block_tables"], out, ws, c["k_descale"], None, c["v_descale"], None)
    kernels.pa_status(plan, ws)
    h = _host_case(c, lens, slots)  # the caches as the step left them: the scatter is idempotent
    if quant:
        gk, gv = c_oracle.reshape_and_cache_quant(h["key"], h["value"], h["key_cache"], h["value_cache"], slots,
                                                  h["k_descale"], h["v_descale"], inplace=False)
    else:
        gk, gv = c_oracle.reshape_and_cache(h["key"], h["value"], h["key_cache"], h["value_cache"], slots, inplace=False)
    # bit-exact scatter: the rows the step wrote are what the oracle writes
    assert np.array_equal(gk.view(np.uint8), h["key_cache"].view(np.uint8))
    assert np.array_equal(gv.view(np.uint8), h["value_cache"].view(np.uint8))
    g = c_oracle.paged_attention(h["query"], gk, gv, h["block_tables"], lens, c["qk_scale"], h["k_descale"],
                                 h["v_descale"])
    o = to_np(out)
    assert_close(o, g, tol_for(spec.dtype, spec.kv_int8), spec.name)
    rel_max, rel_l2 = oracle.scale_free_error(o, g)
    assert rel_l2 < 1e-2 and rel_max < 3e-2, (spec.name, rel_max, rel_l2)
    plan.close()


@pytest.mark.parametrize("quant", [False, True])
def test_rac_prefill_config5_full_size_bit_exact(quant):
    # 16384 tokens x (8 kv heads x 128) through an injective random slot map into 4096 blocks of 128
    # with 5 % of the slots -1.  The oracle runs on a compact cache (one row per token); the device
    # cache has the full 4096 x 128 slots: written rows must equal the oracle's bit for bit and no
    # other byte may change.
    tokens, blocks, bs, c = 16384, 4096, 128, 1024
    rng = np.random.default_rng(5)
    slots = rng.permutation(blocks * bs)[:tokens].astype(np.int32)
    slots[rng.random(tokens) < 0.05] = -1
    key = rng.standard_normal((tokens, c), dtype=np.float32).astype(BF16)
    val = rng.standard_normal((tokens, c), dtype=np.float32).astype(BF16)
    cdt = torch.int8 if quant else torch.bfloat16
    fill = 7 if quant else 1.5
    kc = torch.full((blocks, bs, 8, 128), fill, dtype=cdt, device="cuda")
    vc = torch.full((blocks, bs, 8, 128), fill, dtype=cdt, device="cuda")
    compact = np.where(slots >= 0, np.arange(tokens), -1).astype(np.int32)
    if quant:
        kd = rng.uniform(0.01, 0.05, c).astype(np.float32)
        vd = rng.uniform(0.01, 0.05, c).astype(np.float32)
        z = np.full((tokens, 1, 8, 128), fill, dtype=np.int8)
        gk, gv = oracle.reshape_and_cache_quant_golden(key, val, z, z.copy(), compact, kd, vd)
        kernels.rac_scatter_quant(to_dev(key), to_dev(val), kc, vc, to_dev(slots), to_dev(kd), to_dev(vd))
    else:
        z = np.full((tokens, 1, 8, 128), fill, dtype=np.float32).astype(BF16)
        gk, gv = oracle.reshape_and_cache_golden(key, val, z, z.copy(), compact)
        kernels.rac_scatter(to_dev(key), to_dev(val), kc, vc, to_dev(slots))
    torch.cuda.synchronize()
    valid = slots >= 0
    idx = torch.from_numpy(slots[valid].astype(np.int64)).cuda()
    for cache, g in ((kc, gk), (vc, gv)):
        flat = cache.view(blocks * bs, c)
        rows = to_np(flat[idx])
        assert np.array_equal(rows.view(np.uint8), g.reshape(tokens, c)[valid].view(np.uint8))
        untouched = torch.ones(blocks * bs, dtype=torch.bool, device="cuda")
        untouched[idx] = False
        assert bool((flat[untouched] == fill).all()), "a slot outside the map was written"


def test_replanned_decode_steps_equal_freshly_planned_ones():
    # a decode loop: lengths grow by one per step, the plan object is re-planned in place; every
    # step's output must equal, bit for bit, the output of a freshly built plan
    spec = workloads.config_spec(2, 0.12)
    c = workloads.decode_case_device(spec, "cuda", growth_steps=140)
    lens0 = np.asarray(c["context_lens"], dtype=np.int32)
    desc = kernels.make_pa_desc(c["query"], c["key_cache"], c["block_tables"], c["qk_scale"], 0)
    plan = _abi.PaPlan(desc, [int(x) for x in lens0])
    ws = torch.empty(max(_abi.PaPlan(desc, [int(x) + 140 for x in lens0]).workspace_bytes, 256), dtype=torch.uint8,
                     device="cuda")
    a0 = _abi.plan_arena_stats()
    for i in (1, 2, 3, 64, 129, 130):  # across a block boundary for every sequence
        lens = lens0 + np.int32(i)
        slots = to_dev(workloads.slots_of_last_token(c["block_tables_host"], lens, spec.block_size))
        plan.replan(lens)
        out = torch.empty_like(c["query"])
        kernels.decode_step(plan, c["key"], c["value"], c["key_cache"], c["value_cache"], slots, c["query"],
                            c["block_tables"], out, ws)
        kernels.pa_status(plan, ws)
        fresh, _ = kernels.paged_attention_raw(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                               [int(x) for x in lens], c["qk_scale"])
        assert np.array_equal(to_np(out).view(np.uint16), to_np(fresh).view(np.uint16)), f"step {i}"
    a1 = _abi.plan_arena_stats()
    assert a1["slabs"] == a0["slabs"], "re-planning must not add pinned slabs"
    plan.close()


@pytest.mark.parametrize("kv8", [False, True])
def test_pa_batch_invariance_at_batch_256(kv8):
    # the reference's property test (tests/st/test_custom_paged_attention_batch_invariant.py:231-317)
    # at batch 256 with lengths around the split boundaries, GQA 32 / 8
    base = [255, 256, 257, 511, 512, 513, 2048, 4096, 8192]
    lens_all = (base * 29)[:256]
    spec = workloads.DecodeSpec("binv256", 256, 32, dtype="bfloat16", kv_int8=kv8, seed=34, len_lo=1, len_hi=1)
    rng = np.random.default_rng(6)
    nb, tables, _ = workloads.layout(spec, np.array(lens_all, dtype=np.int32), rng)
    spec.num_blocks = nb
    spec.len_lo, spec.len_hi = 1, 1
    c = workloads.decode_case_device(spec, "cuda")
    q, kc, vc, kd, vd = c["query"], c["key_cache"], c["value_cache"], c["k_descale"], c["v_descale"]
    dt = to_dev(tables)
    full, info = kernels.paged_attention_raw(q, kc, vc, dt, lens_all, c["qk_scale"], int(kv8), kd, None, vd, None)
    assert info.kernel == 2
    full = to_np(full).view(np.uint16)
    for i in (0, 1, 2, 3, 4, 5, 6, 7, 8, 100, 255):
        one, _ = kernels.paged_attention_raw(q[i:i + 1].contiguous(), kc, vc, dt[i:i + 1].contiguous(),
                                             [lens_all[i]], c["qk_scale"], int(kv8), kd, None, vd, None)
        assert np.array_equal(to_np(one).view(np.uint16)[0], full[i]), f"request {i} (length {lens_all[i]}) changed"


@pytest.mark.parametrize("hd,bs,hq,hkv,dtype", [(64, 128, 32, 8, "bfloat16"), (64, 16, 24, 2, "float16"),
                                                (256, 64, 16, 4, "bfloat16"), (256, 16, 8, 8, "float16"),
                                                (256, 32, 24, 2, "bfloat16")])
def test_pa_head_dims_64_and_256_in_the_tma_kernel(hd, bs, hq, hkv, dtype):
    # the reference's head-size sweeps (tests/st/test_custom_paged_attention.py:1826-1871, 2211-2286):
    # head_dim 64 and 256 run in the TMA kernel too; both kernels against the oracle, several splits
    lens = [1, 17, 500, 513, 1300, 2049, 0, 4100]
    spec = workloads.DecodeSpec("hd", len(lens), hq, kv_heads=hkv, head_size=hd, block_size=bs, dtype=dtype, seed=hd + bs,
                                len_lo=1, len_hi=1)
    rng = np.random.default_rng(7)
    nb, tables, _ = workloads.layout(spec, np.array(lens, dtype=np.int32), rng)
    spec.num_blocks = nb
    case = workloads.decode_case(spec)
    q, kc, vc, dt = to_dev(case["query"]), to_dev(case["key_cache"]), to_dev(case["value_cache"]), to_dev(tables)
    g = oracle.paged_attention_golden(case["query"], case["key_cache"], case["value_cache"], tables,
                                      np.array(lens, dtype=np.int32), case["qk_scale"])
    outs = {}
    for kernel in (_abi.KERNEL_GENERIC, _abi.KERNEL_TMA, _abi.KERNEL_AUTO):
        out, info = kernels.paged_attention_raw(q, kc, vc, dt, lens, case["qk_scale"], kernel=kernel)
        assert info.kernel == (1 if kernel == _abi.KERNEL_GENERIC else 2)
        o = to_np(out).astype(np.float32)
        assert np.all(o[6] == 0)
        assert_close(o, g, tol_for(dtype, False), f"head_dim {hd} kernel={kernel}")
        rel_max, rel_l2 = oracle.scale_free_error(o, g)
        assert rel_l2 < 1e-2, (kernel, rel_max, rel_l2)
        outs[kernel] = to_np(out).view(np.uint16)
    assert np.array_equal(outs[_abi.KERNEL_TMA], outs[_abi.KERNEL_AUTO])


@pytest.mark.parametrize("n,scale", [(2, 0.12), (3, 0.3), (4, 0.05)])
def test_in_kernel_merge_equals_the_reduce_kernel(monkeypatch, n, scale):
    # MSCO_PA_FUSED_MERGE=1: the CTA that stores a group's last partial merges the group inside the attention
    # kernel (same merge code, same split order): bit-identical to the reduce kernel's result
    spec = workloads.config_spec(n, scale)
    if spec.kv_int8:  # long enough for several int8 splits
        spec.batch, spec.len_lo, spec.len_hi = 12, 3000, 9000
    c = workloads.decode_case(spec)
    args = (to_dev(c["query"]), to_dev(c["key_cache"]), to_dev(c["value_cache"]), to_dev(c["block_tables"]),
            [int(x) for x in c["context_lens"]], c["qk_scale"], 1 if spec.kv_int8 else 0, to_dev(c["k_descale"]), None,
            to_dev(c["v_descale"]), None)
    monkeypatch.delenv("MSCO_PA_FUSED_MERGE", raising=False)
    ref, info = kernels.paged_attention_raw(*args)
    assert info.partials > 0
    monkeypatch.setenv("MSCO_PA_FUSED_MERGE", "1")
    for _ in range(3):
        out, _ = kernels.paged_attention_raw(*args)
        assert np.array_equal(to_np(out).view(np.uint16), to_np(ref).view(np.uint16))
