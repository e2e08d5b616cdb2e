"""CPU: the oracle is pinned against outputs of the reference's own golden functions.

tests/golden/*.npz were produced by tests/golden/make_golden.py, which imports
the reference's test modules and runs their numpy goldens on inputs from this
repository's seeded generators.  Here the numpy restatement and the C
restatement must reproduce those outputs, and the generators must still
produce the inputs the fixtures were made from (sha256).
"""
import os

import numpy as np
import pytest

from ms_custom_ops_b200 import workloads
from oracle import c_oracle
from oracle import paged_kv_numpy as oracle
from tests.golden import cases

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _fx(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


def _close(a, g, what):
    a = np.asarray(a, dtype=np.float32)
    g = np.asarray(g, dtype=np.float32)
    # float32 re-association only: a few ulp of the largest magnitude involved
    lim = 2e-5 * max(1.0, float(np.abs(g).max())) + 1e-3 * np.abs(g) * (g.dtype == np.float16)
    assert np.all(np.abs(a - g) <= lim), (what, float(np.abs(a - g).max()))


@pytest.mark.parametrize("name", sorted(cases.ST_CASES))
def test_numpy_and_c_oracle_match_reference_golden(name):
    case = cases.st_case(name)
    fx = _fx("pa_" + name)
    for k in ("query", "key_cache", "value_cache", "block_tables"):
        assert str(fx["sha_" + k]) == cases.digest(case[k]), f"generator drifted for {name}/{k}"
    golden = fx["golden"]
    args = (case["query"], case["key_cache"], case["value_cache"], case["block_tables"], case["context_lens"],
            case["qk_scale"], case["k_descale"], case["v_descale"], case["k_offset"], case["v_offset"],
            case["mask"], case["mask_type"])
    out_np = oracle.paged_attention_golden(*args)
    out_c = c_oracle.paged_attention(*args)
    if golden.dtype == np.float16:  # the reference casts fp16 results back to fp16
        tol = 1e-3 * np.maximum(np.abs(golden.astype(np.float32)), 1.0)
        assert np.all(np.abs(out_np - golden.astype(np.float32)) <= tol)
        assert np.all(np.abs(out_c - golden.astype(np.float32)) <= tol)
    else:
        _close(out_np, golden, name + "/numpy")
        _close(out_c, golden, name + "/c")
    ok, _ = oracle.reference_accuracy_verdict(out_np, golden, "float32", case["num_heads"],
                                              int(max(case["context_lens"])))
    assert ok


@pytest.mark.parametrize("name", sorted(cases.RAC_CASES))
def test_scatter_oracles_match_reference_golden(name):
    c = cases.rac_case(name)
    fx = _fx("rac_" + name)
    assert str(fx["sha_in_key"]) == cases.digest(c["key"])
    assert str(fx["sha_in_key_cache"]) == cases.digest(c["key_cache"])
    for impl in (oracle.reshape_and_cache_golden, c_oracle.reshape_and_cache):
        gk, gv = impl(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
        assert cases.digest(gk) == str(fx["sha_key_cache"])
        assert cases.digest(gv) == str(fx["sha_value_cache"])


def test_config1_fixture_reproduced_by_both_oracles():
    fx = _fx("config1")
    spec = workloads.config_spec(1)
    c = workloads.decode_case(spec)
    assert np.array_equal(fx["context_lens"], c["context_lens"])
    assert str(fx["sha_query"]) == cases.digest(c["query"])
    gk, gv = oracle.reshape_and_cache_golden(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
    assert cases.digest(gk) == str(fx["sha_key_cache"]) and cases.digest(gv) == str(fx["sha_value_cache"])
    ck, cv = c_oracle.reshape_and_cache(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
    assert cases.digest(ck) == str(fx["sha_key_cache"])
    for impl in (oracle.paged_attention_golden, c_oracle.paged_attention):
        out = impl(c["query"], gk, gv, c["block_tables"], c["context_lens"], c["qk_scale"])
        g = fx["golden"].astype(np.float32)
        assert np.all(np.abs(out - g) <= 1e-3 * np.maximum(np.abs(g), 1.0))


@pytest.mark.parametrize("name", sorted(cases.MTP_CASES))
def test_multi_token_oracle_matches_reference_golden(name):
    # several query tokens per sequence with the SPEC mask: stored outputs of the reference's golden
    c, fx = cases.mtp_case(name), _fx("pa_mtp_" + name)
    assert cases.digest(c["query"]) == str(fx["sha_query"]) and cases.digest(c["key_cache"]) == str(fx["sha_key_cache"])
    out = oracle.paged_attention_golden(c["query"], c["key_cache"], c["value_cache"], c["block_tables"],
                                        c["context_lens"], c["qk_scale"], mask=c["mask"], mask_type=3,
                                        q_seq_lens=c["q_seq_lens"])
    g = fx["golden"].astype(np.float32)
    assert out.shape == g.shape == (int(c["q_seq_lens"].sum()),) + c["query"].shape[1:]
    np.testing.assert_allclose(out, g, rtol=0, atol=5e-4 if c["q_dtype"] == "float16" else 1e-6)
    # the mask is causal inside the window of new tokens: the last token of a sequence sees everything,
    # so it equals plain decode attention over the same context
    if int(np.sum(c["context_lens"])) > 40000:
        return  # (the long fixtures: the numpy golden above is a minute of CPU time already)
    last = np.cumsum(c["q_seq_lens"]) - 1
    plain = oracle.paged_attention_golden(c["query"][last], c["key_cache"], c["value_cache"], c["block_tables"],
                                          c["context_lens"], c["qk_scale"])
    np.testing.assert_allclose(out[last], plain, rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("name", sorted(cases.PCL_CASES))
def test_cache_load_oracle_matches_reference_golden(name):
    # stored digests of the reference's golden_calc_nd outputs on the same seeded inputs
    c, fx = cases.pcl_case(name), _fx("pcl_" + name)
    assert cases.digest(c["key_cache"]) == str(fx["sha_in_key_cache"])
    k, v = oracle.paged_cache_load_golden(c["key_cache"], c["value_cache"], c["block_tables"], c["seq_lens"],
                                          c["seq_starts"], c["cumsum"])
    assert k.shape[0] == int(fx["rows"])
    assert cases.digest(k) == str(fx["sha_key_out"]) and cases.digest(v) == str(fx["sha_value_out"])


@pytest.mark.parametrize("name", sorted(cases.PCL_CASES))
def test_c_cache_load_matches_reference_golden(name):
    c, fx = cases.pcl_case(name), _fx("pcl_" + name)
    k, v = c_oracle.paged_cache_load(c["key_cache"], c["value_cache"], c["block_tables"], c["seq_lens"],
                                     c["seq_starts"], c["cumsum"])
    assert cases.digest(k) == str(fx["sha_key_out"]) and cases.digest(v) == str(fx["sha_value_out"])


def test_c_cache_load_and_merge_agree_with_numpy_on_irregular_input():
    rng = np.random.default_rng(8)
    kc = rng.integers(-128, 128, (12, 4, 2, 3)).astype(np.int8)
    vc = rng.standard_normal((12, 4, 2, 5)).astype(np.float16)
    tables = rng.integers(-2, 12, (7, 9)).astype(np.int32)
    lens = rng.integers(0, 21, 7)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    starts = (rng.integers(0, 12, 7)).astype(np.int32)
    for args in ((lens.astype(np.int32), None, False), (cu, starts, True), (cu, None, True)):
        a = oracle.paged_cache_load_golden(kc, vc, tables, *args)
        b = c_oracle.paged_cache_load(kc, vc, tables, *args)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    lse = rng.standard_normal((5, 333)).astype(np.float32) * 3
    parts = rng.standard_normal((5, 333, 24)).astype(np.float32)
    np.testing.assert_allclose(c_oracle.fa_update(lse, parts), oracle.fa_update_golden(lse, parts), rtol=2e-6, atol=1e-7)


def test_cache_load_oracle_skips_negative_blocks():
    kc = np.arange(4 * 2 * 1 * 2, dtype=np.int8).reshape(4, 2, 1, 2) + 1
    tables = np.array([[1, -1, 3], [0, 2, -1]], np.int32)
    k, v = oracle.paged_cache_load_golden(kc, kc, tables, np.array([5, 3], np.int32))
    want = np.concatenate([kc[1], kc[3][:1], kc[0], kc[2][:1]])
    assert np.array_equal(k[:6], want) and not k[6:].any() and k.shape[0] == 8 and np.array_equal(k, v)


@pytest.mark.parametrize("name", sorted(cases.FA_CASES))
def test_fa_update_oracle_matches_reference_golden(name):
    c, fx = cases.fa_case(name), _fx("fa_" + name)
    assert cases.digest(c["lse"]) == str(fx["sha_lse"])
    np.testing.assert_allclose(oracle.fa_update_golden(c["lse"], c["local_out"]), fx["golden"], rtol=1e-6, atol=1e-7)


def test_negative_slots_are_skipped_and_later_rows_win():
    rng = np.random.default_rng(0)
    kc = rng.integers(-100, 100, (4, 8, 2, 4)).astype(np.int8)
    key = rng.integers(-100, 100, (5, 8)).astype(np.int8)
    slot = np.array([3, -1, 17, 3, -5], dtype=np.int32)
    out, _ = oracle.reshape_and_cache_golden(key, None, kc, None, slot)
    assert np.array_equal(out[0, 3].ravel(), key[3])      # the later duplicate wins
    assert np.array_equal(out[2, 1].ravel(), key[2])
    untouched = np.ones(32, bool)
    untouched[[3, 17]] = False
    assert np.array_equal(out.reshape(32, 8)[untouched], kc.reshape(32, 8)[untouched])


def test_quantising_scatter_rounding_and_saturation():
    # float32 division, ties to even, saturation to [-128, 127], offset after rounding
    x = np.array([[0.5, 1.5, 2.5, -0.5, -1.5, 1000.0, -1000.0, 0.0374]], dtype=np.float16)
    d = np.array([1, 1, 1, 1, 1, 1, 1, 0.025], dtype=np.float32)
    q = oracle.quantize_rows_golden(x, d)
    assert q.tolist() == [[0, 2, 2, 0, -2, 127, -128, 1]]
    q2 = oracle.quantize_rows_golden(x, d, np.array([1, 1, 1, 1, 1, 1, 1, 1], dtype=np.int32))
    assert q2.tolist() == [[-1, 1, 1, -1, -3, 127, -128, 0]]
    # round trip through the de-quantisation of paged attention: |x - (q + o) * d| <= d / 2
    rng = np.random.default_rng(1)
    xs = rng.standard_normal((64, 32)).astype(np.float32)
    ds = rng.uniform(0.01, 0.05, 32).astype(np.float32)
    os_ = rng.integers(-5, 5, 32).astype(np.int32)
    qs = oracle.quantize_rows_golden(xs, ds, os_).astype(np.float32)
    back = (qs + os_) * ds
    inside = np.abs(xs / ds - os_) < 127
    assert np.all(np.abs(back - xs)[inside] <= ds[None, :].repeat(64, 0)[inside] * 0.5001)


def test_split_merge_equals_unsplit_attention():
    # the partial-softmax merge the kernels use (fa_update golden, tests/st/test_asd_faupdate.py:34-59)
    case = cases.st_case("varied_seqlens", mask_free=True)
    full = oracle.paged_attention_golden(case["query"], case["key_cache"], case["value_cache"],
                                         case["block_tables"], case["context_lens"], case["qk_scale"])
    b, L = 3, 2000
    q = case["query"][b].astype(np.float32)
    K = oracle._gather_seq(case["key_cache"].astype(np.float32), case["block_tables"][b], L, 128)
    V = oracle._gather_seq(case["value_cache"].astype(np.float32), case["block_tables"][b], L, 128)
    outs, lses = [], []
    for s0 in range(0, L, 512):
        k, v = K[s0:s0 + 512], V[s0:s0 + 512]
        sc = np.einsum("hd,thd->ht", q, k) * case["qk_scale"]
        m = sc.max(-1, keepdims=True)
        e = np.exp(sc - m)
        outs.append(np.einsum("ht,thd->hd", e / e.sum(-1, keepdims=True), v))
        lses.append((m + np.log(e.sum(-1, keepdims=True)))[:, 0])
    merged = oracle.fa_update_golden(np.stack(lses), np.stack(outs))
    assert np.allclose(merged, full[b], atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("name", sorted(cases.RACNPD_CASES))
def test_head_major_scatter_oracle_matches_reference_golden(name):
    # digests of the reference's npd_cache_inference (tests/st/test_custom_reshape_and_cache_npd.py:487-515)
    c = cases.racnpd_case(name)
    fx = np.load(os.path.join(GOLDEN_DIR, f"racnpd_{name}.npz"))
    assert str(fx["sha_in_key"]) == cases.digest(c["key"]) and str(fx["sha_in_key_cache"]) == cases.digest(c["key_cache"])
    gk, gv = oracle.reshape_and_cache_bnsd_golden(c["key"], c["value"], c["key_cache"], c["value_cache"], c["slot_mapping"])
    assert cases.digest(gk) == str(fx["sha_key_cache"]) and cases.digest(gv) == str(fx["sha_value_cache"])
    # the same rows in the other block layout: transposing the blocks commutes with the scatter
    bk, bv = oracle.reshape_and_cache_golden(c["key"], c["value"], oracle.bnsd_to_bsnd(c["key_cache"]),
                                             oracle.bnsd_to_bsnd(c["value_cache"]), c["slot_mapping"])
    assert np.array_equal(oracle.bnsd_to_bsnd(gk), bk) and np.array_equal(oracle.bnsd_to_bsnd(gv), bv)
