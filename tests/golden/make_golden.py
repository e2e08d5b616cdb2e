"""Generate the golden fixtures from the reference's own numpy goldens.

Run on a machine that has a checkout of the reference (it cannot travel with
the test-suite):

    python tests/golden/make_golden.py /path/to/reference

For every case of tests/golden/cases.py the inputs come from this
repository's seeded generators; the expected outputs come from the
reference's `PagedAttentionDataGenerator.compute_golden_reference`
(tests/st/test_custom_paged_attention.py:528-699) and
`InferenceEngine.nd_inference` (tests/st/test_custom_reshape_and_cache.py:282-307),
`golden_calc_nd` (tests/st/test_custom_paged_cache_load.py:35-76) and `golden_calc`
(tests/st/test_asd_faupdate.py:34-59), imported unchanged through a stub of the `mindspore` module.  For the
reference-style attention cases the script also checks that our generator
reproduces the reference generator's inputs bit for bit.

Written files (tests/golden/):
  pa_<case>.npz       golden output + sha256 of every input
  pa_mtp_<case>.npz   the same for the multi-token (speculative) query cases
  rac_<case>.npz      sha256 of the golden caches (and of the inputs)
  config1.npz         benchmark configuration 1: cache digests after the scatter + attention output
  pcl_<case>.npz      sha256 of the gathered K / V (and of the input caches)
  fa_<case>.npz       golden output of the partial-output merge
  racnpd_<case>.npz   sha256 of the golden head-major caches of `npd_cache_inference`
                      (tests/st/test_custom_reshape_and_cache_npd.py:487-515)
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ms_stub  # noqa: E402
from tests.golden import cases  # noqa: E402
from ms_custom_ops_b200 import workloads  # noqa: E402


def main(ref_root):
    ms = ms_stub.install()
    sys.path.insert(0, os.path.join(ref_root, "tests", "st"))
    import test_custom_paged_attention as tpa
    import test_custom_reshape_and_cache as trc
    msd = {"float16": ms.float16, "bfloat16": ms.bfloat16, "int8": ms.int8}

    for name, cfg in cases.ST_CASES.items():
        seed, h, kvh, hd, bs, nb, lens, qd, kvd, quant, off, scale, mask = cfg
        case = cases.st_case(name)
        gen = tpa.PagedAttentionDataGenerator(seed)
        ref_in = gen.generate_inputs(h, kvh, hd, bs, nb, [1] * len(lens), lens, msd[qd], msd[kvd or qd], mask,
                                     quant, off)
        for key in ("query", "key_cache", "value_cache", "block_tables", "k_descale", "v_descale", "k_offset",
                    "v_offset", "mask"):
            a, b = ref_in[key], case[key]
            assert (a is None) == (b is None), (name, key)
            if a is not None:
                assert np.array_equal(np.asarray(a).astype(np.float32), np.asarray(b).astype(np.float32)), (name, key)
        golden = gen.compute_golden_reference(
            ref_in["query"], ref_in["key_cache"], ref_in["value_cache"], ref_in["block_tables"],
            ref_in["q_seq_lens"], ref_in["kv_seq_lens"], case["qk_scale"], ref_in["mask"], mask,
            ref_in["k_descale"], ref_in["v_descale"], ref_in["k_offset"], ref_in["v_offset"])
        digests = {k: cases.digest(case[k]) for k in ("query", "key_cache", "value_cache", "block_tables")}
        np.savez_compressed(os.path.join(HERE, f"pa_{name}.npz"), golden=np.asarray(golden),
                            **{f"sha_{k}": np.array(v) for k, v in digests.items()})
        print("pa", name, golden.dtype, golden.shape)

    for name, (seed, h, kvh, hd, bs, nb, qlens, lens, dt, _scale) in cases.MTP_CASES.items():
        case = cases.mtp_case(name)
        gen = tpa.PagedAttentionDataGenerator(seed)
        ref_in = gen.generate_inputs(h, kvh, hd, bs, nb, qlens, lens, msd[dt], msd[dt], 3, 0, False)
        for key in ("query", "key_cache", "value_cache", "block_tables", "mask"):
            assert np.array_equal(np.asarray(ref_in[key]).astype(np.float32),
                                  np.asarray(case[key]).astype(np.float32)), (name, key)
        golden = gen.compute_golden_reference(
            ref_in["query"], ref_in["key_cache"], ref_in["value_cache"], ref_in["block_tables"],
            ref_in["q_seq_lens"], ref_in["kv_seq_lens"], case["qk_scale"], ref_in["mask"], 3)
        np.savez_compressed(os.path.join(HERE, f"pa_mtp_{name}.npz"), golden=np.asarray(golden),
                            sha_query=np.array(cases.digest(case["query"])),
                            sha_key_cache=np.array(cases.digest(case["key_cache"])))
        print("pa_mtp", name, golden.dtype, golden.shape)

    for name in cases.RAC_CASES:
        c = cases.rac_case(name)
        gk, gv = trc.InferenceEngine.nd_inference(c["key"], c["value"], c["key_cache"], c["value_cache"],
                                                  c["slot_mapping"])
        np.savez_compressed(os.path.join(HERE, f"rac_{name}.npz"), sha_key_cache=np.array(cases.digest(gk)),
                            sha_value_cache=np.array(cases.digest(gv)),
                            sha_in_key=np.array(cases.digest(c["key"])),
                            sha_in_key_cache=np.array(cases.digest(c["key_cache"])))
        print("rac", name)

    # head-major ("BNSD") cache scatter: the golden of the reference's reshape_and_cache_npd test.  Its loop
    # has no skip for negative slots (its inputs have none); for the padded case the reference golden is
    # run on the valid tokens only, which is what the device code does (reshape_and_cache_npd.cpp:149-150).
    import test_custom_reshape_and_cache_npd as tnpd
    from oracle import paged_kv_numpy as restated_npd
    for name in cases.RACNPD_CASES:
        c = cases.racnpd_case(name)
        valid = c["slot_mapping"] >= 0
        gk, gv = tnpd.npd_cache_inference(c["key"][valid], c["value"][valid], c["key_cache"], c["value_cache"],
                                          c["slot_mapping"][valid])
        ok, ov = restated_npd.reshape_and_cache_bnsd_golden(c["key"], c["value"], c["key_cache"], c["value_cache"],
                                                            c["slot_mapping"])
        assert cases.digest(ok) == cases.digest(gk) and cases.digest(ov) == cases.digest(gv), name
        np.savez_compressed(os.path.join(HERE, f"racnpd_{name}.npz"), sha_key_cache=np.array(cases.digest(gk)),
                            sha_value_cache=np.array(cases.digest(gv)), sha_in_key=np.array(cases.digest(c["key"])),
                            sha_in_key_cache=np.array(cases.digest(c["key_cache"])))
        print("racnpd", name)

    import test_custom_paged_cache_load as tpcl
    import test_asd_faupdate as tfa
    from oracle import paged_kv_numpy as restated
    for name, (kd, vd, cumsum, _seed, geo) in cases.PCL_CASES.items():
        c = cases.pcl_case(name)
        nb, bs, heads, dk, dv, batch, _ = geo
        total = int(c["seq_lens"][-1]) if cumsum else int(c["seq_lens"].sum())
        # float16 stands in for the reference's dtype tag where it only picks the dtype of the
        # expected array: the rows are copied unchanged, and are compared in the cache dtype
        gk, gv = tpcl.golden_calc_nd(batch, heads, dk, dv, bs, c["block_tables"], c["seq_lens"], c["seq_starts"],
                                     c["key_cache"], c["value_cache"], msd[kd], msd[vd], total)
        gk, gv = gk.astype(c["key_cache"].dtype), gv.astype(c["value_cache"].dtype)
        ok, ov = restated.paged_cache_load_golden(c["key_cache"], c["value_cache"], c["block_tables"], c["seq_lens"],
                                                  c["seq_starts"], cumsum)
        assert cases.digest(ok) == cases.digest(gk) and cases.digest(ov) == cases.digest(gv), name
        np.savez_compressed(os.path.join(HERE, f"pcl_{name}.npz"), sha_key_out=np.array(cases.digest(gk)),
                            sha_value_out=np.array(cases.digest(gv)), rows=np.array(total),
                            sha_in_key_cache=np.array(cases.digest(c["key_cache"])),
                            sha_in_block_tables=np.array(cases.digest(c["block_tables"])))
        print("pcl", name, gk.shape, gv.shape)

    for name in cases.FA_CASES:
        c = cases.fa_case(name)
        g = np.asarray(tfa.golden_calc(c["lse"], c["local_out"]), dtype=np.float32)
        g = g.reshape(c["local_out"].shape[1], c["local_out"].shape[2])
        np.savez_compressed(os.path.join(HERE, f"fa_{name}.npz"), golden=g,
                            sha_lse=np.array(cases.digest(c["lse"])))
        print("fa", name, g.shape)
    # the reference's full-size fa_update shapes (tests/st/test_asd_faupdate.py:95-123): restatement == golden
    for sp, rows, hd in ((3, 1000 * 13, 128), (3, 2 * 4000 * 32, 128)):
        rng = np.random.default_rng(sp * rows)
        lse = rng.random((sp, rows), dtype=np.float32)
        lo = rng.random((sp, rows, hd), dtype=np.float32)
        g = np.asarray(tfa.golden_calc(lse, lo)).reshape(rows, hd)
        assert np.allclose(restated.fa_update_golden(lse, lo), g, rtol=1e-5, atol=1e-6), (sp, rows, hd)
        print("fa full size", sp, rows, hd, "restatement agrees")

    # benchmark configuration 1, exactly: scatter of the newest token, then attention
    spec = workloads.config_spec(1)
    c = workloads.decode_case(spec)
    gk, gv = trc.InferenceEngine.nd_inference(c["key"], c["value"], c["key_cache"], c["value_cache"],
                                              c["slot_mapping"])
    gen = tpa.PagedAttentionDataGenerator(0)
    golden = gen.compute_golden_reference(c["query"], gk, gv, c["block_tables"], np.ones(spec.batch, np.int32),
                                          c["context_lens"], 1.0 / math.sqrt(spec.head_size), None, 0)
    np.savez_compressed(os.path.join(HERE, "config1.npz"), golden=np.asarray(golden),
                        context_lens=c["context_lens"], sha_key_cache=np.array(cases.digest(gk)),
                        sha_value_cache=np.array(cases.digest(gv)), sha_query=np.array(cases.digest(c["query"])),
                        sha_in_key_cache=np.array(cases.digest(c["key_cache"])))
    print("config1", golden.dtype, golden.shape, c["context_lens"])


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
