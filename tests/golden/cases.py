"""Case tables shared by the fixture generator (make_golden.py) and the parity tests.

ST_CASES: seeds, shapes and mask types of the reference's own decode tests
(tests/st/test_custom_paged_attention.py:1562-2311).  Tuple layout:
(seed, q heads, kv heads, head size, block size, num blocks, context lens,
 q dtype, kv dtype or None (= q dtype), quant_type, has_quant_offset,
 qk_scale or None (= 1/sqrt(head size)), mask_type)
"""
import hashlib

import numpy as np

L4 = [192, 193, 194, 195]
ST_CASES = {
    "basic_fp16": (3001, 32, 1, 128, 128, 64, L4, "float16", None, 0, False, 1.0, 0),
    "basic_bf16": (3001, 32, 1, 128, 128, 64, L4, "bfloat16", None, 0, False, 1.0, 0),
    "no_mask_mha": (4115, 32, 32, 128, 128, 64, L4, "float16", None, 0, False, 1.0, 0),
    "norm_mask_fp16": (4116, 32, 32, 128, 128, 64, L4, "float16", None, 0, False, None, 1),
    "norm_mask_bf16": (4116, 32, 32, 128, 128, 64, L4, "bfloat16", None, 0, False, None, 1),
    "alibi_fp16": (4100, 32, 32, 128, 128, 64, [500, 500], "float16", None, 0, False, None, 2),
    "alibi_bf16": (4100, 32, 32, 128, 128, 64, [500, 500], "bfloat16", None, 0, False, None, 2),
    "gqa_8to1_alibi": (4101, 8, 1, 128, 128, 1024, [88] * 13, "float16", None, 0, False, None, 2),
    "gqa_4to2_alibi": (4102, 4, 2, 128, 128, 1024, [88] * 13, "float16", None, 0, False, None, 2),
    "gqa_32to8_alibi": (4103, 32, 8, 128, 128, 1024, [88] * 13, "float16", None, 0, False, None, 2),
    "odd_heads": (4104, 7, 7, 128, 128, 1024, [88] * 13, "float16", None, 0, False, None, 1),
    "heads_20_bf16": (4110, 20, 20, 128, 128, 64, [500, 500], "bfloat16", None, 0, False, None, 1),
    "head_256_block_16": (4107, 16, 16, 256, 16, 512, L4, "float16", None, 0, False, None, 0),
    "block_16": (4108, 32, 32, 128, 16, 512, L4, "float16", None, 0, False, None, 0),
    "small_seqlen": (4105, 32, 32, 128, 128, 64, [33, 33, 33, 33], "float16", None, 0, False, None, 1),
    "large_seqlen_bf16": (4106, 32, 32, 128, 128, 128, [3000, 3000], "bfloat16", None, 0, False, None, 1),
    "varied_seqlens": (4111, 32, 32, 128, 128, 256, [100, 500, 1000, 2000], "float16", None, 0, False, None, 1),
    "int8_kv": (3003, 32, 1, 128, 128, 64, L4, "float16", "int8", 1, False, None, 0),
    "int8_kv_offset": (3004, 32, 1, 128, 128, 64, L4, "float16", "int8", 1, True, None, 0),
    "gqa_int8_bf16": (4112, 32, 8, 128, 128, 64, L4, "bfloat16", "int8", 1, False, None, 1),
    "gqa_int8_offset": (4113, 32, 8, 128, 128, 64, L4, "float16", "int8", 1, True, None, 1),
    "bf16_int8_768": (6001, 32, 32, 128, 128, 256, [768], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_len128": (6002 + 128, 24, 24, 64, 128, 256, [128], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_len513": (6002 + 513, 24, 24, 64, 128, 256, [513], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_len1025": (6002 + 1025, 24, 24, 64, 128, 256, [1025], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_head32": (6100 + 32, 32, 32, 32, 16, 512, [512], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_head33": (6100 + 33, 32, 32, 33, 16, 512, [512], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_head128": (6100 + 128, 32, 32, 128, 16, 512, [512], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_gqa_4to1": (6200 + 401, 4, 1, 128, 128, 512, [766], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_gqa_24to2": (6200 + 2402, 24, 2, 128, 128, 512, [766], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_gqa_64to32": (6200 + 6432, 64, 32, 128, 128, 512, [766], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_block16": (6300 + 16, 32, 8, 64, 16, 1024, [1024], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_block128": (6300 + 128, 32, 8, 64, 128, 1024, [1024], "bfloat16", "int8", 1, False, None, 1),
    "bf16_int8_len309": (6400, 64, 64, 32, 16, 256, [309], "bfloat16", "int8", 1, False, None, 1),
}

# reshape_and_cache cases: (dtype, key rank, key head dim, value head dim, seed); cache geometry of
# tests/st/test_custom_reshape_and_cache.py:50-56 (20 blocks x 64 slots, 16 heads, 39 tokens)
RAC_CASES = {
    "fp16_rank3": ("float16", 3, 32, 32, 101),
    "fp16_rank2": ("float16", 2, 32, 32, 102),
    "bf16_rank3": ("bfloat16", 3, 32, 32, 103),
    "int8_rank2": ("int8", 2, 32, 32, 104),
    "fp16_kv_dims_differ": ("float16", 3, 32, 48, 105),
}


# multi-token (speculative) query cases: (seed, heads, kv_heads, head_size, block_size, num_blocks,
#   q_seq_lens, context_lens, dtype, qk_scale); SPEC mask.  Shapes of the reference's MTP / lookahead tests
#   (tests/st/test_custom_paged_attention.py:1673-1696, 2753-2830).
MTP_CASES = {
    "spec_mtp_fp16": (3002, 32, 1, 128, 128, 64, [2, 2, 2, 2], [192, 193, 194, 195], "float16", 0.01),
    "spec_mtp_bf16": (3002, 32, 1, 128, 128, 64, [2, 2, 2, 2], [192, 193, 194, 195], "bfloat16", 0.01),
    "lookahead_mixed": (9001, 32, 32, 128, 128, 64, [1, 15, 30, 6], [10, 64, 64, 64], "float16", None),
    "lookahead_block16": (9003, 32, 32, 128, 16, 256, [1, 15, 30, 6], [10, 64, 64, 64], "float16", None),
    "lookahead_gqa_bf16": (9004, 16, 4, 64, 32, 128, [3, 1, 8], [515, 40, 1300], "bfloat16", None),
    # tests/st/test_custom_paged_attention.py:2853-2875 (contexts up to 33,331 tokens) and :2878-2900 (GQA 32 / 8)
    "lookahead_very_long": (5005, 40, 40, 128, 128, 1234, [1, 1, 1], [13333, 23333, 33331], "float16", None),
    "lookahead_gqa_32to8": (5006, 32, 8, 128, 128, 512, [1, 15, 30, 6], [10, 64, 64, 64], "float16", None),
}


def mtp_case(name):
    from tests.golden import st_inputs
    seed, h, kvh, hd, bs, nb, qlens, lens, dt, scale = MTP_CASES[name]
    return st_inputs.st_style_case(seed, h, kvh, hd, bs, nb, lens, dt, None, 0, False, 3, scale, q_seq_lens=qlens)


def st_case(name, mask_free=False):
    from tests.golden import st_inputs
    seed, h, kvh, hd, bs, nb, lens, qd, kvd, quant, off, scale, mask = ST_CASES[name]
    return st_inputs.st_style_case(seed, h, kvh, hd, bs, nb, lens, qd, kvd, quant, off, 0 if mask_free else mask,
                                   scale)


def rac_case(name):
    """Seeded inputs in the reference test's shapes; slots are a permutation as in :207-210."""
    import ml_dtypes
    dtype, rank, khd, vhd, seed = RAC_CASES[name]
    rng = np.random.default_rng(seed)
    nb, bs, heads, batch, seq = 20, 64, 16, 13, 3
    t = batch * seq
    npdt = {"float16": np.float16, "bfloat16": ml_dtypes.bfloat16, "int8": np.int8}[dtype]

    def rnd(shape):
        if dtype == "int8":
            return rng.integers(-128, 127, shape, dtype=np.int8)
        return rng.random(shape, dtype=np.float32).astype(npdt)
    kshape = (t, heads * khd) if rank == 2 else (batch, seq, heads * khd)
    vshape = (t, heads * vhd) if rank == 2 else (batch, seq, heads * vhd)
    return {"key": rnd(kshape), "value": rnd(vshape), "key_cache": rnd((nb, bs, heads, khd)),
            "value_cache": rnd((nb, bs, heads, vhd)),
            "slot_mapping": rng.permutation(t).astype(np.int32)}


# reshape_and_cache_npd cases, head-major ("BNSD") cache: (dtype, heads, head_dim, batch, seed); geometry of
# tests/st/test_custom_reshape_and_cache_npd.py:51-58, 620-626 (16 tokens per sequence, pages of 16 slots)
RACNPD_CASES = {
    "fp16_h32_d128_b13": ("float16", 32, 128, 13, 201),
    "bf16_h8_d256_b2": ("bfloat16", 8, 256, 2, 202),
    "int8_h4_d32_b16": ("int8", 4, 32, 16, 203),
    "fp16_h8_d128_b8_pad": ("float16", 8, 128, 8, 204),   # with -1 slots (padding tokens)
}


def racnpd_case(name):
    import ml_dtypes
    dtype, heads, hd, batch, seed = RACNPD_CASES[name]
    rng = np.random.default_rng(seed)
    seq = slot_size = 16
    t, pages = batch * seq, batch
    npdt = {"float16": np.float16, "bfloat16": ml_dtypes.bfloat16, "int8": np.int8}[dtype]

    def rnd(shape):
        if dtype == "int8":
            return rng.integers(-128, 127, shape, dtype=np.int8)
        return rng.random(shape, dtype=np.float32).astype(npdt)
    slots = rng.permutation(pages * slot_size)[:t].astype(np.int32)
    if name.endswith("_pad"):
        slots[rng.random(t) < 0.2] = -1
    return {"key": rnd((t, heads * hd)), "value": rnd((t, heads * hd)), "key_cache": rnd((pages, heads, slot_size, hd)),
            "value_cache": rnd((pages, heads, slot_size, hd)), "slot_mapping": slots}


# paged_cache_load cases: (key dtype, value dtype, cumulative lengths + seq_starts, seed,
#   (num_blocks, block_size, heads, head_size_k, head_size_v, batch, max_len)).
# "ref" geometry = tests/st/test_custom_paged_cache_load.py:268 ([128, 128, 16, 144, 128, 16, 1], lengths 1..1024)
_PCL_REF = (128, 128, 16, 144, 128, 16, 1024)
PCL_CASES = {
    "fp16_fp16_lens": ("float16", "float16", False, 201, _PCL_REF),
    "bf16_int8_cumsum_starts": ("bfloat16", "int8", True, 202, _PCL_REF),
    "int8_fp16_cumsum_starts": ("int8", "float16", True, 203, (32, 16, 4, 24, 40, 9, 150)),
    "fp16_rows_2byte": ("float16", "float16", False, 204, (24, 8, 3, 5, 7, 7, 60)),
    "fp16_int8_rows_1byte": ("float16", "int8", True, 205, (24, 8, 3, 5, 7, 7, 60)),
    "bf16_bf16_block16": ("bfloat16", "bfloat16", False, 206, (256, 16, 8, 128, 128, 12, 300)),
}

# fa_update cases: (sp, rows, head_size, seed); shapes of tests/st/test_asd_faupdate.py:80-123 scaled in rows
FA_CASES = {
    "base_sp1": (1, 11 * 13, 8, 301),
    "sp3_head128": (3, 260, 128, 302),
    "sp8_head64": (8, 77, 64, 303),
    "sp2_head512": (2, 19, 512, 304),
}


def pcl_case(name):
    """Seeded inputs laid out like the reference test's generate_data_nd (:112-166): caches of small
    integers, random block tables with 4 spare columns, seq_starts a multiple of block_size."""
    import ml_dtypes
    kd, vd, cumsum, seed, (nb, bs, heads, dk, dv, batch, max_len) = PCL_CASES[name]
    rng = np.random.default_rng(seed)
    npdt = {"float16": np.float16, "bfloat16": ml_dtypes.bfloat16, "int8": np.int8}
    kc = rng.integers(1, 11, (nb, bs, heads, dk)).astype(npdt[kd])
    vc = rng.integers(1, 11, (nb, bs, heads, dv)).astype(npdt[vd])
    lens = rng.integers(1, max_len + 1, batch)
    cols = (int(lens.max()) + bs - 1) // bs + 4
    tables = rng.integers(0, nb, (batch, cols)).astype(np.int32)
    out = {"key_cache": kc, "value_cache": vc, "block_tables": tables, "cumsum": cumsum}
    if cumsum:
        out["seq_lens"] = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        out["seq_starts"] = (rng.integers(0, 5, batch) * bs).astype(np.int32)
    else:
        out["seq_lens"] = lens.astype(np.int32)
        out["seq_starts"] = None
    return out


def fa_case(name):
    """lse and partial outputs uniform in [0, 1) as in tests/st/test_asd_faupdate.py:67-70."""
    sp, rows, hd, seed = FA_CASES[name]
    rng = np.random.default_rng(seed)
    return {"lse": rng.random((sp, rows), dtype=np.float32), "local_out": rng.random((sp, rows, hd), dtype=np.float32),
            "sp": sp}


def digest(a) -> str:
    a = np.ascontiguousarray(a)
    return hashlib.sha256(a.view(np.uint8).tobytes()).hexdigest()
