"""Inputs distributed like the reference's system tests (test infrastructure).

tests/st/test_custom_paged_attention.py:104-340 of the reference: uniform(-1, 1) query and caches,
int8 caches as clip(rint(u * 127 / 4)), i.i.d. random block tables, integer de-quantisation scales in
{-1, 0, 1} and offsets in [-20, 20), drawn in the same order from the same generators so that a given
seed reproduces the reference test's inputs bit for bit (asserted by make_golden.py when the fixtures
are made).
"""
from __future__ import annotations

import math
import random

import numpy as np

from ms_custom_ops_b200.workloads import NP_DTYPES, bfloat16


def st_style_case(seed, num_heads, kv_heads, head_size, block_size, num_blocks, context_lens,
                  q_dtype="float16", kv_dtype=None, quant_type=0, has_quant_offset=False,
                  mask_type=0, qk_scale=None, q_seq_lens=None):
    """Inputs of one reference-style decode test (one query token per sequence; with `q_seq_lens`
    several per sequence, the multi-token / speculative form with the SPEC mask, mask_type 3).

    Draw order and distributions follow the reference generator
    (tests/st/test_custom_paged_attention.py:87-92,176-190,196-246,280-299):
    numpy ``default_rng(seed)`` for tensors, Python ``random`` (same seed) for
    the block tables.  bf16 tensors are float32 draws rounded to bf16.
    """
    kv_dtype = kv_dtype or q_dtype
    rng = np.random.default_rng(seed)
    random.seed(seed)
    batch = len(context_lens)
    num_tokens = batch if q_seq_lens is None else int(sum(q_seq_lens))
    q32 = rng.uniform(-1.0, 1.0, (num_tokens, num_heads, head_size))
    if q_dtype == "float16":
        query = q32.astype(np.float16)
    else:
        query = q32.astype(np.float32).astype(bfloat16)
    shape = (num_blocks, block_size, kv_heads, head_size)
    if kv_dtype == "int8":
        kc = np.clip(np.rint(rng.uniform(-4.0, 4.0, shape).astype(np.float32) * 127.0 / 4.0), -127, 127).astype(np.int8)
        vc = np.clip(np.rint(rng.uniform(-4.0, 4.0, shape).astype(np.float32) * 127.0 / 4.0), -127, 127).astype(np.int8)
    elif kv_dtype == "float16":
        kc = rng.uniform(-1.0, 1.0, shape).astype(np.float16)
        vc = rng.uniform(-1.0, 1.0, shape).astype(np.float16)
    else:  # the reference keeps bf16 caches as raw float32 draws; the operator sees them rounded
        kc = rng.uniform(-1.0, 1.0, shape).astype(np.float32)
        vc = rng.uniform(-1.0, 1.0, shape).astype(np.float32)
    max_blocks = (max(context_lens) + block_size - 1) // block_size
    tables = np.array([[random.randint(0, num_blocks - 1) for _ in range(max_blocks)] for _ in range(batch)],
                      dtype=np.int32).reshape(batch, max_blocks)
    mask = None
    if mask_type == 1:  # NORM decode mask (:430-447)
        mask = np.zeros((batch, 1, max(context_lens)), dtype=np.float32)
        for i in range(1, batch):
            mask[i, :, :i] = -10000.0
    elif mask_type == 2:  # ALIBI (:465-507, slopes :340-368)
        p2 = 2 ** int(np.floor(np.log2(num_heads)))
        m0 = 2.0 ** (-8.0 / p2)
        slopes = np.array([m0 ** i for i in range(1, p2 + 1)], dtype=np.float32)
        if p2 < num_heads:
            m1 = 2.0 ** (-4.0 / p2)
            extra = np.array([m1 ** i for i in range(1, 1 + 2 * (num_heads - p2), 2)], dtype=np.float32)
            slopes = np.concatenate([slopes, extra])
        mask = np.zeros((batch, num_heads, 1, max(context_lens)), dtype=np.float32)
        for i, kl in enumerate(context_lens):
            if kl:
                bias = (np.arange(kl, dtype=np.int32) - kl + 1).astype(np.float32)
                mask[i, :, :, :kl] = slopes.reshape(-1, 1, 1) * bias.reshape(1, 1, -1)
    elif mask_type == 3:  # SPEC (:509-524): causal inside the window of the last q_len context positions
        ql_all = [1] * batch if q_seq_lens is None else list(q_seq_lens)
        mask = np.zeros((num_tokens, max(context_lens)), dtype=np.float32)
        pre = 0
        for ql, kl in zip(ql_all, context_lens):
            if ql and kl:
                start = max(0, kl - ql)
                mask[pre:pre + ql, start:kl] = np.triu(np.ones((ql, ql), dtype=np.float32), 1) * -10000.0
            pre += ql
    k_descale = v_descale = k_offset = v_offset = None
    if quant_type == 1:
        k_descale = rng.integers(-1, 2, size=(kv_heads * head_size,)).astype(np.float32)
        v_descale = rng.integers(-1, 2, size=(kv_heads * head_size,)).astype(np.float32)
        if has_quant_offset:
            k_offset = rng.integers(-20, 20, size=(kv_heads * head_size,)).astype(np.int32)
            v_offset = rng.integers(-20, 20, size=(kv_heads * head_size,)).astype(np.int32)
    return {
        "query": query, "key_cache": kc, "value_cache": vc, "block_tables": tables,
        "context_lens": np.array(context_lens, dtype=np.int32), "mask": mask, "mask_type": mask_type,
        "q_seq_lens": None if q_seq_lens is None else np.array(q_seq_lens, dtype=np.int32),
        "k_descale": k_descale, "v_descale": v_descale, "k_offset": k_offset, "v_offset": v_offset,
        "q_dtype": q_dtype, "kv_dtype": kv_dtype, "quant_type": quant_type,
        "has_quant_offset": has_quant_offset,
        "qk_scale": (1.0 / math.sqrt(head_size)) if qk_scale is None else qk_scale,
        "num_heads": num_heads, "kv_heads": kv_heads, "head_size": head_size, "block_size": block_size,
    }


def operator_view(case):
    """The tensors as the operator receives them (bf16 caches rounded to bf16)."""
    out = dict(case)
    if case["kv_dtype"] == "bfloat16" and case["key_cache"].dtype == np.float32:
        out["key_cache"] = case["key_cache"].astype(bfloat16)
        out["value_cache"] = case["value_cache"].astype(bfloat16)
    if case["mask"] is not None:
        out["mask"] = case["mask"].astype(NP_DTYPES[case["q_dtype"]])
    return out
