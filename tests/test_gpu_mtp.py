"""GPU: multi-token (speculative) queries, calc_type = 1 with the SPEC mask, against the stored outputs
of the reference's golden and the oracle."""
import os

import numpy as np
import pytest
import torch

import ms_custom_ops_b200 as ops
from ms_custom_ops_b200 import workloads
from oracle import paged_kv_numpy as oracle
from tests.golden import cases, st_inputs
from tests.helpers import assert_close, to_dev, to_np, tol_for

pytestmark = pytest.mark.gpu
GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _run(c, with_mask=True):
    v = st_inputs.operator_view(c)
    kw = dict(q_head_num=c["num_heads"], kv_head_num=c["kv_heads"], qk_scale=c["qk_scale"], calc_type=1,
              q_seq_lens=torch.from_numpy(c["q_seq_lens"]))
    if with_mask:
        kw.update(mask_type=3, attn_mask=to_dev(v["mask"]))
    out = ops.paged_attention(to_dev(v["query"]), to_dev(v["key_cache"]), to_dev(v["value_cache"]),
                              to_dev(v["block_tables"]), torch.from_numpy(c["context_lens"]), **kw)
    ops.paged_attention_check_status()
    return v, to_np(out)


@pytest.mark.parametrize("name", sorted(cases.MTP_CASES))
def test_multi_token_queries_match_reference_golden(name):
    c = cases.mtp_case(name)
    fx = np.load(os.path.join(GOLDEN_DIR, "pa_mtp_" + name + ".npz"))
    assert cases.digest(c["query"]) == str(fx["sha_query"])
    v, out = _run(c)
    assert out.shape == fx["golden"].shape
    ok, detail = oracle.reference_accuracy_verdict(out, fx["golden"], c["q_dtype"], c["num_heads"],
                                                   int(max(c["context_lens"])))
    assert ok, (name, detail)
    g = oracle.paged_attention_golden(v["query"], v["key_cache"], v["value_cache"], v["block_tables"],
                                      c["context_lens"], c["qk_scale"], mask=v["mask"], mask_type=3,
                                      q_seq_lens=c["q_seq_lens"])
    assert_close(out, g, tol_for(c["q_dtype"], False), name)


def test_multi_token_queries_without_mask_and_with_empty_sequences():
    # no mask: every token of a sequence sees the whole context; q_len 0 and context 0 are legal
    c = st_inputs.st_style_case(77, 8, 2, 128, 16, 64, [40, 0, 130, 17], "bfloat16", None, 0, False, 0, None,
                                q_seq_lens=[3, 2, 0, 4])
    v, out = _run(c, with_mask=False)
    g = oracle.paged_attention_golden(v["query"], v["key_cache"], v["value_cache"], v["block_tables"],
                                      c["context_lens"], c["qk_scale"], q_seq_lens=c["q_seq_lens"])
    assert out.shape == (9, 8, 128)
    assert_close(out, g, 1e-2, "mask-free multi-token")
    assert not out[3:5].any()  # the sequence with an empty context
    # one token per sequence is plain decode
    c1 = st_inputs.st_style_case(78, 8, 2, 128, 16, 64, [40, 9, 130], "float16", None, 0, False, 0, None,
                                 q_seq_lens=[1, 1, 1])
    v1, out1 = _run(c1, with_mask=False)
    plain = ops.paged_attention(to_dev(v1["query"]), to_dev(v1["key_cache"]), to_dev(v1["value_cache"]),
                                to_dev(v1["block_tables"]), torch.from_numpy(c1["context_lens"]), q_head_num=8,
                                kv_head_num=2, qk_scale=c1["qk_scale"])
    assert np.array_equal(out1, to_np(plain))


@pytest.mark.parametrize("mask", [False, True])
@pytest.mark.parametrize("heads,kvh,dtype", [(32, 8, "bfloat16"), (16, 16, "float16"), (64, 8, "float16")])
def test_stacked_query_tokens_over_long_contexts(heads, kvh, dtype, mask):
    # several query tokens per sequence over contexts of several KV splits: the tokens of a sequence are
    # stacked into the q rows of one work item (one read of the context), partials are kept per token
    c = st_inputs.st_style_case(91, heads, kvh, 128, 128, 128, [5000, 1300, 700, 2049], dtype, None, 0, False,
                                3 if mask else 0, None, q_seq_lens=[4, 3, 9, 1])
    v, out = _run(c, with_mask=mask)
    g = oracle.paged_attention_golden(v["query"], v["key_cache"], v["value_cache"], v["block_tables"],
                                      c["context_lens"], c["qk_scale"], mask=v["mask"] if mask else None,
                                      mask_type=3 if mask else 0, q_seq_lens=c["q_seq_lens"])
    assert_close(out, g, tol_for(dtype, False), f"stacked {heads}/{kvh} mask={mask}")
    rel_max, rel_l2 = oracle.scale_free_error(out, g)
    assert rel_l2 < 1e-2, (rel_max, rel_l2)
