"""GPU: the log-sum-exp output of paged attention and the sequence-sharded decode built on it
(attention over parts of every context, merged by fa_update).  One GPU: the ranks' launches run one
after another on the same caches."""
import numpy as np
import pytest
import torch

import ms_custom_ops_b200 as ops
from ms_custom_ops_b200 import _abi, kernels, sharding, workloads
from oracle import paged_kv_numpy as oracle
from tests.golden import cases, st_inputs
from tests.helpers import assert_close, to_dev, to_np, tol_for

pytestmark = pytest.mark.gpu


def _golden_with_lse(v):
    return oracle.paged_attention_golden(
        v["query"], v["key_cache"], v["value_cache"], v["block_tables"], v["context_lens"], v["qk_scale"],
        v["k_descale"], v["v_descale"], v["k_offset"], v["v_offset"], v["mask"], v.get("mask_type", 0),
        return_lse=True)


@pytest.mark.parametrize("kernel", [_abi.KERNEL_GENERIC, _abi.KERNEL_TMA])
@pytest.mark.parametrize("name", ["basic_fp16", "basic_bf16", "gqa_32to8_alibi", "norm_mask_bf16", "varied_seqlens",
                                  "int8_kv_offset", "gqa_int8_bf16", "bf16_int8_gqa_24to2", "bf16_int8_len1025",
                                  "large_seqlen_bf16"])
def test_lse_output_matches_oracle(name, kernel):
    v = st_inputs.operator_view(cases.st_case(name))
    q = to_dev(v["query"])
    lse = torch.full(q.shape[:2], 12345.0, dtype=torch.float32, device="cuda")
    try:
        out, info = kernels.paged_attention_raw(
            q, to_dev(v["key_cache"]), to_dev(v["value_cache"]), to_dev(v["block_tables"]),
            [int(x) for x in v["context_lens"]], v["qk_scale"], v["quant_type"], to_dev(v["k_descale"]),
            to_dev(v["k_offset"]), to_dev(v["v_descale"]), to_dev(v["v_offset"]), to_dev(v["mask"]),
            v.get("mask_type", 0), kernel, lse=lse)
    except _abi.MscoError as e:
        if e.code == _abi.ERR_UNSUPPORTED:
            pytest.skip("shape not covered by this kernel")
        raise
    assert info.kernel == kernel
    g, g_lse = _golden_with_lse(v)
    quant = v["quant_type"] != 0
    assert_close(to_np(out), g, tol_for(v["q_dtype"], quant), name)
    # scores of the reference's int8 cases reach several hundred: relative tolerance on top of 2e-2
    np.testing.assert_allclose(to_np(lse), g_lse, rtol=1e-3, atol=2e-2)
    # the second output must not change the first
    out2, _ = kernels.paged_attention_raw(
        q, to_dev(v["key_cache"]), to_dev(v["value_cache"]), to_dev(v["block_tables"]),
        [int(x) for x in v["context_lens"]], v["qk_scale"], v["quant_type"], to_dev(v["k_descale"]),
        to_dev(v["k_offset"]), to_dev(v["v_descale"]), to_dev(v["v_offset"]), to_dev(v["mask"]),
        v.get("mask_type", 0), kernel)
    assert_close(to_np(out2), to_np(out).astype(np.float32), 2e-3 if quant else 0.0, name + "/with vs without lse")


def test_lse_of_an_empty_context_is_minus_infinity():
    q = torch.randn(3, 8, 128, device="cuda").half()
    kc = torch.randn(16, 16, 2, 128, device="cuda").half()
    tables = torch.zeros(3, 4, dtype=torch.int32, device="cuda")
    out, lse = ops.paged_attention_with_lse(q, kc, kc, tables, np.array([20, 0, 1], np.int32), q_head_num=8,
                                            kv_head_num=2, qk_scale=0.1)
    ops.paged_attention_check_status()
    lse = to_np(lse)
    assert np.isneginf(lse[1]).all() and np.isfinite(lse[0]).all() and np.isfinite(lse[2]).all()
    assert not to_np(out)[1].any()
    # one token: softmax weight 1, lse = its score
    s = (q[2].float() * kc[0, 0].float().repeat_interleave(4, 0)).sum(-1) * 0.1
    np.testing.assert_allclose(lse[2], to_np(s), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("config", [4, 3])
def test_sequence_sharded_decode_equals_unsharded(config, world):
    # benchmark configurations 4 (bf16, long skewed) and 3 (int8 KV) scaled down; every rank sees a
    # contiguous range of whole blocks of every sequence, short sequences leave ranks empty
    spec = workloads.config_spec(config, 0.15 if config == 4 else 0.1)
    v = workloads.decode_case(spec)
    lens = np.asarray(v["context_lens"], np.int32)
    lens[0] = 5  # shorter than one block: lives on the last rank only
    q, kc, vc = to_dev(v["query"]), to_dev(v["key_cache"]), to_dev(v["value_cache"])
    kw = dict(q_head_num=spec.num_heads, kv_head_num=spec.kv_heads, qk_scale=v["qk_scale"])
    if spec.kv_int8:
        kw.update(quant_type=1, k_descale=to_dev(v["k_descale"]), v_descale=to_dev(v["v_descale"]))
    full = ops.paged_attention(q, kc, vc, to_dev(v["block_tables"]), torch.from_numpy(lens), **kw)
    outs, lses = [], []
    for r in range(world):
        lt, ll = sharding.seq_shard_tables(v["block_tables"], lens, spec.block_size, r, world)
        o, l = ops.paged_attention_with_lse(q, kc, vc, to_dev(lt), torch.from_numpy(ll), **kw)
        outs.append(o.float().view(-1, spec.head_size))
        lses.append(l.view(-1))
    ops.paged_attention_check_status()
    merged = ops.fa_update(torch.stack(lses), torch.stack(outs), 0, world).view(full.shape)
    tol = tol_for(v["q_dtype"], spec.kv_int8)
    assert_close(to_np(merged), to_np(full).astype(np.float32), tol, f"c{config} merged vs unsharded, {world} ranks")
    g = oracle.paged_attention_golden(v["query"], v["key_cache"], v["value_cache"], v["block_tables"], lens,
                                      v["qk_scale"], v["k_descale"], v["v_descale"])
    assert_close(to_np(merged), g, tol, f"c{config} merged vs oracle, {world} ranks")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_strided_merge_of_gathered_records(dtype):
    # records as the sequence-sharded step all-gathers them: [output rows | lse], one per rank
    sp, rows, hd = 4, 96, 128
    es = torch.empty((), dtype=dtype).element_size()
    off_lse = (rows * hd * es + 255) // 256 * 256
    rec = (off_lse + rows * 4 + 255) // 256 * 256
    g = torch.zeros(sp, rec, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(4)
    outs = torch.randn(sp, rows, hd, device="cuda", generator=gen).to(dtype)
    lses = torch.randn(sp, rows, device="cuda", generator=gen) * 3
    lses[1, 5] = -float("inf")
    for s in range(sp):
        g[s, :rows * hd * es].view(dtype).view(rows, hd).copy_(outs[s])
        g[s, off_lse:off_lse + rows * 4].view(torch.float32).copy_(lses[s])
    merged = torch.empty(rows, hd, dtype=dtype, device="cuda")
    kernels.merge_partials_strided(g[0, off_lse:].view(torch.float32), rec // 4, g[0, :rows * hd * es].view(dtype),
                                   rec // es, merged, sp)
    want = oracle.fa_update_golden(to_np(lses), to_np(outs.float()))
    tol = {torch.float32: 1e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    np.testing.assert_allclose(to_np(merged.float()), want, rtol=tol, atol=tol)
    # and the packed float32 operator gives the same as the strided entry on packed float32 input
    if dtype == torch.float32:
        assert torch.equal(ops.fa_update(lses, outs, 0, sp), merged)
