"""GPU parity of paged_cache_load and fa_update (the operators either side of the decode path)."""
import os

import numpy as np
import pytest
import torch

import ms_custom_ops_b200 as ops
from ms_custom_ops_b200 import _abi, kernels
from oracle import paged_kv_numpy as oracle
from tests.golden import cases
from tests.helpers import to_dev, to_np

pytestmark = pytest.mark.gpu
GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _fixture(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


def reference_compare(output, expect, limit):
    """The reference's acceptance rule (tests/st/st_utils.py:23-49): at most `limit` of the elements
    may be off by more than `limit` relatively."""
    o, e = np.asarray(output, np.float64).ravel(), np.asarray(expect, np.float64).ravel()
    with np.errstate(divide="ignore", invalid="ignore"):
        bad = int(np.sum(np.abs(o - e) / np.abs(e) > limit))
    return bad <= int(o.size * limit)


# ----------------------------------------------------------------------------- paged_cache_load
@pytest.mark.parametrize("name", sorted(cases.PCL_CASES))
def test_paged_cache_load_reference_fixtures_bit_exact(name):
    # outputs of the reference's own golden_calc_nd on these inputs, stored as digests
    c, fx = cases.pcl_case(name), _fixture("pcl_" + name)
    assert cases.digest(c["key_cache"]) == str(fx["sha_in_key_cache"])
    assert cases.digest(c["block_tables"]) == str(fx["sha_in_block_tables"])
    starts = None if c["seq_starts"] is None else to_dev(c["seq_starts"])
    k, v = ops.paged_cache_load(to_dev(c["key_cache"]), to_dev(c["value_cache"]), to_dev(c["block_tables"]),
                                torch.from_numpy(c["seq_lens"]), starts, 0, c["cumsum"], c["cumsum"])
    assert k.shape[0] == int(fx["rows"]) and v.shape[0] == int(fx["rows"])
    assert k.shape[1:] == c["key_cache"].shape[2:] and v.shape[1:] == c["value_cache"].shape[2:]
    assert cases.digest(to_np(k)) == str(fx["sha_key_out"])
    assert cases.digest(to_np(v)) == str(fx["sha_value_out"])


@pytest.mark.parametrize("cumsum,with_starts", [(False, False), (True, False), (False, True), (True, True)])
def test_paged_cache_load_flag_combinations_against_oracle(cumsum, with_starts):
    # the operator has one flag for cumulative lengths and one for seq_starts; the reference's golden
    # only exercises both-or-neither
    rng = np.random.default_rng(77 + 2 * cumsum + with_starts)
    nb, bs, heads, dk, dv, batch = 40, 16, 2, 64, 32, 11
    kc = rng.integers(-100, 100, (nb, bs, heads, dk)).astype(np.int8)
    vc = rng.standard_normal((nb, bs, heads, dv)).astype(np.float16)
    lens = rng.integers(0, 90, batch)  # zero-length sequences included
    tables = rng.integers(0, nb, (batch, 12)).astype(np.int32)
    seq_lens = (np.concatenate([[0], np.cumsum(lens)]) if cumsum else lens).astype(np.int32)
    starts = (rng.integers(0, 5, batch) * bs + rng.integers(0, bs, batch)).astype(np.int32) if with_starts else None
    gk, gv = oracle.paged_cache_load_golden(kc, vc, tables, seq_lens, starts, cumsum)
    k, v = ops.paged_cache_load(to_dev(kc), to_dev(vc), to_dev(tables), to_dev(seq_lens),
                                None if starts is None else to_dev(starts), 0, cumsum, with_starts)
    assert np.array_equal(to_np(k), gk) and np.array_equal(to_np(v), gv)


def test_paged_cache_load_negative_block_ids_compact_and_zero_the_tail():
    # blocks with a negative id contribute no rows, later rows move up, the rest stays zero
    rng = np.random.default_rng(5)
    nb, bs, heads, d, batch = 16, 8, 2, 16, 6
    kc = rng.integers(1, 100, (nb, bs, heads, d)).astype(np.int8)
    vc = rng.integers(1, 100, (nb, bs, heads, d)).astype(np.int8)
    lens = np.array([20, 8, 1, 33, 16, 7], np.int32)
    tables = rng.integers(0, nb, (batch, 6)).astype(np.int32)
    tables[0, 1] = -1
    tables[3, 0] = -1
    tables[3, 4] = -7
    tables[5, 0] = -1
    gk, gv = oracle.paged_cache_load_golden(kc, vc, tables, lens)
    assert not gk[-1].any() and gk[0].any()
    k, v = ops.paged_cache_load(to_dev(kc), to_dev(vc), to_dev(tables), torch.from_numpy(lens))
    assert np.array_equal(to_np(k), gk) and np.array_equal(to_np(v), gv)


def test_paged_cache_load_out_of_range_ids_are_counted_not_read():
    nb, bs, heads, d, batch = 8, 4, 1, 16, 3
    kc = torch.arange(nb * bs * heads * d, dtype=torch.int32, device="cuda").to(torch.int8).view(nb, bs, heads, d)
    vc = kc.clone()
    tables = torch.tensor([[0, 1, 2], [99, 3, 4], [5, 6, 7]], dtype=torch.int32, device="cuda")
    lens = torch.tensor([12, 12, 30], dtype=torch.int32, device="cuda")  # row 2 needs 8 columns, has 3
    rows = 54
    ko = torch.full((rows, heads, d), 7, dtype=torch.int8, device="cuda")
    vo = torch.full((rows, heads, d), 7, dtype=torch.int8, device="cuda")
    ws = torch.empty(kernels.cache_load_workspace_bytes(batch, 3), dtype=torch.uint8, device="cuda")
    oob = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.cache_load(kc, vc, tables, lens, None, ko, vo, ws, False, oob)
    torch.cuda.synchronize()
    assert int(oob.item()) == 1 + 5  # one id past the cache, five columns past the table
    want = torch.cat([kc[0], kc[1], kc[2], kc[3], kc[4], kc[5], kc[6], kc[7]]).view(-1, heads, d)
    assert torch.equal(ko[:32], want) and not ko[32:].any()
    assert torch.equal(vo[:32], want) and not vo[32:].any()


def test_paged_cache_load_round_trip_with_reshape_and_cache():
    # scatter rows into the cache through reshape_and_cache, gather them back: same bytes
    rng = np.random.default_rng(9)
    nb, bs, heads, d, batch = 64, 32, 8, 128, 5
    lens = np.array([100, 1, 64, 33, 250], np.int32)
    blocks_per = [(n + bs - 1) // bs for n in lens]
    perm = rng.permutation(nb)
    tables = np.zeros((batch, max(blocks_per)), np.int32)
    slots, p = [], 0
    for i, nblk in enumerate(blocks_per):
        tables[i, :nblk] = perm[p:p + nblk]
        p += nblk
        slots += [int(tables[i, j // bs]) * bs + j % bs for j in range(lens[i])]
    total = int(lens.sum())
    key = torch.randn(total, heads * d, device="cuda").to(torch.bfloat16)
    val = torch.randn(total, heads * d, device="cuda").to(torch.bfloat16)
    kc = torch.zeros(nb, bs, heads, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.reshape_and_cache(key, val, kc, vc, torch.tensor(slots, dtype=torch.int32, device="cuda"))
    k, v = ops.paged_cache_load(kc, vc, to_dev(tables), torch.from_numpy(lens))
    assert torch.equal(k.view(total, -1), key) and torch.equal(v.view(total, -1), val)


def test_paged_cache_load_empty_and_errors():
    kc = torch.zeros(4, 8, 2, 16, dtype=torch.float16, device="cuda")
    tables = torch.zeros(2, 3, dtype=torch.int32, device="cuda")
    k, v = ops.paged_cache_load(kc, kc, tables, np.zeros(2, np.int32))
    assert k.shape == (0, 2, 16) and v.shape == (0, 2, 16)
    with pytest.raises(ops.MscoError, match="seq_lens dtype must be int32"):
        ops.paged_cache_load(kc, kc, tables, np.ones(2, np.int64))
    with pytest.raises(ops.UnsupportedOnB200):
        ops.paged_cache_load(kc, kc, tables, np.ones(2, np.int32), None, 1)
    with pytest.raises(ValueError, match="seq_starts"):
        ops.paged_cache_load(kc, kc, tables, np.ones(2, np.int32), None, 0, False, True)
    with pytest.raises(ValueError, match="3 elements"):
        ops.paged_cache_load(kc, kc, tables, np.ones(2, np.int32), None, 0, True, False)
    small = torch.empty(8, dtype=torch.uint8, device="cuda")
    out = torch.empty(2, 2, 16, dtype=torch.float16, device="cuda")
    with pytest.raises(_abi.MscoError, match="workspace too small"):
        kernels.cache_load(kc, kc, tables, to_dev(np.ones(2, np.int32)), None, out, out.clone(), small)


# ----------------------------------------------------------------------------- fa_update
@pytest.mark.parametrize("name", sorted(cases.FA_CASES))
def test_fa_update_reference_fixtures(name):
    c, fx = cases.fa_case(name), _fixture("fa_" + name)
    assert cases.digest(c["lse"]) == str(fx["sha_lse"])
    out = ops.fa_update(to_dev(c["lse"]), to_dev(c["local_out"]), 0, c["sp"])
    assert out.dtype == torch.float32 and tuple(out.shape) == fx["golden"].shape
    o = to_np(out)
    assert reference_compare(o, fx["golden"], 1e-4)  # the reference's float32 limit
    np.testing.assert_allclose(o, fx["golden"], rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("sp,rows,hd", [(3, 1000 * 13, 128), (3, 2 * 4000 * 32, 128), (8, 4096, 512), (5, 333, 40)])
def test_fa_update_reference_shapes_against_oracle(sp, rows, hd):
    # tests/st/test_asd_faupdate.py:95-123 at full size (13000 and 256000 rows), and the extremes
    g = torch.Generator(device="cuda").manual_seed(sp * rows)
    lse = torch.rand(sp, rows, device="cuda", generator=g) * 6 - 3
    lo = torch.rand(sp, rows, hd, device="cuda", generator=g)
    out = ops.fa_update(lse, lo, 0, sp)
    golden = oracle.fa_update_golden(to_np(lse), to_np(lo))
    np.testing.assert_allclose(to_np(out), golden, rtol=3e-6, atol=1e-7)


def test_fa_update_is_the_merge_of_split_attention():
    # attention over a context == fa_update of attention over its parts, with lse = log(sum exp)
    rng = np.random.default_rng(3)
    rows, d, ctx, sp = 24, 64, 96, 4
    q = rng.standard_normal((rows, d)).astype(np.float32)
    k = rng.standard_normal((ctx, d)).astype(np.float32)
    v = rng.standard_normal((ctx, d)).astype(np.float32)
    s = q @ k.T / np.sqrt(d)
    full = (np.exp(s - s.max(1, keepdims=True)) / np.exp(s - s.max(1, keepdims=True)).sum(1, keepdims=True)) @ v
    lses, outs = [], []
    for part in np.array_split(np.arange(ctx), sp):
        sp_ = s[:, part]
        e = np.exp(sp_)
        lses.append(np.log(e.sum(1)))
        outs.append((e / e.sum(1, keepdims=True)) @ v[part])
    out = ops.fa_update(to_dev(np.stack(lses).astype(np.float32)), to_dev(np.stack(outs).astype(np.float32)), 0, sp)
    np.testing.assert_allclose(to_np(out), full, rtol=2e-5, atol=2e-6)


def test_fa_update_partitions_without_tokens_and_large_lse():
    # lse = -inf marks a partition that saw no token; huge lse must not overflow
    lse = torch.tensor([[-float("inf"), 500.0, -float("inf")], [0.0, 499.0, -float("inf")]], device="cuda")
    lo = torch.ones(2, 3, 8, device="cuda")
    lo[1] *= 3
    out = to_np(ops.fa_update(lse, lo, 0, 2))
    w = 1 / (1 + np.exp(-1.0))
    np.testing.assert_allclose(out[0], 3.0, rtol=1e-6)
    np.testing.assert_allclose(out[1], w * 1 + (1 - w) * 3, rtol=1e-6)
    assert not out[2].any()


def test_fa_update_errors():
    lse = torch.zeros(2, 5, device="cuda")
    with pytest.raises(ValueError, match="local_out dim must be 3"):
        ops.fa_update(lse, torch.zeros(2, 40, device="cuda"), 0, 2)
    with pytest.raises(ValueError, match="multiple of 8"):
        ops.fa_update(lse, torch.zeros(2, 5, 12, device="cuda"), 0, 2)
    with pytest.raises(ValueError, match="sp is 3"):
        ops.fa_update(lse, torch.zeros(2, 5, 8, device="cuda"), 0, 3)
    with pytest.raises(ValueError, match="fa_update_type"):
        ops.fa_update(lse, torch.zeros(2, 5, 8, device="cuda"), 1, 2)
    with pytest.raises(TypeError):
        ops.fa_update(lse.half(), torch.zeros(2, 5, 8, device="cuda"), 0, 2)
