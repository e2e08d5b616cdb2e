"""CPU: property tests (hypothesis) of the host-side bookkeeping and of the oracle's data movement."""
import numpy as np
from hypothesis import given, settings
from hypothesis import strategies as st

from ms_custom_ops_b200 import _abi, sharding
from oracle import paged_kv_numpy as oracle


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(0, 700), min_size=1, max_size=9), st.sampled_from([1, 16, 128]), st.integers(1, 8),
       st.integers(0, 2 ** 31 - 1))
def test_sequence_shards_partition_every_context(lens, bs, world, seed):
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, np.int32)
    cols = int((lens.max() + bs - 1) // bs) + 2
    tables = rng.integers(0, 1000, (len(lens), cols)).astype(np.int32)
    parts = [sharding.seq_shard_tables(tables, lens, bs, r, world) for r in range(world)]
    for b, n in enumerate(lens):
        assert sum(int(p[1][b]) for p in parts) == n
        used = np.concatenate([p[0][b, :(int(p[1][b]) + bs - 1) // bs] for p in parts])
        assert np.array_equal(used, tables[b, :(n + bs - 1) // bs])
        # only the last non-empty part may end with a partial block
        nonempty = [int(p[1][b]) for p in parts if int(p[1][b]) > 0]
        assert all(x % bs == 0 for x in nonempty[:-1])


def _naive_cache_load(kc, vc, tables, lens, starts, cumsum):
    # the reference's per-token loop (tests/st/test_custom_paged_cache_load.py:35-76), literally
    bs = kc.shape[1]
    lens = np.asarray(lens)
    total = int(lens[-1]) if cumsum else int(lens.sum())
    ko, vo = np.zeros((total,) + kc.shape[2:], kc.dtype), np.zeros((total,) + vc.shape[2:], vc.dtype)
    row, prev = 0, 0
    for i in range(tables.shape[0]):
        if cumsum:
            n, prev = int(lens[i + 1]) - prev, int(lens[i + 1])
        else:
            n = int(lens[i])
        off = 0 if starts is None else int(starts[i]) // bs
        for j in range(n):
            bid = int(tables[i][off + j // bs])
            if bid < 0:
                continue
            ko[row], vo[row] = kc[bid][j % bs], vc[bid][j % bs]
            row += 1
    return ko, vo


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.sampled_from([1, 4, 16]), st.integers(1, 6), st.booleans(), st.booleans())
def test_cache_load_oracle_equals_the_per_token_loop(seed, bs, batch, cumsum, with_starts):
    rng = np.random.default_rng(seed)
    nb = 12
    kc = rng.integers(-128, 128, (nb, bs, 2, 3)).astype(np.int8)
    vc = rng.integers(-128, 128, (nb, bs, 2, 5)).astype(np.int8)
    lens = rng.integers(0, 5 * bs + 1, batch)
    starts = (rng.integers(0, 3 * bs, batch)).astype(np.int32) if with_starts else None
    tables = rng.integers(-2, nb, (batch, 5 + 3)).astype(np.int32)  # negative ids: skipped blocks
    seq_lens = (np.concatenate([[0], np.cumsum(lens)]) if cumsum else lens).astype(np.int32)
    got = oracle.paged_cache_load_golden(kc, vc, tables, seq_lens, starts, cumsum)
    want = _naive_cache_load(kc, vc, tables, seq_lens, starts, cumsum)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.integers(1, 8), st.integers(1, 40), st.sampled_from([8, 64]))
def test_fa_update_oracle_is_a_convex_combination_and_splits_consistently(seed, sp, rows, hd):
    rng = np.random.default_rng(seed)
    lse = (rng.standard_normal((sp, rows)) * 4).astype(np.float32)
    parts = rng.standard_normal((sp, rows, hd)).astype(np.float32)
    out = oracle.fa_update_golden(lse, parts)
    assert np.all(out <= parts.max(0) + 1e-5) and np.all(out >= parts.min(0) - 1e-5)
    if sp >= 2:  # merging the first k partitions, then the rest, equals merging all at once
        k = sp // 2
        def merged_lse(x):
            m = x.max(0)
            return m + np.log(np.exp(x - m).sum(0))
        a, b = oracle.fa_update_golden(lse[:k], parts[:k]), oracle.fa_update_golden(lse[k:], parts[k:])
        two = oracle.fa_update_golden(np.stack([merged_lse(lse[:k]), merged_lse(lse[k:])]), np.stack([a, b]))
        np.testing.assert_allclose(two, out, rtol=2e-5, atol=2e-6)


@settings(max_examples=50, deadline=None)
@given(st.integers(1, 300000), st.sampled_from([_abi.DTYPE_F16, _abi.DTYPE_BF16, _abi.DTYPE_I8]))
def test_split_rule_is_a_function_of_length_and_dtype_only(n, dt):
    L = _abi.lib()
    t = L.msco_paged_attention_split_tokens(n, dt)
    assert t >= 512 and t % 128 == 0
    # a longer context never has fewer splits
    t1 = L.msco_paged_attention_split_tokens(n + 1, dt)
    assert (n + 1 + t1 - 1) // t1 >= (n + t - 1) // t


def test_algorithmic_bytes_formulas_match_the_stated_per_unit_figures():
    # the roofline numerators: 512 B (16-bit) / 256 B (int8) per context token per kv head at head_dim 128,
    # plus Q in / O out; 8196 B per valid token for the bf16 copy scatter of 8 x 128 rows
    from ms_custom_ops_b200 import workloads
    lens = [1000, 24, 4096]
    kv = workloads.algorithmic_bytes_attention(lens, 32, 8, 128, 2)
    assert kv == sum(lens) * 8 * 512 + 3 * 32 * 128 * 4
    kv8 = workloads.algorithmic_bytes_attention(lens, 64, 8, 128, 1, quant=True)
    assert kv8 == sum(lens) * 8 * 256 + 3 * 64 * 128 * 4 + 2 * 8 * 128 * 4
    slots = np.array([5, -1, 9, 2, -1], np.int32)
    assert workloads.algorithmic_bytes_scatter(slots, 1024, 2, 2) == 3 * 8192 + 5 * 4
    assert workloads.algorithmic_bytes_scatter(slots, 1024, 2, 1, quant=True) == 3 * 6144 + 5 * 4 + 2 * 1024 * 4
    # benchmark configuration 2 as published: 64 sequences, 32 q / 8 kv heads, bf16
    spec = workloads.config_spec(2)
    assert (spec.batch, spec.num_heads, spec.kv_heads, spec.head_size, spec.block_size) == (64, 32, 8, 128, 128)
