"""CPU: kv-head sharding bookkeeping, exercised over a real 2-rank gloo process group.

The device kernels are not involved here: each rank computes its shard with the CPU oracle (test
stand-in), the outputs are all-gathered exactly as bench.py does on GPUs, reassembled, and compared
with the unsharded result.  This pins the slice / gather / reassembly layout and that per-head
results do not depend on the shard count.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ms_custom_ops_b200 import _abi, sharding, workloads  # noqa: E402
from oracle import paged_kv_numpy as oracle  # noqa: E402


def test_head_ranges():
    assert sharding.kv_head_range(0, 1, 8) == (0, 8)
    assert [sharding.kv_head_range(r, 4, 8) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert sharding.q_head_range(3, 8, 64, 8) == (24, 32)
    with pytest.raises(ValueError):
        sharding.kv_head_range(0, 3, 8)
    with pytest.raises(ValueError):
        sharding.kv_head_range(2, 2, 8)


def test_assemble_gathered_layout():
    world, batch, per, d = 4, 3, 2, 5
    full = np.arange(batch * world * per * d, dtype=np.float32).reshape(batch, world * per, d)
    gathered = np.stack([full[:, r * per:(r + 1) * per] for r in range(world)])
    assert np.array_equal(sharding.assemble_gathered(gathered), full)
    assert torch.equal(sharding.assemble_gathered(torch.from_numpy(gathered)), torch.from_numpy(full))


def test_split_plan_is_the_same_for_every_shard():
    # the split rule sees lengths only, so a shard plans exactly 1/N of the unsharded work items
    lens = [5000, 300, 70000, 513]
    def info(hq, hkv):
        d = _abi.MscoPaDesc()
        d.q_dtype = d.kv_dtype = _abi.DTYPE_BF16
        d.num_q_heads, d.num_kv_heads, d.head_dim, d.block_size = hq, hkv, 128, 128
        d.num_blocks, d.max_blocks_per_seq, d.qk_scale = 1 << 20, 1024, 0.1
        return _abi.PaPlan(d, lens).info()
    full, shard = info(64, 8), info(16, 2)
    assert shard.max_splits == full.max_splits and shard.partials == full.partials
    assert shard.work_items * 4 == full.work_items


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = workloads.config_spec(3, 0.03)   # int8 KV: scales are sharded too
        case = workloads.decode_case(spec)
        mine = sharding.shard_arrays(case, rank, world)
        gk, gv = oracle.reshape_and_cache_quant_golden(mine["key"], mine["value"], mine["key_cache"],
                                                       mine["value_cache"], mine["slot_mapping"],
                                                       mine["k_descale"], mine["v_descale"])
        out_local = oracle.paged_attention_golden(mine["query"], gk, gv, mine["block_tables"], mine["context_lens"],
                                                  mine["qk_scale"], mine["k_descale"], mine["v_descale"])
        gathered = sharding.all_gather_outputs(torch.from_numpy(out_local))
        full = sharding.assemble_gathered(gathered).numpy()
        fk, fv = oracle.reshape_and_cache_quant_golden(case["key"], case["value"], case["key_cache"],
                                                       case["value_cache"], case["slot_mapping"],
                                                       case["k_descale"], case["v_descale"])
        want = oracle.paged_attention_golden(case["query"], fk, fv, case["block_tables"], case["context_lens"],
                                             case["qk_scale"], case["k_descale"], case["v_descale"])
        h0, h1 = sharding.kv_head_range(rank, world, spec.kv_heads)
        ok_cache = np.array_equal(gk, fk[:, :, h0:h1]) and np.array_equal(gv, fv[:, :, h0:h1])
        ret[rank] = (bool(np.allclose(full, want, rtol=1e-5, atol=1e-6)), ok_cache, full.shape == want.shape)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharded_decode_matches_unsharded():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        assert p.exitcode == 0, "a rank failed or timed out"
    assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}


# ----------------------------------------------------------------------------- sequence sharding
def test_seq_block_ranges_cover_every_block_once():
    for nblk in (0, 1, 2, 5, 8, 64, 513):
        for world in (1, 2, 3, 8):
            ranges = [sharding.seq_block_range(nblk, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == nblk
            assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1


def test_seq_shard_tables_lengths_and_columns():
    tables = np.arange(3 * 6, dtype=np.int32).reshape(3, 6) + 100
    lens = np.array([41, 3, 96], np.int32)  # block 16: 3, 1, 6 blocks
    parts = [sharding.seq_shard_tables(tables, lens, 16, r, 4) for r in range(4)]
    for b in range(3):
        assert sum(int(p[1][b]) for p in parts) == lens[b]
        cols = np.concatenate([p[0][b, :(int(p[1][b]) + 15) // 16] for p in parts])
        assert np.array_equal(cols, tables[b, :(lens[b] + 15) // 16])
    assert int(parts[0][1][1]) == 0 and int(parts[3][1][1]) == 3   # the short sequence lives on the last rank


def _seq_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(11)
        nb, bs, hkv, hq, d, batch = 48, 16, 2, 8, 32, 5
        kc = rng.standard_normal((nb, bs, hkv, d)).astype(np.float32)
        vc = rng.standard_normal((nb, bs, hkv, d)).astype(np.float32)
        q = rng.standard_normal((batch, hq, d)).astype(np.float32)
        lens = np.array([100, 7, 16, 33, 128], np.int32)
        tables = np.stack([rng.permutation(nb)[:8] for _ in range(batch)]).astype(np.int32)
        want = oracle.paged_attention_golden(q, kc, vc, tables, lens, 0.2)
        lt, ll = sharding.seq_shard_tables(tables, lens, bs, rank, world)
        o, lse = oracle.paged_attention_golden(q, kc, vc, lt, ll, 0.2, return_lse=True)

        def merge(lse_all, parts):
            return torch.from_numpy(oracle.fa_update_golden(lse_all.numpy(), parts.numpy()))
        got = sharding.seq_parallel_merge(torch.from_numpy(o), torch.from_numpy(lse), merge).numpy()
        ret[rank] = (bool(np.allclose(got, want, rtol=1e-5, atol=1e-6)), got.shape == want.shape,
                     bool(np.isneginf(lse[ll == 0]).all()))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sequence_sharded_decode_matches_unsharded():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_seq_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        assert p.exitcode == 0, "a rank failed or timed out"
    assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}
