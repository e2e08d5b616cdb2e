"""KV-head sharding of the decode path across the GPUs of one node.

Softmax is per q head and every q head reads exactly one kv head, so the path
partitions by kv head with no exchange inside attention: rank r owns kv heads
[r * H/N, (r+1) * H/N) of every cache block, the matching q heads, and full
copies of block_tables / context_lens / slot_mapping.  The only collective is
an all-gather of the per-rank outputs.  The reference has no multi-device
code on this path; this module is the host-side bookkeeping of that scheme.
"""
from __future__ import annotations

import numpy as np


def kv_head_range(rank: int, world: int, kv_heads: int):
    """Half-open range of kv heads owned by `rank`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if kv_heads % world != 0:
        raise ValueError(f"{kv_heads} kv heads cannot be split evenly over {world} ranks")
    per = kv_heads // world
    return rank * per, (rank + 1) * per


def q_head_range(rank: int, world: int, q_heads: int, kv_heads: int):
    """Half-open range of q heads that read the kv heads of `rank`."""
    h0, h1 = kv_head_range(rank, world, kv_heads)
    g = q_heads // kv_heads
    return h0 * g, h1 * g


def shard_arrays(case: dict, rank: int, world: int) -> dict:
    """Slice a host-side decode case (numpy arrays in operator layouts) down to one rank's shard."""
    kc = case["key_cache"]
    kv_heads, d = kc.shape[2], kc.shape[3]
    q_heads = case["query"].shape[1]
    h0, h1 = kv_head_range(rank, world, kv_heads)
    q0, q1 = q_head_range(rank, world, q_heads, kv_heads)
    out = dict(case)
    out["query"] = np.ascontiguousarray(case["query"][:, q0:q1])
    out["key_cache"] = np.ascontiguousarray(kc[:, :, h0:h1])
    out["value_cache"] = np.ascontiguousarray(case["value_cache"][:, :, h0:h1])
    for name in ("key", "value"):
        if case.get(name) is not None:
            t = case[name].shape[0]
            out[name] = np.ascontiguousarray(case[name].reshape(t, kv_heads, d)[:, h0:h1].reshape(t, -1))
    for name in ("k_descale", "v_descale", "k_offset", "v_offset"):
        if case.get(name) is not None:
            out[name] = np.ascontiguousarray(np.asarray(case[name]).reshape(kv_heads, d)[h0:h1].reshape(-1))
    return out


def assemble_gathered(gathered):
    """[world, batch, q_heads / world, head_dim] (all-gather order) -> [batch, q_heads, head_dim].

    Works on numpy arrays and torch tensors: q head h of sequence b is
    gathered[h // per_rank, b, h % per_rank].
    """
    world, batch, per, d = gathered.shape
    if hasattr(gathered, "permute"):
        return gathered.permute(1, 0, 2, 3).reshape(batch, world * per, d)
    return np.transpose(gathered, (1, 0, 2, 3)).reshape(batch, world * per, d)


def all_gather_outputs(out_local, gathered=None, group=None):
    """All-gather the per-rank outputs ([batch, q_heads / world, head_dim]) into
    [world, batch, q_heads / world, head_dim] on every rank (NCCL on GPU tensors, gloo on CPU)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = torch.empty((world,) + tuple(out_local.shape), dtype=out_local.dtype, device=out_local.device)
    # rank-major concatenation along dim 0 is the same memory as [world, batch, heads, head_dim]
    flat = gathered.view((world * out_local.shape[0],) + tuple(out_local.shape[1:]))
    dist.all_gather_into_tensor(flat, out_local.contiguous(), group=group)
    return gathered
