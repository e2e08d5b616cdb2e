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


# --------------------------------------------------------------------------
# Sequence sharding: the second axis, for contexts so long (or kv heads so few) that kv-head
# sharding runs out.  Rank r holds a contiguous range of whole cache blocks of EVERY sequence,
# computes attention over its part with the log-sum-exp as a second output, the ranks all-gather
# (lse, output) and every rank merges them with fa_update -- exact, because
# softmax over the whole context = sum_r exp(lse_r - lse) * softmax over part r.
# --------------------------------------------------------------------------
def seq_block_range(num_blocks_of_seq: int, rank: int, world: int):
    """Half-open range of a sequence's block-table columns owned by `rank` (balanced, contiguous)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    return rank * num_blocks_of_seq // world, (rank + 1) * num_blocks_of_seq // world


def seq_shard_tables(block_tables, context_lens, block_size: int, rank: int, world: int):
    """One rank's view of the block tables and lengths under sequence sharding.

    Returns (local_tables int32 [batch, cols], local_lens int32 [batch]): row b holds the columns
    seq_block_range(ceil(len_b / block_size), rank, world) of block_tables[b], left-aligned and padded
    with 0; local_lens[b] is the number of context tokens in them (0 when the rank holds nothing of
    a short sequence).  The newest token of a sequence lives on the rank that owns its last block.
    Additive masks index absolute context positions, so a masked launch over a part needs the mask
    columns of that part (column offset lo * block_size); the helpers here cover the mask-free case.
    """
    tables = np.asarray(block_tables)
    lens = np.asarray(context_lens).astype(np.int64).reshape(-1)
    nblk = (lens + block_size - 1) // block_size
    lo = rank * nblk // world
    hi = (rank + 1) * nblk // world
    cols = max(int((hi - lo).max()) if len(lens) else 0, 1)
    local = np.zeros((len(lens), cols), dtype=np.int32)
    for b in range(len(lens)):
        local[b, :hi[b] - lo[b]] = tables[b, lo[b]:hi[b]]
    local_lens = np.clip(np.minimum(lens, hi * block_size) - lo * block_size, 0, None).astype(np.int32)
    return local, local_lens


def seq_parallel_merge(out_local, lse_local, merge, group=None):
    """All-gather the per-rank (output, lse) of a sequence-sharded decode step and merge them.

    out_local [batch, q_heads, head_dim] (any float dtype), lse_local float32 [batch, q_heads];
    `merge(lse [world, rows], partial [world, rows, head_dim]) -> [rows, head_dim]` is
    ms_custom_ops_b200.fa_update on GPUs.  Returns float32 [batch, q_heads, head_dim] on every rank.
    One collective: lse rides as an extra column of the float32 rows.
    """
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    b, h, d = out_local.shape
    packed = torch.empty((b * h, d + 1), dtype=torch.float32, device=out_local.device)
    packed[:, :d] = out_local.reshape(b * h, d)
    packed[:, d] = lse_local.reshape(b * h)
    gathered = torch.empty((world * b * h, d + 1), dtype=torch.float32, device=out_local.device)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    gathered = gathered.view(world, b * h, d + 1)
    merged = merge(gathered[:, :, d].contiguous(), gathered[:, :, :d].contiguous())
    return merged.view(b, h, d)


class SeqParallelExchange:
    """Device side of a sequence-sharded decode step: the all-gather of the per-rank (output, lse)
    records and their merge.

    Every rank's attention launch writes its output (query dtype) and its log-sum-exps (float32) into
    ONE record buffer, `out_local` and `lse_local` being views of it; `exchange_and_merge()` all-gathers
    the raw records (this library's peer-store kernel over NVLink, or NCCL) and merges them where they
    lie with msco_fa_update_strided.  No packing or conversion kernel in between.
    """

    def __init__(self, batch, q_heads, head_dim, dtype, device, use_peer_stores=True, group=None):
        import torch
        import torch.distributed as dist
        from . import kernels
        self._torch, self._dist, self._kernels, self.group = torch, dist, kernels, group
        self.world = dist.get_world_size(group)
        es = torch.empty((), dtype=dtype).element_size()
        rows = batch * q_heads
        n_out = rows * head_dim * es
        self.off_lse = (n_out + 255) // 256 * 256
        self.rec_bytes = (self.off_lse + rows * 4 + 255) // 256 * 256
        self.es, self.rows = es, rows
        self.record = torch.zeros(self.rec_bytes, dtype=torch.uint8, device=device)
        self.out_local = self.record[:n_out].view(dtype).view(batch, q_heads, head_dim)
        self.lse_local = self.record[self.off_lse:self.off_lse + rows * 4].view(torch.float32).view(batch, q_heads)
        self.merged = torch.empty((batch, q_heads, head_dim), dtype=dtype, device=device)
        self.peer = PeerGather((self.rec_bytes,), torch.uint8, device, group) if use_peer_stores else None
        self.gathered = None if use_peer_stores else torch.empty((self.world, self.rec_bytes), dtype=torch.uint8,
                                                                 device=device)

    def exchange_and_merge(self):
        """All-gather the records, merge; returns the merged output [batch, q_heads, head_dim]."""
        torch = self._torch
        if self.peer is not None:
            g = self.peer.gather(self.record)
        else:
            g = self.gathered
            self._dist.all_gather_into_tensor(g.view(-1), self.record, group=self.group)
        lse0 = g[0, self.off_lse:self.off_lse + self.rows * 4].view(torch.float32)
        out0 = g[0, :self.rows * self.merged.shape[-1] * self.es].view(self.merged.dtype)
        self._kernels.merge_partials_strided(lse0, self.rec_bytes // 4, out0, self.rec_bytes // self.es,
                                             self.merged.view(self.rows, -1), self.world)
        return self.merged

    def check(self):
        if self.peer is not None:
            self.peer.check()

    def release(self):
        if self.peer is not None:
            self.peer.release()


class PeerGather:
    """All-gather of per-rank outputs by peer stores over NVLink (msco_peer_allgather).

    Set-up exchanges CUDA IPC handles of each rank's gathered buffers and flag arrays through the
    process group (host side); after that a gather is one small kernel per rank on the caller's
    stream -- no library collective.  Two gathered buffers alternate from step to step, so a
    consumer of step k may still be reading while step k+1 is pushed.

        pg = PeerGather(out_local.shape, out_local.dtype, device)      # collective: call on all ranks
        gathered = pg.gather(out_local)                                # [world, *out_local.shape]
    """

    def __init__(self, slice_shape, dtype, device, group=None, packets=True):
        """`packets=False`: msco_decode_step_gather then uses the flag protocol of msco_peer_allgather
        (fences and a flag per rank) instead of the packet form."""
        import ctypes as C

        import torch
        import torch.distributed as dist

        from . import _abi
        self._abi, self._C, self._torch = _abi, C, torch
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _abi.MAX_PEERS:
            raise ValueError(f"at most {_abi.MAX_PEERS} ranks")
        self.slice_shape = tuple(slice_shape)
        self.slice_bytes = int(torch.empty(self.slice_shape, dtype=dtype, device="meta").numel()) * \
            torch.empty((), dtype=dtype).element_size()
        if self.slice_bytes % 16:
            raise ValueError("slice size must be a multiple of 16 bytes")
        L = _abi.lib()
        # one arena per rank, exported once: [gathered 0 | gathered 1 | flags 0 | flags 1 | packets 0 | packets 1],
        # 256-byte aligned parts; the packet buffers (twice the gathered size: every 4 data bytes travel with
        # their step number) serve the decode step that does the exchange itself (msco_decode_step_gather)
        gbytes = self.world * self.slice_bytes
        goff = [0, (gbytes + 255) // 256 * 256]
        foff = [goff[1] * 2, goff[1] * 2 + 256]
        poff = [foff[1] + 256, foff[1] + 256 + 2 * goff[1]]
        self.arena = torch.zeros(poff[1] + 2 * goff[1], dtype=torch.uint8, device=device)
        self.buffers = [self.arena[o:o + gbytes].view(dtype).view((self.world,) + self.slice_shape) for o in goff]
        self.words = torch.zeros(4, dtype=torch.int32, device=device)  # [ticket, status, -, -]
        torch.cuda.synchronize(device)
        h = C.create_string_buffer(_abi.IPC_HANDLE_BYTES)
        off = C.c_int64()
        _abi.check(L.msco_ipc_export(C.c_void_p(self.arena.data_ptr()), h, C.byref(off)))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (bytes(h.raw), int(off.value)), group=group)
        self._mapped = []  # (ptr, offset) of imported peer arenas, for release()
        bases = []
        for r in range(self.world):
            if r == self.rank:
                bases.append(self.arena.data_ptr())
            else:
                handle, roff = everyone[r]
                p = C.c_void_p()
                _abi.check(L.msco_ipc_import(handle, roff, C.byref(p)))
                self._mapped.append((p.value, roff))
                bases.append(p.value)
        self.descs = []
        for parity in range(2):
            d = _abi.MscoGatherDesc()
            d.world, d.rank, d.slice_bytes = self.world, self.rank, self.slice_bytes
            d.ticket = self.words.data_ptr()
            d.status = self.words.data_ptr() + 4
            for r in range(self.world):
                d.gathered[r] = bases[r] + goff[parity]
                d.flags[r] = bases[r] + foff[parity]
                if packets:
                    d.packets[r] = bases[r] + poff[parity]
            self.descs.append(d)
        self.step = 0
        dist.barrier(group=group)  # every rank has mapped every buffer before the first push

    def gather(self, out_local):
        """Push `out_local` to every rank and wait for every rank's push; returns this rank's
        gathered buffer [world, *slice_shape] (valid until the gather after next)."""
        C, torch = self._C, self._torch
        self.step += 1
        parity = self.step & 1
        # each parity has its own flag array, so its step counter advances by one per use
        self._abi.check(self._abi.lib().msco_peer_allgather(
            C.byref(self.descs[parity]), C.c_void_p(out_local.data_ptr()), C.c_uint32((self.step + 1) // 2),
            C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.buffers[parity]

    def next_step(self):
        """(descriptor by reference, step counter, gathered buffer) of the next exchange, for
        msco_decode_step_gather: the decode step's own finishing kernel does the push and the wait."""
        self.step += 1
        parity = self.step & 1
        return self._C.byref(self.descs[parity]), self._C.c_uint32((self.step + 1) // 2), self.buffers[parity]

    def check(self):
        """After a synchronise: raises if a bounded wait for a peer expired."""
        if int(self.words[1].item()) != 0:
            raise self._abi.MscoError(self._abi.ERR_TIMEOUT, "peer all-gather: a peer's flag never arrived")

    def release(self):
        L = self._abi.lib()
        for p, off in self._mapped:
            L.msco_ipc_release(self._C.c_void_p(p), off)
        self._mapped = []
