"""Seeded synthetic workloads for the paged-KV decode path.

No dataset is involved anywhere on this path: every input is drawn from a
seeded generator with the shapes, sizes and value distributions of the
benchmark configurations (C1..C5 below) or of the reference's system tests.

``decode_case`` / ``config_spec`` -- the benchmark configurations: N(0, 1)
query / cache / new rows, block tables that are a shuffled assignment of a
block pool, one new token per sequence written by reshape_and_cache at the
last position, per-channel int8 scales uniform in [0.01, 0.05].
(The generator that reproduces the inputs of the reference's own system tests
is test infrastructure and lives beside the golden fixtures, tests/golden/st_inputs.py.)

Host arrays are numpy (bf16 as ``ml_dtypes.bfloat16``).  ``decode_case_device``
builds the same kind of case directly in GPU memory for the full-size
benchmark configurations, where host generation would take minutes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import ml_dtypes
import numpy as np

bfloat16 = ml_dtypes.bfloat16

NP_DTYPES = {"float16": np.float16, "bfloat16": bfloat16, "int8": np.int8}


def _round_to(a32: np.ndarray, dtype: str) -> np.ndarray:
    return a32.astype(NP_DTYPES[dtype])


# --------------------------------------------------------------------------
# benchmark configurations
# --------------------------------------------------------------------------
@dataclass
class DecodeSpec:
    """Shape of one decode step (reshape_and_cache of one token per sequence, then attention)."""
    name: str
    batch: int
    num_heads: int
    kv_heads: int = 8
    head_size: int = 128
    block_size: int = 128
    dtype: str = "bfloat16"
    kv_int8: bool = False
    len_dist: str = "uniform"        # "uniform" | "loguniform"
    len_lo: int = 1
    len_hi: int = 1024
    num_blocks: Optional[int] = None  # None: ceil(1.1 * blocks needed)
    seed: int = 0
    extra: dict = field(default_factory=dict)

    @property
    def qk_scale(self):
        return 1.0 / math.sqrt(self.head_size)


def config_spec(n: int, scale: float = 1.0) -> DecodeSpec:
    """Benchmark configuration n (1..5); scale < 1 shrinks batch and lengths for tests."""
    def s(v, lo=1):
        return max(lo, int(round(v * scale)))
    if n == 1:
        return DecodeSpec("C1-st-style-fp16", 4, 32, dtype="float16", len_lo=1, len_hi=1024, num_blocks=64, seed=0)
    if n == 2:
        return DecodeSpec("C2-8B-bf16", s(64), 32, len_lo=s(2048, 2), len_hi=s(8192, 4), seed=2)
    if n == 3:
        return DecodeSpec("C3-int8kv", s(128), 64, kv_int8=True, len_lo=s(1024, 2), len_hi=s(4096, 4), seed=3)
    if n == 4:
        return DecodeSpec("C4-long-skewed-bf16", s(32), 64, len_dist="loguniform", len_lo=s(512, 2),
                          len_hi=s(131072, 8), seed=4)
    if n == 5:
        return DecodeSpec("C5-mixed-decode-bf16", s(256), 32, len_lo=s(128, 2), len_hi=s(2048, 4), seed=5,
                          extra={"rac_tokens": s(16384, 8), "rac_blocks": s(4096, 4), "pad_frac": 0.05})
    raise ValueError(n)


def draw_lens(spec: DecodeSpec, rng) -> np.ndarray:
    if spec.len_dist == "loguniform":
        u = rng.uniform(math.log(spec.len_lo), math.log(spec.len_hi), spec.batch)
        return np.minimum(np.floor(np.exp(u)).astype(np.int64), spec.len_hi).astype(np.int32)
    return rng.integers(spec.len_lo, spec.len_hi + 1, spec.batch).astype(np.int32)


def layout(spec: DecodeSpec, lens: np.ndarray, rng):
    """Block tables (shuffled assignment of a pool) and the slot of each sequence's last token."""
    bs = spec.block_size
    need = (lens.astype(np.int64) + bs - 1) // bs
    total = int(need.sum())
    nb = spec.num_blocks if spec.num_blocks is not None else int(math.ceil(total * 1.1)) + 1
    if total > nb:
        raise ValueError("block pool too small")
    pool = rng.permutation(nb)[:total].astype(np.int32)
    width = max(1, int(need.max()))
    tables = np.zeros((spec.batch, width), dtype=np.int32)
    off = 0
    for b in range(spec.batch):
        tables[b, :need[b]] = pool[off:off + need[b]]
        off += int(need[b])
    last = lens.astype(np.int64) - 1
    slots = np.where(lens > 0, tables[np.arange(spec.batch), np.maximum(last, 0) // bs].astype(np.int64) * bs
                     + np.maximum(last, 0) % bs, -1).astype(np.int32)
    return nb, tables, slots


def slots_of_last_token(tables, lens, block_size):
    """slot_mapping of a decode step: the cache slot of every sequence's newest token (position
    len - 1), -1 for an empty sequence."""
    tables = np.asarray(tables)
    lens = np.asarray(lens).astype(np.int64)
    last = np.maximum(lens - 1, 0)
    rows = np.arange(len(lens))
    return np.where(lens > 0, tables[rows, last // block_size].astype(np.int64) * block_size + last % block_size,
                    -1).astype(np.int32)


def grow_tables(tables, lens, num_blocks, block_size, steps):
    """Room for `steps` more tokens per sequence: a decode loop appends one token to every sequence
    per step and needs a fresh cache block whenever a sequence crosses a block boundary.  The blocks
    the sequences will need are taken from new ids appended to the pool ([num_blocks, num_blocks +
    extra)) and entered into wider block tables up front -- a block allocator that reserves ahead; an
    attention launch only ever reads the first ceil(len / block_size) columns of a row.
    Returns (tables, num_blocks) after growth."""
    tables = np.asarray(tables)
    lens = np.asarray(lens).astype(np.int64)
    now = (lens + block_size - 1) // block_size
    later = (lens + steps + block_size - 1) // block_size
    width = max(int(later.max()) if len(lens) else 1, tables.shape[1])
    out = np.zeros((tables.shape[0], width), dtype=np.int32)
    out[:, :tables.shape[1]] = tables
    nxt = int(num_blocks)
    for b in range(len(lens)):
        n = int(later[b] - now[b])
        out[b, now[b]:now[b] + n] = np.arange(nxt, nxt + n, dtype=np.int32)
        nxt += n
    return out, nxt


def quantize_per_channel(x32: np.ndarray, descale: np.ndarray) -> np.ndarray:
    """int8 = clip(rint(x / descale)) in float32 (offset 0)."""
    return np.clip(np.rint(x32.astype(np.float32) / descale.astype(np.float32)), -128, 127).astype(np.int8)


def decode_case(spec: DecodeSpec):
    """One decode step on the host: caches, new K/V rows, slots, query, tables, lengths.

    The cache holds N(0, 1) values everywhere (for int8 KV: N(0, 1) quantised
    per channel); the rows of the newest token are *not* in the cache yet --
    reshape_and_cache writes them at `slot_mapping` before attention runs.
    """
    rng = np.random.default_rng(spec.seed)
    lens = draw_lens(spec, rng)
    nb, tables, slots = layout(spec, lens, rng)
    c = spec.kv_heads * spec.head_size
    shape = (nb, spec.block_size, spec.kv_heads, spec.head_size)
    out = {"spec": spec, "context_lens": lens, "block_tables": tables, "slot_mapping": slots,
           "num_blocks": nb, "qk_scale": spec.qk_scale, "q_dtype": spec.dtype,
           "k_descale": None, "v_descale": None, "k_offset": None, "v_offset": None}
    out["query"] = _round_to(rng.standard_normal((spec.batch, spec.num_heads, spec.head_size), dtype=np.float32), spec.dtype)
    out["key"] = _round_to(rng.standard_normal((spec.batch, c), dtype=np.float32), spec.dtype)
    out["value"] = _round_to(rng.standard_normal((spec.batch, c), dtype=np.float32), spec.dtype)
    if spec.kv_int8:
        kd = rng.uniform(0.01, 0.05, c).astype(np.float32)
        vd = rng.uniform(0.01, 0.05, c).astype(np.float32)
        out["k_descale"], out["v_descale"] = kd, vd
        out["key_cache"] = quantize_per_channel(rng.standard_normal(shape, dtype=np.float32), kd.reshape(spec.kv_heads, -1))
        out["value_cache"] = quantize_per_channel(rng.standard_normal(shape, dtype=np.float32), vd.reshape(spec.kv_heads, -1))
        out["kv_dtype"] = "int8"
    else:
        out["key_cache"] = _round_to(rng.standard_normal(shape, dtype=np.float32), spec.dtype)
        out["value_cache"] = _round_to(rng.standard_normal(shape, dtype=np.float32), spec.dtype)
        out["kv_dtype"] = spec.dtype
    return out


def scatter_case(tokens, num_blocks, block_size=128, kv_heads=8, head_size=128, dtype="bfloat16",
                 pad_frac=0.05, seed=5, quant=False):
    """Prefill-heavy reshape_and_cache: `tokens` rows through an injective random slot map
    with a fraction of the slots set to -1 (padding)."""
    rng = np.random.default_rng(seed)
    c = kv_heads * head_size
    nslots = num_blocks * block_size
    slots = rng.permutation(nslots)[:tokens].astype(np.int32)
    pad = rng.random(tokens) < pad_frac
    slots[pad] = -1
    key = _round_to(rng.standard_normal((tokens, c), dtype=np.float32), dtype)
    value = _round_to(rng.standard_normal((tokens, c), dtype=np.float32), dtype)
    cdt = np.int8 if quant else NP_DTYPES[dtype]
    shape = (num_blocks, block_size, kv_heads, head_size)
    if quant:
        kcache = rng.integers(-128, 128, shape, dtype=np.int8)
        vcache = rng.integers(-128, 128, shape, dtype=np.int8)
    else:
        kcache = _round_to(rng.standard_normal(shape, dtype=np.float32), dtype)
        vcache = _round_to(rng.standard_normal(shape, dtype=np.float32), dtype)
    out = {"key": key, "value": value, "key_cache": kcache.astype(cdt), "value_cache": vcache.astype(cdt),
           "slot_mapping": slots, "k_descale": None, "v_descale": None}
    if quant:
        out["k_descale"] = rng.uniform(0.01, 0.05, c).astype(np.float32)
        out["v_descale"] = rng.uniform(0.01, 0.05, c).astype(np.float32)
    return out


def algorithmic_bytes_attention(lens, q_heads, kv_heads, head_size, kv_bytes, q_bytes=2, out_bytes=2,
                                quant=False, offsets=False):
    """Bytes paged attention must move: K and V of every context token once, Q in, O out
    (+ the per-channel scale vectors once for int8 KV).  Tables, lengths and split
    partials are not counted."""
    total = int(np.asarray(lens, dtype=np.int64).sum()) * 2 * kv_heads * head_size * kv_bytes
    total += len(lens) * q_heads * head_size * (q_bytes + out_bytes)
    if quant:
        total += 2 * kv_heads * head_size * 4 * (2 if offsets else 1)
    return total


def algorithmic_bytes_scatter(slots, row_elems, in_bytes, cache_bytes, quant=False):
    """Bytes reshape_and_cache must move: each valid K and V row read once and written
    once, plus the slot map (+ the scale vectors once for the quantising variant)."""
    slots = np.asarray(slots)
    valid = int((slots >= 0).sum())
    total = valid * row_elems * (in_bytes + cache_bytes) * 2 + slots.size * 4
    if quant:
        total += 2 * row_elems * 4
    return total


# --------------------------------------------------------------------------
# full-size cases generated directly in GPU memory
# --------------------------------------------------------------------------
def decode_case_device(spec: DecodeSpec, device="cuda", kv_head_range=None, growth_steps=0):
    """Same kind of case as `decode_case`, built on the GPU with torch's seeded generator.

    Lengths, block tables and slots come from the same numpy draws as the host
    version (they are small); the large tensors (caches, query, new rows) are
    N(0, 1) draws of a `torch.Generator` seeded with `spec.seed`.  The caches
    are filled in pieces so that no float32 temporary larger than 256 MB exists.
    `kv_head_range = (h0, h1)` builds only that slice of kv heads (and the
    matching q heads): the shard one GPU owns when the cache is partitioned by
    kv head.  Each head's values depend on (seed, head) only, so a shard holds
    exactly the values the same heads have in the unsharded case.
    `growth_steps` > 0 reserves cache blocks and block-table columns for that many further decode
    steps (see grow_tables); "block_tables_host" is the host copy of the tables.
    """
    import torch

    rng = np.random.default_rng(spec.seed)
    lens = draw_lens(spec, rng)
    nb, tables, slots = layout(spec, lens, rng)
    if growth_steps > 0:
        tables, nb = grow_tables(tables, lens, nb, spec.block_size, growth_steps)
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[spec.dtype]
    h0, h1 = kv_head_range if kv_head_range is not None else (0, spec.kv_heads)
    nh = h1 - h0
    g = spec.num_heads // spec.kv_heads
    d = spec.head_size
    out = {"spec": spec, "context_lens": lens, "num_blocks": nb, "qk_scale": spec.qk_scale,
           "kv_head_range": (h0, h1), "block_tables_host": tables,
           "block_tables": torch.from_numpy(tables).to(device),
           "slot_mapping": torch.from_numpy(slots).to(device),
           "k_descale": None, "v_descale": None}

    def gen_for(head, tag):
        gtor = torch.Generator(device=device)
        gtor.manual_seed((spec.seed * 1000003 + head * 101 + tag) & 0x7FFFFFFF)
        return gtor

    cdt = torch.int8 if spec.kv_int8 else tdt
    kc = torch.empty((nb, spec.block_size, nh, d), dtype=cdt, device=device)
    vc = torch.empty_like(kc)
    q = torch.empty((spec.batch, nh * g, d), dtype=tdt, device=device)
    key = torch.empty((spec.batch, nh * d), dtype=tdt, device=device)
    val = torch.empty_like(key)
    kd = vd = None
    if spec.kv_int8:
        kd = torch.empty(nh * d, dtype=torch.float32, device=device)
        vd = torch.empty_like(kd)
    step = max(1, (64 << 20) // (spec.block_size * d))  # blocks per piece: 256 MB of float32
    for i, h in enumerate(range(h0, h1)):
        gq = gen_for(h, 0)
        q[:, i * g:(i + 1) * g] = torch.randn((spec.batch, g, d), generator=gq, device=device).to(tdt)
        key[:, i * d:(i + 1) * d] = torch.randn((spec.batch, d), generator=gq, device=device).to(tdt)
        val[:, i * d:(i + 1) * d] = torch.randn((spec.batch, d), generator=gq, device=device).to(tdt)
        if spec.kv_int8:
            kd[i * d:(i + 1) * d] = torch.rand(d, generator=gq, device=device) * 0.04 + 0.01
            vd[i * d:(i + 1) * d] = torch.rand(d, generator=gq, device=device) * 0.04 + 0.01
        for cache, scale, tag in ((kc, kd, 1), (vc, vd, 2)):
            gc = gen_for(h, tag)
            for b0 in range(0, nb, step):
                b1 = min(nb, b0 + step)
                x = torch.randn((b1 - b0, spec.block_size, d), generator=gc, device=device)
                if spec.kv_int8:
                    x = torch.clamp(torch.round(x / scale[i * d:(i + 1) * d]), -128, 127)
                cache[b0:b1, :, i] = x.to(cdt)
    out.update(query=q, key=key, value=val, key_cache=kc, value_cache=vc, k_descale=kd, v_descale=vd)
    return out
