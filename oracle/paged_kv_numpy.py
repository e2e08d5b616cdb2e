"""numpy restatement of the reference goldens for the paged-KV decode path.

TEST INFRASTRUCTURE ONLY -- never imported by the product package.

Every function cites the reference file (path inside the reference project)
whose arithmetic it follows.  The restatement vectorises the reference's
per-token Python loops but keeps the same float32 operations in the same
order where order matters (de-quantise -> gather -> grouped QK^T -> scale ->
(+mask) -> max-subtracted softmax -> grouped PV).

Parity status: `paged_attention_golden` and `reshape_and_cache_golden` are
pinned by tests/golden (outputs of the reference's own golden functions on the
same seeded inputs), and so are `paged_cache_load_golden` and
`fa_update_golden`.  `reshape_and_cache_quant_golden` is "parity unpinned":
the reference's reshape_and_cache has no quantising mode.
"""
from __future__ import annotations

import numpy as np

try:  # bf16 host representation (same package the fixtures were made with)
    import ml_dtypes

    bfloat16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover - ml_dtypes ships with the image
    bfloat16 = None


# --------------------------------------------------------------------------
# reshape_and_cache
# --------------------------------------------------------------------------
def reshape_and_cache_bnsd_golden(key, value, key_cache, value_cache, slot_mapping):
    """The same scatter into head-major cache blocks [num_blocks, heads, block_size, head_dim].

    Follows tests/st/test_custom_reshape_and_cache_npd.py:487-515 (`npd_cache_inference`):
    ``cache[slot // block_size][h][slot % block_size] = row.reshape(heads, head_dim)[h]``; device twin
    ops/ascendc/aclnn_src/reshape_and_cache_npd/op_kernel/reshape_and_cache_npd.cpp:167-173.  Negative slots
    are skipped (:149-150 of the device twin).  Returns new arrays.
    """
    slot = np.asarray(slot_mapping).reshape(-1).astype(np.int64)
    out = []
    for rows, cache in ((key, key_cache), (value, value_cache)):
        if rows is None or cache is None:
            out.append(None)
            continue
        c = np.array(cache, copy=True)
        bs = c.shape[2]
        r = np.asarray(rows).reshape(-1, c.shape[1], c.shape[3])
        for i in np.flatnonzero(slot >= 0):
            c[slot[i] // bs, :, slot[i] % bs] = r[i]
        out.append(c)
    return out[0], out[1]


def bnsd_to_bsnd(cache):
    """[num_blocks, heads, block_size, head_dim] -> [num_blocks, block_size, heads, head_dim] (a copy)."""
    return np.ascontiguousarray(np.transpose(np.asarray(cache), (0, 2, 1, 3)))


def reshape_and_cache_golden(key, value, key_cache, value_cache, slot_mapping):
    """Scatter rows of `key`/`value` into copies of the paged caches.

    Follows tests/st/test_custom_reshape_and_cache.py:282-307 (`nd_inference`):
    ``blk = slot // block_size; off = slot % block_size;
    cache[blk, off] = row.reshape(heads, head_dim)``.
    Negative slots are skipped, as in the in-repo device twin
    ops/ascendc/aclnn_src/reshape_and_cache_npd/op_kernel/reshape_and_cache_npd.cpp:149-150
    and the sibling golden tests/st/test_custom_kv_rmsnorm_rope_cache.py:413-418.

    `value`/`value_cache` may be None (key-only mode,
    tests/st/test_custom_reshape_and_cache.py:379-401).  Returns new arrays.
    """
    slot = np.asarray(slot_mapping).reshape(-1).astype(np.int64)
    kc = np.array(key_cache, copy=True)
    bs = kc.shape[1]
    rows = np.asarray(key).reshape(-1, kc.shape[2], kc.shape[3])
    # later rows win on duplicate slots, exactly like the reference's loop
    for i in np.flatnonzero(slot >= 0):
        kc[slot[i] // bs, slot[i] % bs] = rows[i]
    vc = None
    if value is not None and value_cache is not None:
        vc = np.array(value_cache, copy=True)
        vrows = np.asarray(value).reshape(-1, vc.shape[2], vc.shape[3])
        vbs = vc.shape[1]
        for i in np.flatnonzero(slot >= 0):
            vc[slot[i] // vbs, slot[i] % vbs] = vrows[i]
    return kc, vc


def quantize_rows_golden(x, descale, offset=None, qmin=-128, qmax=127):
    """int8 = saturate(rint(float32(x) / float32(descale)) - offset).

    Exact inverse of the reference's de-quantisation
    ``(int8 + offset) * descale`` (tests/st/test_custom_paged_attention.py:599-614);
    rounding is numpy's round-half-to-even and saturation is to [-128, 127]
    as in tests/st/test_custom_kv_rmsnorm_rope_cache.py:310-314.
    All arithmetic is float32.  "parity unpinned" (no reference counterpart
    for this op).  `x` is [T, C]; `descale` (float32) and `offset` (int32) [C].
    """
    xf = np.asarray(x).astype(np.float32)
    d = np.asarray(descale, dtype=np.float32).reshape(1, -1)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.rint(xf / d)
    if offset is not None:
        q = q - np.asarray(offset).astype(np.float32).reshape(1, -1)
    q = np.nan_to_num(q, nan=0.0, posinf=float(qmax), neginf=float(qmin))
    return np.clip(q, qmin, qmax).astype(np.int8)


def reshape_and_cache_quant_golden(key, value, key_cache, value_cache, slot_mapping,
                                   k_descale, v_descale, k_offset=None, v_offset=None):
    """Quantise rows per channel (kv_head x head_dim) then scatter them.

    Composition of `quantize_rows_golden` and `reshape_and_cache_golden`.
    """
    t = np.asarray(slot_mapping).size
    kq = quantize_rows_golden(np.asarray(key).reshape(t, -1), k_descale, k_offset)
    vq = None
    if value is not None:
        vq = quantize_rows_golden(np.asarray(value).reshape(t, -1), v_descale, v_offset)
    return reshape_and_cache_golden(kq, vq, key_cache, value_cache, slot_mapping)


# --------------------------------------------------------------------------
# paged_attention (decode)
# --------------------------------------------------------------------------
def _gather_seq(cache_f32, table_row, kv_len, block_size):
    """Rows 0..kv_len-1 of one sequence: ``cache[table[j // bs], j % bs]``.

    Follows tests/st/test_custom_paged_attention.py:701-731 (vectorised).
    """
    j = np.arange(kv_len)
    blk = np.asarray(table_row).astype(np.int64)[j // block_size]
    return cache_f32[blk, j % block_size]  # [kv_len, kv_heads, head]


def paged_attention_golden(query, key_cache, value_cache, block_tables, context_lens, scale,
                           k_descale=None, v_descale=None, k_offset=None, v_offset=None,
                           mask=None, mask_type=0, return_lse=False, q_seq_lens=None):
    """float32 decode attention over a paged KV cache, one query token per sequence.

    Follows tests/st/test_custom_paged_attention.py:
      :586-614  inputs to float32; optional ``(int8 + offset) * descale`` per
                (kv_head, head_dim) channel,
      :701-731  paged gather through the block table,
      :937-1003 grouped matmuls (q heads ``h*g .. (h+1)*g-1`` use kv head ``h``),
      :788-822  ``scores * scale`` (+ mask), max-subtracted softmax, ``P @ V``,
      :644-646  sequences of length 0 produce zeros,
      :880-903  additive masks: NORM ``mask[b, 0, :kl]`` (mask_type 1),
                ALIBI ``mask[b, :, 0, :kl]`` (mask_type 2).
      :641-693  with ``q_seq_lens`` (multi-token queries) sequence ``b`` owns
                ``q_seq_lens[b]`` consecutive query rows, each attending the whole
                context of the sequence,
      :877-879  SPEC ``mask[token, :kl]`` per query row (mask_type 3).
    Returns float32 ``[tokens, q_heads, head_dim]``; the caller casts to the
    query dtype as the reference does (:693-699).  With ``return_lse`` also
    ``log(sum(exp(scores)))`` per (sequence, q head), -inf for an empty context
    (the quantity tests/st/test_asd_faupdate.py:34-59 merges partial outputs by).
    """
    q = np.asarray(query).astype(np.float32)
    kc = np.asarray(key_cache).astype(np.float32)
    vc = np.asarray(value_cache).astype(np.float32)
    nt, hq, d = q.shape
    hkv = kc.shape[2]
    bs = kc.shape[1]
    g = hq // hkv
    if k_descale is not None and v_descale is not None:
        if k_offset is not None:
            kc += np.asarray(k_offset).astype(np.float32).reshape(1, 1, hkv, -1)
        if v_offset is not None:
            vc += np.asarray(v_offset).astype(np.float32).reshape(1, 1, hkv, -1)
        kc *= np.asarray(k_descale, dtype=np.float32).reshape(1, 1, hkv, -1)
        vc *= np.asarray(v_descale, dtype=np.float32).reshape(1, 1, hkv, -1)
    tables = np.asarray(block_tables)
    lens = np.asarray(context_lens).reshape(-1)
    out = np.zeros((nt, hq, vc.shape[3]), dtype=np.float32)
    lse = np.full((nt, hq), -np.inf, dtype=np.float32)
    m = None if mask is None else np.asarray(mask).astype(np.float32)
    # one entry per query row: (row, sequence it belongs to)
    if q_seq_lens is None:
        rows = [(b, b) for b in range(nt)]
    else:
        rows = [(t, b) for b, (t0, n) in enumerate(zip(np.concatenate([[0], np.cumsum(q_seq_lens)[:-1]]),
                                                       q_seq_lens)) for t in range(int(t0), int(t0) + int(n))]
    for b, seq in rows:
        kl = int(lens[seq])
        if kl == 0:
            continue
        ks = _gather_seq(kc, tables[seq], kl, bs)  # [kl, hkv, d]
        vs = _gather_seq(vc, tables[seq], kl, bs)
        qg = q[b].reshape(hkv, g, d)
        scores = np.matmul(qg, np.transpose(ks, (1, 2, 0))) * np.float32(scale)  # [hkv, g, kl]
        if m is not None:
            if mask_type == 2:  # ALIBI [batch, heads, 1, max_ctx]
                scores = scores + m[b, :, 0, :kl].reshape(hkv, g, kl)
            elif mask_type == 1:  # NORM decode [tokens, 1, max_ctx]
                scores = scores + m[b, 0, :kl][None, None, :]
            elif mask_type == 3:  # SPEC [tokens, max_ctx]
                scores = scores + m[b, :kl][None, None, :]
            else:
                raise ValueError("oracle supports the masks NORM(1) / ALIBI(2) of decode and SPEC(3)")
        smax = np.max(scores, axis=-1, keepdims=True)
        e = np.exp(scores - smax)
        p = e / np.sum(e, axis=-1, keepdims=True)
        o = np.matmul(p, np.transpose(vs, (1, 0, 2)))  # [hkv, g, dv]
        out[b] = o.reshape(hq, -1)
        lse[b] = (smax[..., 0] + np.log(np.sum(e, axis=-1))).reshape(hq)
    return (out, lse) if return_lse else out


def paged_cache_load_golden(key_cache, value_cache, block_tables, seq_lens, seq_starts=None,
                            seq_lens_cumsum=False):
    """Gather the token rows of every sequence from the paged caches (ND layout).

    Follows tests/st/test_custom_paged_cache_load.py:35-76 (``golden_calc_nd``):
      * sequence ``i`` has ``seq_lens[i]`` tokens, or ``seq_lens[i+1] - seq_lens[i]``
        when `seq_lens` holds running sums (``seq_lens_cumsum``),
      * its token ``j`` lies in block ``block_tables[i][seq_starts[i] // bs + j // bs]``
        at offset ``j % bs`` (`seq_starts` absent: column ``j // bs``),
      * a negative block id contributes no row and does not advance the output
        row; the rows left over at the end stay zero.
    The reference's golden ties the cumulative lengths to the presence of
    `seq_starts`; the operator has one flag for each, so both are arguments.
    Caches ``[num_blocks, bs, heads, head_size]``; returns
    ``(key_out [sum, heads, dk], value_out [sum, heads, dv])`` in the cache dtypes.
    """
    kc, vc = np.asarray(key_cache), np.asarray(value_cache)
    tables = np.asarray(block_tables)
    lens = np.asarray(seq_lens).astype(np.int64).reshape(-1)
    bs = kc.shape[1]
    if seq_lens_cumsum:
        total, lens = int(lens[-1]), np.diff(lens)
    else:
        total = int(lens.sum())
    k_out = np.zeros((total,) + kc.shape[2:], dtype=kc.dtype)
    v_out = np.zeros((total,) + vc.shape[2:], dtype=vc.dtype)
    row = 0
    for i, n in enumerate(lens):
        n = int(n)
        col0 = 0 if seq_starts is None else int(np.asarray(seq_starts)[i]) // bs
        for j in range(0, n, bs):
            bid = int(tables[i][col0 + j // bs])
            if bid < 0:
                continue
            m = min(bs, n - j)
            k_out[row:row + m] = kc[bid, :m]
            v_out[row:row + m] = vc[bid, :m]
            row += m
    return k_out, v_out


def fa_update_golden(lse, partial_out):
    """Merge `sp` normalised partial attention outputs by their log-sum-exps.

    Follows tests/st/test_asd_faupdate.py:34-59:
    ``w = exp(lse) / sum_s exp(lse); out = sum_s w_s * O_s``.
    `lse` [sp, n] (natural log), `partial_out` [sp, n, d]; returns [n, d].
    """
    lse = np.asarray(lse, dtype=np.float32)
    po = np.asarray(partial_out, dtype=np.float32)
    w = np.exp(lse)
    w = w / np.sum(w, axis=0, keepdims=True)
    return np.sum(po * w[:, :, None], axis=0)


# --------------------------------------------------------------------------
# acceptance rules
# --------------------------------------------------------------------------
def reference_accuracy_verdict(output, golden, dtype, num_heads, max_context_len, is_quant=False):
    """The reference's acceptance rule: ``adaptive_pass or legacy_pass``.

    Follows tests/st/test_custom_paged_attention.py:1005-1099.  `dtype` is one
    of "float16", "bfloat16", "float32".  Returns (ok, detail dict).
    """
    o = np.asarray(output).astype(np.float32).ravel()
    g = np.asarray(golden).astype(np.float32).ravel()
    diff = np.abs(o - g)
    rel_strict = abs_strict = 0.005
    s = 2.0 if (dtype == "bfloat16" and is_quant) else 1.0
    strict_limit = np.maximum(np.abs(g) * rel_strict * s, abs_strict * s)
    n = max(1, o.size)
    ratio = float(np.sum(diff > strict_limit)) / n
    if dtype == "bfloat16" or is_quant:
        legacy = ratio <= rel_strict * s
    else:
        legacy = ratio <= 0.001
    calc = num_heads * max_context_len + 4
    if dtype == "bfloat16":
        f = (2.0 ** -7 if calc < 2048 else 2.0 ** -6) * (2.0 if is_quant else 1.0)
    elif dtype == "float16":
        f = 2.0 ** -8 if calc < 2048 else 2.0 ** -7
    else:
        f = 2.0 ** -11 if calc < 2048 else (2.0 ** -10 if calc < 16384 else 2.0 ** -9)
    adaptive = bool(np.all(diff <= np.maximum(np.abs(g), 1.0) * f))
    return bool(adaptive or legacy), {
        "max_diff": float(diff.max()) if diff.size else 0.0,
        "strict_error_ratio": ratio, "legacy": bool(legacy), "adaptive": adaptive,
    }


def scale_free_error(output, golden):
    """(max|diff| / max|golden|, relative L2): magnitude-independent metrics."""
    o = np.asarray(output).astype(np.float32)
    g = np.asarray(golden).astype(np.float32)
    gm = float(np.max(np.abs(g))) or 1.0
    gn = float(np.linalg.norm(g)) or 1.0
    return float(np.max(np.abs(o - g))) / gm, float(np.linalg.norm(o - g)) / gn
