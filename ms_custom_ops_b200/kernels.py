"""Thin-ABI launchers: torch tensors in, libmsco_b200.so kernels on torch's current stream.

PyTorch is used here only as the owner of device memory and streams; every
byte of arithmetic happens in the library's CUDA kernels.  These helpers do no
argument validation beyond what the C ABI itself checks -- the operator-level
API (``ms_custom_ops_b200.reshape_and_cache`` / ``paged_attention``) does that.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _abi

_TORCH2MSCO = {torch.float16: _abi.DTYPE_F16, torch.bfloat16: _abi.DTYPE_BF16, torch.int8: _abi.DTYPE_I8,
               torch.float32: _abi.DTYPE_F32, torch.int32: _abi.DTYPE_I32, torch.int64: _abi.DTYPE_I64}


def msco_dtype(t: torch.dtype) -> int:
    return _TORCH2MSCO[t]


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def rac_scatter(key, value, key_cache, value_cache, slot_mapping, oob_count=None):
    """msco_reshape_and_cache on the current stream (bit copy of token rows into cache slots)."""
    t = slot_mapping.numel()
    krow = key.numel() // max(t, 1) * key.element_size()
    vrow = 0 if value is None else value.numel() // max(t, 1) * value.element_size()
    nslots = key_cache.shape[0] * key_cache.shape[1]
    _abi.check(_abi.lib().msco_reshape_and_cache(
        _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache), _ptr(slot_mapping), t, krow, vrow, nslots,
        _ptr(oob_count), _stream()))


def rac_scatter_bnsd(key, value, key_cache, value_cache, slot_mapping, oob_count=None):
    """msco_reshape_and_cache_bnsd on the current stream: caches are [num_blocks, heads, block_size, head_dim]."""
    t = slot_mapping.numel()
    nb, heads, bs, kd = key_cache.shape
    vd = 0 if value_cache is None else value_cache.shape[3]
    _abi.check(_abi.lib().msco_reshape_and_cache_bnsd(
        _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache), _ptr(slot_mapping), t, heads,
        kd * key.element_size(), 0 if value is None else vd * value.element_size(), bs, nb * bs, _ptr(oob_count),
        _stream()))


def rac_scatter_quant(key, value, key_cache, value_cache, slot_mapping, k_descale, v_descale,
                      k_offset=None, v_offset=None, oob_count=None):
    """msco_reshape_and_cache_quant on the current stream (fp16/bf16 rows -> int8 cache)."""
    t = slot_mapping.numel()
    krow = key.numel() // max(t, 1)
    vrow = 0 if value is None else value.numel() // max(t, 1)
    nslots = key_cache.shape[0] * key_cache.shape[1]
    _abi.check(_abi.lib().msco_reshape_and_cache_quant(
        _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache), _ptr(slot_mapping), t, krow, vrow,
        msco_dtype(key.dtype), _ptr(k_descale), _ptr(k_offset), _ptr(v_descale), _ptr(v_offset), nslots,
        _ptr(oob_count), _stream()))


def cache_load_workspace_bytes(batch: int, max_blocks_per_seq: int) -> int:
    return int(_abi.lib().msco_paged_cache_load_workspace_bytes(int(batch), int(max_blocks_per_seq)))


def cache_load(key_cache, value_cache, block_tables, seq_lens, seq_starts, key_out, value_out, workspace,
               seq_lens_cumsum=False, oob_count=None):
    """msco_paged_cache_load on the current stream (gather the rows of every sequence)."""
    nb, bs = key_cache.shape[0], key_cache.shape[1]
    krow = key_cache[0, 0].numel() * key_cache.element_size()
    vrow = value_cache[0, 0].numel() * value_cache.element_size()
    _abi.check(_abi.lib().msco_paged_cache_load(
        _ptr(key_cache), _ptr(value_cache), _ptr(block_tables), _ptr(seq_lens), _ptr(seq_starts), _ptr(key_out),
        _ptr(value_out), block_tables.shape[0], block_tables.shape[1], bs, nb, krow, vrow, key_out.shape[0],
        int(bool(seq_lens_cumsum)), _ptr(workspace), workspace.numel() * workspace.element_size(), _ptr(oob_count),
        _stream()))


def merge_partials(lse, local_out, out):
    """msco_fa_update on the current stream: out[r] = sum_s softmax_s(lse)[s, r] * local_out[s, r]."""
    sp, rows, hd = local_out.shape
    _abi.check(_abi.lib().msco_fa_update(_ptr(lse), _ptr(local_out), _ptr(out), rows, hd, sp, _stream()))


def merge_partials_strided(lse, lse_stride, local_out, local_out_stride, out, sp):
    """msco_fa_update_strided on the current stream.  `lse` / `local_out` point at partition 0; partition s
    lies lse_stride floats / local_out_stride elements further; `out` [rows, head_size] has local_out's dtype."""
    rows, hd = out.shape[-2] if out.dim() == 2 else out.numel() // out.shape[-1], out.shape[-1]
    _abi.check(_abi.lib().msco_fa_update_strided(_ptr(lse), int(lse_stride), _ptr(local_out), int(local_out_stride),
                                                 msco_dtype(out.dtype), _ptr(out), rows, hd, int(sp), _stream()))


def make_pa_desc(query, key_cache, block_tables, qk_scale, quant_type=0, has_quant_offset=False,
                 mask=None, mask_type=0, kernel=_abi.KERNEL_AUTO, cache_layout=0) -> _abi.MscoPaDesc:
    """`cache_layout` 0: caches [num_blocks, block_size, kv_heads, head_dim]; 1: [num_blocks, kv_heads, block_size, head_dim]."""
    d = _abi.MscoPaDesc()
    d.q_dtype = msco_dtype(query.dtype)
    d.kv_dtype = msco_dtype(key_cache.dtype)
    d.num_q_heads = query.shape[1]
    d.num_kv_heads = key_cache.shape[1 if cache_layout else 2]
    d.head_dim = query.shape[2]
    d.block_size = key_cache.shape[2 if cache_layout else 1]
    d.cache_layout = int(cache_layout)
    d.num_blocks = key_cache.shape[0]
    d.max_blocks_per_seq = block_tables.shape[1]
    d.qk_scale = float(qk_scale)
    d.quant_type = int(quant_type)
    d.has_quant_offset = int(bool(has_quant_offset))
    d.mask_type = int(mask_type)
    if mask is not None and mask_type:
        d.mask_dtype = msco_dtype(mask.dtype)
        d.mask_batch_stride = mask.stride(0)
        d.mask_head_stride = mask.stride(1) if mask_type == 2 else 0
    d.kernel = int(kernel)
    return d


def pa_launch(plan: _abi.PaPlan, query, key_cache, value_cache, block_tables, out, workspace,
              k_descale=None, k_offset=None, v_descale=None, v_offset=None, mask=None, lse=None):
    """msco_paged_attention_launch on the current stream (with `lse`: ..._launch_lse)."""
    if lse is not None:
        _abi.check(_abi.lib().msco_paged_attention_launch_lse(
            plan.handle, _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(block_tables), _ptr(k_descale),
            _ptr(k_offset), _ptr(v_descale), _ptr(v_offset), _ptr(mask), _ptr(out), _ptr(lse), _ptr(workspace),
            workspace.numel() * workspace.element_size(), _stream()))
        return
    _abi.check(_abi.lib().msco_paged_attention_launch(
        plan.handle, _ptr(query), _ptr(key_cache), _ptr(value_cache), _ptr(block_tables), _ptr(k_descale),
        _ptr(k_offset), _ptr(v_descale), _ptr(v_offset), _ptr(mask), _ptr(out), _ptr(workspace),
        workspace.numel() * workspace.element_size(), _stream()))


def decode_step(plan: _abi.PaPlan, key, value, key_cache, value_cache, slot_mapping, query, block_tables, out,
                workspace, k_descale=None, k_offset=None, v_descale=None, v_offset=None, mask=None, gather=None):
    """msco_decode_step on the current stream: cache scatter + attention in one call.
    `gather` (a sharding.PeerGather): msco_decode_step_gather instead -- the kernel that finishes the
    output rows also pushes them to the peers; returns this rank's gathered buffer then."""
    args = (plan.handle, _ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache), _ptr(slot_mapping),
            slot_mapping.numel(), _ptr(query), _ptr(block_tables), _ptr(k_descale), _ptr(k_offset), _ptr(v_descale),
            _ptr(v_offset), _ptr(mask), _ptr(out), _ptr(workspace), workspace.numel() * workspace.element_size(),
            _stream())
    if gather is None:
        _abi.check(_abi.lib().msco_decode_step(*args))
        return None
    desc, step, buf = gather.next_step()
    _abi.check(_abi.lib().msco_decode_step_gather(*args, desc, step))
    return buf


def pa_status(plan: _abi.PaPlan, workspace) -> int:
    """Status word left by the kernels (synchronises); raises MscoError unless OK."""
    torch.cuda.current_stream().synchronize()
    _abi.check(_abi.lib().msco_paged_attention_status(plan.handle, _ptr(workspace)))
    return _abi.OK


def paged_attention_raw(query, key_cache, value_cache, block_tables, context_lens, qk_scale, quant_type=0,
                        k_descale=None, k_offset=None, v_descale=None, v_offset=None, mask=None, mask_type=0,
                        kernel=_abi.KERNEL_AUTO, check_status=True, lse=None, cache_layout=0):
    """Plan + launch + (optionally) status check in one call; returns (out, plan info).
    `lse`: optional float32 [batch, q_heads] tensor that receives the log-sum-exp of the scores."""
    desc = make_pa_desc(query, key_cache, block_tables, qk_scale, quant_type,
                        k_offset is not None, mask, mask_type, kernel, cache_layout)
    plan = _abi.PaPlan(desc, [int(x) for x in context_lens])
    ws = torch.empty(max(plan.workspace_bytes, 256), dtype=torch.uint8, device=query.device)
    out = torch.empty_like(query)
    pa_launch(plan, query, key_cache, value_cache, block_tables, out, ws, k_descale, k_offset, v_descale,
              v_offset, mask, lse)
    info = plan.info()
    if check_status:
        pa_status(plan, ws)
    else:
        torch.cuda.current_stream().synchronize()
    plan.close()
    return out, info
