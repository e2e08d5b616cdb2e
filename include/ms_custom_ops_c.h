/*
 * ms_custom_ops_c.h -- operator-level C ABI of libms_custom_ops_host.so.
 *
 * One entry point per operator the plugin registers for the paged-KV decode
 * path, with the registered argument lists unchanged (names, order, meaning,
 * defaults are in the *_op.yaml files next to the C++ sources):
 *
 *   reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, cache_mode, head_num)
 *       reference: ops/c_api/reshape_and_cache/reshape_and_cache_op.yaml:2-31,
 *                  pybind definition ops/c_api/reshape_and_cache/reshape_and_cache.cc:204-217
 *   paged_attention(query, key_cache, value_cache, block_tables, context_lens, attn_mask,
 *                   batch_run_status, k_descale, k_offset, v_descale, v_offset, razor_offset,
 *                   p_scale, log_n, q_seq_lens, q_head_num, qk_scale, kv_head_num, mask_type,
 *                   batch_run_status_enable, quant_type, out_data_type, has_quant_offset,
 *                   compress_type, calc_type, scale_type, input_layout, mla_v_dim, input_format)
 *       reference: ops/c_api/paged_attention/paged_attention_op.yaml:2-88,
 *                  pybind definition ops/c_api/paged_attention/paged_attention_pynative.cc:743-777
 *   paged_cache_load(key_cache, value_cache, block_tables, seq_lens, seq_starts, kv_cache_cfg,
 *                    is_seq_lens_cumsum_type, has_seq_starts) -> (key_out, value_out)
 *       reference: ops/c_api/paged_cache_load/paged_cache_load_op.yaml:2-28,
 *                  pybind definition ops/c_api/paged_cache_load/paged_cache_load_pynative.cc:129-134
 *   reshape_and_cache_npd(key, value, key_cache, value_cache, slot_mapping, actual_seq_qlen,
 *                         actual_seq_kvlen, block_tbl, kv_cache_layout, key_value_layout) -> (out_key, out_value)
 *       reference: ops/ascendc/ms_glue/reshape_and_cache_npd/reshape_and_cache_npd_op.yaml
 *   fa_update(lse, local_out, fa_update_type, sp) -> output
 *       reference: ops/c_api/fa_update/fa_update_op.yaml:2-16,
 *                  pybind definition ops/c_api/fa_update/fa_update_pynative.cc:85-88
 *
 * This is what a binding (pybind11, ctypes, a framework's custom-op adapter)
 * calls instead of the reference's `pyboost_*` functions.  Tensors are passed
 * as plain descriptors; optional tensors are NULL.  The functions validate
 * exactly as the reference's eager path does, then plan and launch on the
 * given CUDA stream through libmsco_b200.so.  They never allocate device
 * memory: outputs and the attention workspace come from the caller (the
 * framework's allocator), as in the reference where MindSpore allocates both.
 */
#ifndef MS_CUSTOM_OPS_C_H_
#define MS_CUSTOM_OPS_C_H_

#include <stddef.h>
#include <stdint.h>

#include "msco_b200.h" /* MSCO_DTYPE_*, MSCO_* status codes */

#ifdef __cplusplus
extern "C" {
#endif

/* error kinds: which exception the reference would have raised */
#define MS_ERR_KIND_NONE 0
#define MS_ERR_KIND_VALUE 1       /* MS_EXCEPTION(ValueError) / MS_CHECK_VALUE          */
#define MS_ERR_KIND_TYPE 2        /* dtype rules                                          */
#define MS_ERR_KIND_RUNTIME 3     /* MS_LOG(EXCEPTION), launch failures                   */
#define MS_ERR_KIND_UNSUPPORTED 4 /* valid in the reference, not built for B200           */

#define MS_MAX_DIMS 8

typedef struct MsTensorDesc {
  void *data;                  /* device address (host address when on_host != 0)          */
  int32_t dtype;               /* MSCO_DTYPE_*                                              */
  int32_t ndim;
  int64_t shape[MS_MAX_DIMS];
  int64_t strides[MS_MAX_DIMS]; /* in elements; must describe a contiguous tensor          */
  int32_t on_host;             /* context_lens / q_seq_lens / batch_run_status live on host */
  int32_t reserved;
} MsTensorDesc;

/* reshape_and_cache.  Returns MSCO_OK or an MSCO_ERR_* code.  The operator's
 * dummy output ("fake_out", same shape and dtype as key) is not materialised. */
int ms_custom_ops_reshape_and_cache(const MsTensorDesc *key, const MsTensorDesc *value,
                                    const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                    const MsTensorDesc *slot_mapping, int64_t cache_mode, int64_t head_num,
                                    void *stream);

/* Shape / dtype inference of the operator's placeholder output after the operator's checks: key's
 * shape and dtype (CustomReshapeAndCacheOpFuncImpl::InferShape / InferType,
 * ops/c_api/reshape_and_cache/reshape_and_cache.cc:66-75).  Graph-mode frameworks need it to wire the
 * side-effect operator into a graph; the eager entry point has no output
 * (PyboostRunner::Call<0>, reshape_and_cache.cc:204-210) and nothing is ever written to it. */
int ms_custom_ops_reshape_and_cache_infer(const MsTensorDesc *key, const MsTensorDesc *value,
                                          const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                          const MsTensorDesc *slot_mapping, int64_t cache_mode, int64_t head_num,
                                          int32_t *out_dtype, int32_t *out_ndim,
                                          int64_t *out_shape /* [MS_MAX_DIMS] */);

/* reshape_and_cache_npd (reference: ops/ascendc/ms_glue/reshape_and_cache_npd/reshape_and_cache_npd_op.yaml,
 * argument meaning reshape_and_cache_npd.md:11-34): the cache write in either block layout,
 * kv_cache_layout "BSND" (num_blocks, block_size, heads, head_dim) or "BNSD" (num_blocks, heads, block_size,
 * head_dim), with the current key / value returned in the "TH" layout (tokens, heads * head_dim): out_key /
 * out_value are caller-allocated with key's / value's shape and dtype and receive copies (NULL: no output).
 * key_value_layout "NPD" (re-blocked outputs with the cached history, an input format of the Ascend attention
 * kernels) fails with MSCO_ERR_UNSUPPORTED.  actual_seq_qlen / actual_seq_kvlen / block_tbl only serve
 * that layout; they are type-checked when given and otherwise unused. */
int ms_custom_ops_reshape_and_cache_npd_infer(
    const MsTensorDesc *key, const MsTensorDesc *value, const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
    const MsTensorDesc *slot_mapping, const MsTensorDesc *actual_seq_qlen, const MsTensorDesc *actual_seq_kvlen,
    const MsTensorDesc *block_tbl, const char *kv_cache_layout, const char *key_value_layout, int32_t *out_key_dtype,
    int32_t *out_value_dtype, int32_t *out_ndim, int64_t *out_key_shape /* [MS_MAX_DIMS] */,
    int64_t *out_value_shape /* [MS_MAX_DIMS] */);
int ms_custom_ops_reshape_and_cache_npd(
    const MsTensorDesc *key, const MsTensorDesc *value, const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
    const MsTensorDesc *slot_mapping, const MsTensorDesc *actual_seq_qlen, const MsTensorDesc *actual_seq_kvlen,
    const MsTensorDesc *block_tbl, const char *kv_cache_layout, const char *key_value_layout,
    const MsTensorDesc *out_key, const MsTensorDesc *out_value, void *stream);

/* Extension (no reference counterpart): quantise fp16/bf16 rows to the int8
 * cache on the way in; inverse of paged_attention's quant_type = 1 formula. */
int ms_custom_ops_reshape_and_cache_quant(const MsTensorDesc *key, const MsTensorDesc *value,
                                          const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                          const MsTensorDesc *slot_mapping, const MsTensorDesc *k_descale,
                                          const MsTensorDesc *v_descale, const MsTensorDesc *k_offset,
                                          const MsTensorDesc *v_offset, void *stream);

/* The 29 registered arguments of paged_attention, in registration order. */
typedef struct MsPagedAttentionArgs {
  const MsTensorDesc *query;
  const MsTensorDesc *key_cache;
  const MsTensorDesc *value_cache;
  const MsTensorDesc *block_tables;
  const MsTensorDesc *context_lens; /* int32, on host */
  const MsTensorDesc *attn_mask;
  const MsTensorDesc *batch_run_status;
  const MsTensorDesc *k_descale;
  const MsTensorDesc *k_offset;
  const MsTensorDesc *v_descale;
  const MsTensorDesc *v_offset;
  const MsTensorDesc *razor_offset;
  const MsTensorDesc *p_scale;
  const MsTensorDesc *log_n;
  const MsTensorDesc *q_seq_lens;
  int64_t q_head_num;
  double qk_scale;
  int64_t kv_head_num;
  int64_t mask_type;
  int32_t batch_run_status_enable;
  int64_t quant_type;
  int64_t out_data_type;
  int32_t has_quant_offset;
  int64_t compress_type;
  int64_t calc_type;
  int64_t scale_type;
  int64_t input_layout;
  int64_t mla_v_dim;
  int64_t input_format;
} MsPagedAttentionArgs;

/* Shape / dtype inference of attention_out (query's shape and dtype), after
 * the same parameter, shape and type checks the launch performs. */
int ms_custom_ops_paged_attention_infer(const MsPagedAttentionArgs *args, int32_t *out_dtype,
                                        int32_t *out_ndim, int64_t *out_shape /* [MS_MAX_DIMS] */);

/* Bytes of device workspace the launch with these arguments needs (plan phase;
 * reads context_lens on the host; no device work). */
int ms_custom_ops_paged_attention_workspace_size(const MsPagedAttentionArgs *args, size_t *bytes);

/* Validate, plan (cached by a hash of attributes, shapes and context_lens),
 * launch on `stream`.  `attention_out` is caller-allocated with the inferred
 * shape / dtype; `workspace` is 256-byte aligned device memory of at least
 * the size reported above and must stay untouched until the launch finished. */
int ms_custom_ops_paged_attention(const MsPagedAttentionArgs *args, const MsTensorDesc *attention_out,
                                  void *workspace, size_t workspace_bytes, void *stream);

/* Extension (no reference counterpart): the same operator with a second output, `lse_out` Float32
 * (batch, q_head_num) = log of the sum over the context of exp(qk_scale * q.k + mask) (natural
 * logarithm; -inf for an empty context).  It is what fa_update needs to merge attention outputs
 * computed over different parts of a context (sequence-parallel decode).  Same workspace rules. */
int ms_custom_ops_paged_attention_with_lse(const MsPagedAttentionArgs *args, const MsTensorDesc *attention_out,
                                           const MsTensorDesc *lse_out, void *workspace, size_t workspace_bytes,
                                           void *stream);

/* Workspace bytes the calling thread's last ms_custom_ops_paged_attention call needed.  A caller
 * that keeps a grow-only workspace can skip the separate size query: launch with what it has and,
 * if the call fails because the workspace is too small (nothing was launched), grow it to this
 * size and call again. */
size_t ms_custom_ops_paged_attention_last_workspace_need(void);

/* After synchronising `stream`: MSCO_OK, MSCO_ERR_TIMEOUT or MSCO_ERR_OOB as
 * left in `workspace` by the last paged_attention launch that used it. */
int ms_custom_ops_paged_attention_status(const void *workspace);

/* paged_cache_load.  Shape / dtype inference of (key_out, value_out) after the operator's checks:
 * both have rank 3, (sum_context_lens, num_heads, head_size_k / head_size_v), in the dtypes of the
 * caches.  sum_context_lens is the sum of seq_lens (its last element in cumulative mode) when
 * `seq_lens` is readable on the host (on_host != 0), else -1: a dimension only known at run time,
 * as in the reference's infer function (paged_cache_load_graph.cc:23-60). */
int ms_custom_ops_paged_cache_load_infer(const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                         const MsTensorDesc *block_tables, const MsTensorDesc *seq_lens,
                                         const MsTensorDesc *seq_starts, int64_t kv_cache_cfg,
                                         int32_t is_seq_lens_cumsum_type, int32_t has_seq_starts,
                                         int32_t *key_out_dtype, int32_t *value_out_dtype, int32_t *out_ndim,
                                         int64_t *key_out_shape /* [MS_MAX_DIMS] */,
                                         int64_t *value_out_shape /* [MS_MAX_DIMS] */);

/* Bytes of device workspace the launch needs for this block table (0 for a malformed descriptor). */
size_t ms_custom_ops_paged_cache_load_workspace_size(const MsTensorDesc *block_tables);

/* Validate and launch on `stream`.  block_tables, seq_lens and seq_starts are device tensors (the
 * kernels read them; nothing is copied to the host).  key_out / value_out are caller-allocated with
 * the inferred shapes: their first dimension is the row count the caller computed from seq_lens; rows
 * the lengths do not cover are never written past, rows no block was gathered into are zeroed.
 * `workspace`: 4-byte aligned device memory of the size reported above, not shared with a launch in flight. */
int ms_custom_ops_paged_cache_load(const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                   const MsTensorDesc *block_tables, const MsTensorDesc *seq_lens,
                                   const MsTensorDesc *seq_starts, int64_t kv_cache_cfg,
                                   int32_t is_seq_lens_cumsum_type, int32_t has_seq_starts,
                                   const MsTensorDesc *key_out, const MsTensorDesc *value_out, void *workspace,
                                   size_t workspace_bytes, void *stream);

/* fa_update.  Inference: output is Float32 (rows, head_size) for local_out (sp, rows, head_size). */
int ms_custom_ops_fa_update_infer(const MsTensorDesc *lse, const MsTensorDesc *local_out, int64_t fa_update_type,
                                  int64_t sp, int32_t *out_dtype, int32_t *out_ndim,
                                  int64_t *out_shape /* [MS_MAX_DIMS] */);
int ms_custom_ops_fa_update(const MsTensorDesc *lse, const MsTensorDesc *local_out, int64_t fa_update_type,
                            int64_t sp, const MsTensorDesc *output, void *stream);

const char *ms_custom_ops_last_error(void);
int ms_custom_ops_last_error_kind(void);

/* Registered operators (the plugin's registry): count, names, signatures. */
int ms_custom_ops_num_ops(void);
const char *ms_custom_ops_op_name(int index);
const char *ms_custom_ops_op_signature(int index);

/* Plan cache (the role of the reference's tiling cache): statistics and reset. */
void ms_custom_ops_plan_cache_stats(int64_t *hits, int64_t *misses, int64_t *entries);
void ms_custom_ops_plan_cache_clear(void);
/* How the misses were served: by re-planning an existing plan in place (no allocation), or by
 * building a new plan.  In a decode loop, where every step is a miss, only `recycled` grows. */
void ms_custom_ops_plan_cache_miss_stats(int64_t *recycled, int64_t *created);
/* The pinned plan memory pool behind the plans (role of the reference's TilingMemMgr,
 * ops/framework/ms_kernels_internal/tiling_mem_mgr.cc:82-137): same six numbers as
 * msco_plan_arena_stats. */
void ms_custom_ops_plan_arena_stats(int64_t *stats /* [6] */);

#ifdef __cplusplus
}
#endif
#endif /* MS_CUSTOM_OPS_C_H_ */
