/*
 * msco_b200.h -- C ABI of libmsco_b200.so: the B200 (sm_100a) kernels behind
 * the `reshape_and_cache` and `paged_attention` operators.
 *
 * This is the boundary the reference crosses when its operator glue calls the
 * closed kernel library (`internal_v2::InternalOp`): create an op, hand it a
 * host-side parameter block (which for paged attention includes the host copy
 * of `context_lens`), ask for the workspace size, then launch on the caller's
 * stream with raw device addresses.  Reference call sites replaced:
 *   ops/c_api/reshape_and_cache/reshape_and_cache.cc:48-60      (CreateAsdReshapeAndCacheOp)
 *   ops/c_api/paged_attention/paged_attention_graph.cc:718-806  (CreateCustomPagedAttentionOp + param fill)
 *   ops/c_api/paged_attention/paged_attention_graph.cc:808-856  (UpdateParam on new lengths, tiling key)
 *   ops/framework/ms_kernels_internal/graphmode/internal_kernel_mod.cc:158-203,341-365
 *   ops/framework/ms_kernels_internal/pyboost/internal_pyboost_runner.cc:93-141,210-231
 *                                                               (tiling, workspace, InternalOp::Launch)
 *
 * Conventions
 *   - plain pointers and sizes only; every `void *stream` is a cudaStream_t;
 *   - all tensors are contiguous, row-major, in the layouts documented below;
 *   - every function returns an MSCO_* code; msco_last_error() gives the
 *     message of the last failure on the calling thread;
 *   - launches are asynchronous on `stream`; nothing here synchronises;
 *   - no entry point below allocates device memory: caches, outputs and the
 *     paged-attention workspace are caller-owned.
 */
#ifndef MSCO_B200_H_
#define MSCO_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSCO_ABI_VERSION 1

/* status codes */
#define MSCO_OK 0
#define MSCO_ERR_INVALID_ARG 1 /* a shape / pointer / attribute violates the contract      */
#define MSCO_ERR_UNSUPPORTED 2 /* valid for the reference operator, not built for B200     */
#define MSCO_ERR_CUDA 3        /* a CUDA runtime / driver call failed                      */
#define MSCO_ERR_TIMEOUT 4     /* a bounded device-side wait gave up (see msco_paged_attention_status) */
#define MSCO_ERR_OOB 5         /* a slot or block id is outside the cache                  */
#define MSCO_ERR_INTERNAL 6

/* element types */
#define MSCO_DTYPE_F16 0
#define MSCO_DTYPE_BF16 1
#define MSCO_DTYPE_I8 2
#define MSCO_DTYPE_F32 3
#define MSCO_DTYPE_I32 4
#define MSCO_DTYPE_I64 5

int msco_version(void);
const char *msco_last_error(void);

/* ------------------------------------------------------------------------
 * reshape_and_cache: scatter token rows into the paged cache.
 *
 * Replaces the device op created at reshape_and_cache.cc:55-59 (ND cache
 * format only).  For every token i with s = slot_mapping[i] >= 0 the row
 * key[i, :] (k_row_bytes bytes) is copied bit-for-bit to
 * key_cache + s * k_row_bytes, i.e. to cache[s / block_size, s % block_size]
 * of a contiguous [num_blocks, block_size, kv_heads, head_dim] cache; the
 * same for value.  Negative slots are skipped.  Duplicate non-negative slots
 * race (as in the reference, which requires unique slots).
 *
 * value / value_cache may both be NULL (key-only mode).  Row sizes must be
 * multiples of 2 bytes; the fast path needs 16-byte aligned pointers and row
 * sizes that are multiples of 16 bytes and falls back to a 2-byte path
 * otherwise.  num_slots = num_blocks * block_size bounds the slot check:
 * slots >= num_slots are not written and are counted in *oob_count when
 * oob_count (device int32, may be NULL) is given.
 * ---------------------------------------------------------------------- */
int msco_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                           const int32_t *slot_mapping, int64_t num_tokens, int64_t k_row_bytes,
                           int64_t v_row_bytes, int64_t num_slots, int32_t *oob_count, void *stream);

/* The same scatter into head-major cache blocks, [num_blocks, num_heads, block_size, head_dim] -- the
 * "BNSD" cache layout of the reference's reshape_and_cache_npd (cache shapes
 * ops/ascendc/ms_glue/reshape_and_cache_npd/reshape_and_cache_npd.md:24-25, addressing
 * ops/ascendc/aclnn_src/reshape_and_cache_npd/op_kernel/reshape_and_cache_npd.cpp:167-173): head h of
 * token i goes to key_cache + ((s / block_size * num_heads + h) * block_size + s % block_size) * k_head_bytes
 * for s = slot_mapping[i] >= 0.  key [num_tokens, num_heads * k_head_bytes], value likewise (may be NULL
 * together with value_cache). */
int msco_reshape_and_cache_bnsd(const void *key, const void *value, void *key_cache, void *value_cache,
                                const int32_t *slot_mapping, int64_t num_tokens, int32_t num_heads,
                                int64_t k_head_bytes, int64_t v_head_bytes, int32_t block_size,
                                int64_t num_slots, int32_t *oob_count, void *stream);

/* Asynchronous device-to-device copy on `stream` (the pass-through outputs of reshape_and_cache_npd;
 * lets the operator layer stay free of the CUDA runtime). */
int msco_copy_device(void *dst, const void *src, size_t bytes, void *stream);

/* ------------------------------------------------------------------------
 * Quantising variant (extension; the reference operator has no such mode).
 * Rows arrive in fp16/bf16 (in_dtype), the caches are int8, and per channel
 * c = (kv_head, head_dim):
 *     q = saturate_int8( rint( (float)x / descale[c] ) - offset[c] )
 * with IEEE float32 division and round-half-to-even: the exact inverse of the
 * de-quantisation paged_attention applies with quant_type = 1.
 * k_offset / v_offset may be NULL (offset 0).
 * ---------------------------------------------------------------------- */
int msco_reshape_and_cache_quant(const void *key, const void *value, int8_t *key_cache,
                                 int8_t *value_cache, const int32_t *slot_mapping,
                                 int64_t num_tokens, int64_t k_row_elems, int64_t v_row_elems,
                                 int32_t in_dtype, const float *k_descale, const int32_t *k_offset,
                                 const float *v_descale, const int32_t *v_offset, int64_t num_slots,
                                 int32_t *oob_count, void *stream);

/* ------------------------------------------------------------------------
 * paged_cache_load: gather the token rows of every sequence from the paged
 * caches into contiguous outputs -- the inverse movement of reshape_and_cache.
 * Replaces the device work behind npu_paged_cache_load
 * (ops/c_api/paged_cache_load/paged_cache_load_pynative.cc:48-117), ND layout
 * (kv_cache_cfg = 0; argument meaning ops/c_api/paged_cache_load/paged_cache_load_doc.md:9-27,
 * arithmetic tests/st/test_custom_paged_cache_load.py:35-76):
 *
 *   key_cache   [num_blocks, block_size, k_row_bytes]   value_cache likewise with v_row_bytes
 *   block_tables int32 [batch, max_blocks_per_seq]
 *   seq_lens     int32 [batch] lengths, or [batch + 1] running sums when seq_lens_cumsum != 0
 *   seq_starts   int32 [batch] or NULL: sequence i is read from block-table column
 *                seq_starts[i] / block_size on (has_seq_starts of the operator)
 *   key_out / value_out [sum_tokens, k_row_bytes / v_row_bytes]
 *
 * Rows are bytes: K and V may differ in element type and head size.  Blocks
 * with a negative id contribute no rows (later rows move up) and the rows left
 * at the end of the outputs are zeroed, as in the reference's golden.  Lengths,
 * start columns or block ids out of range are skipped and counted in
 * *oob_count (may be NULL); nothing is written outside the outputs.
 * Everything is read on the device: no host copy of seq_lens is needed, and
 * the call only enqueues two kernels on `stream`.  `workspace` (4-byte aligned,
 * msco_paged_cache_load_workspace_bytes) holds the row offsets of every
 * (sequence, block) pair and must not be shared with a call in flight.
 * ---------------------------------------------------------------------- */
size_t msco_paged_cache_load_workspace_bytes(int32_t batch, int32_t max_blocks_per_seq);
int msco_paged_cache_load(const void *key_cache, const void *value_cache, const int32_t *block_tables,
                          const int32_t *seq_lens, const int32_t *seq_starts, void *key_out,
                          void *value_out, int32_t batch, int32_t max_blocks_per_seq, int32_t block_size,
                          int32_t num_blocks, int64_t k_row_bytes, int64_t v_row_bytes, int64_t sum_tokens,
                          int32_t seq_lens_cumsum, void *workspace, size_t workspace_bytes,
                          int32_t *oob_count, void *stream);

/* ------------------------------------------------------------------------
 * fa_update (DECODE_UPDATE): merge `sp` partial attention outputs by their
 * log-sum-exps.  Replaces the device work behind npu_fa_update
 * (ops/c_api/fa_update/fa_update_pynative.cc:48-77; doc fa_update_doc.md:3-24;
 * arithmetic tests/st/test_asd_faupdate.py:34-59):
 *   lse [sp, rows] float32 (natural log), local_out [sp, rows, head_size] float32,
 *   out [rows, head_size] float32 = sum_s softmax_s(lse)[s, row] * local_out[s, row, :].
 * A row whose lse are all -inf gives zeros.  sp <= 64.
 * ---------------------------------------------------------------------- */
int msco_fa_update(const float *lse, const float *local_out, float *out, int64_t rows, int32_t head_size,
                   int32_t sp, void *stream);

/* Extension (no reference counterpart): the same merge for partial outputs that are not one packed
 * float32 tensor.  `dtype` (MSCO_DTYPE_F32 / F16 / BF16) is the element type of local_out AND out
 * (what paged attention writes); partition s starts `lse_stride` floats after partition s - 1 in lse
 * and `local_out_stride` elements after it in local_out, so that the per-rank (output, lse) records of
 * an all-gathered buffer are merged where they lie.  head_size must be a multiple of 4; local_out, out
 * and the partition stride must be aligned to four elements. */
int msco_fa_update_strided(const float *lse, int64_t lse_stride, const void *local_out, int64_t local_out_stride,
                           int32_t dtype, void *out, int64_t rows, int32_t head_size, int32_t sp, void *stream);

/* ------------------------------------------------------------------------
 * paged_attention (decode: one query token per sequence).
 *
 * The descriptor carries what the reference puts into
 * CustomASDPagedAttentionParam (paged_attention_graph.cc:726-790) plus the
 * shapes the reference reads from its tensor infos.
 * ---------------------------------------------------------------------- */
typedef struct MscoPaDesc {
  int32_t q_dtype;            /* MSCO_DTYPE_F16 | MSCO_DTYPE_BF16; also the output dtype        */
  int32_t kv_dtype;           /* same as q_dtype, or MSCO_DTYPE_I8 when quant_type == 1         */
  int32_t num_q_heads;        /* q_head_num                                                     */
  int32_t num_kv_heads;       /* kv_head_num; divides num_q_heads                               */
  int32_t head_dim;           /* <= 256                                                         */
  int32_t block_size;         /* tokens per cache block                                         */
  int64_t num_blocks;         /* blocks in each cache                                           */
  int32_t max_blocks_per_seq; /* row length of block_tables                                     */
  float qk_scale;             /* "tor": multiplies q.k before the softmax                       */
  int32_t quant_type;         /* 0 = none, 1 = int8 KV with (x + offset) * descale              */
  int32_t has_quant_offset;   /* offsets are read only when non-zero                            */
  int32_t mask_type;          /* 0 = none, 1 = NORM, 2 = ALIBI (additive, decode shapes)        */
  int32_t mask_dtype;         /* dtype of attn_mask (F16 / BF16 / F32) when mask_type != 0      */
  int64_t mask_batch_stride;  /* elements between sequences in attn_mask                        */
  int64_t mask_head_stride;   /* elements between q heads (0 for NORM)                          */
  int32_t kernel;             /* 0 = auto, 1 = force the generic kernel, 2 = require the TMA kernel */
  int32_t cache_layout;       /* 0 = [num_blocks, block_size, kv_heads, head_dim] (the operator's input_layout 0,
                                 "BSND"); 1 = [num_blocks, kv_heads, block_size, head_dim] (input_layout 1, "BNSD") */
} MscoPaDesc;

typedef struct MscoPaPlan MscoPaPlan;

typedef struct MscoPaPlanInfo {
  int32_t kernel;          /* 1 = generic, 2 = TMA + tensor-core kernel                 */
  int32_t grid;            /* CTAs of the attention kernel                              */
  int32_t work_items;      /* (sequence, kv head, q-row block, KV split) items          */
  int32_t partials;        /* split partials that go through the reduce kernel          */
  int32_t max_splits;      /* largest split count of any sequence                       */
  int32_t rows_per_item;   /* q rows of one kv-head group handled by one item           */
  int64_t workspace_bytes; /* same as msco_paged_attention_workspace_bytes              */
  int64_t kv_tokens;       /* sum of context_lens                                       */
} MscoPaPlanInfo;

/* Split rule: tokens per KV split as a function of one sequence's length and
 * the cache element type (MSCO_DTYPE_*) only -- never of the batch -- so a
 * request's result is bitwise independent of what it is batched with. */
int32_t msco_paged_attention_split_tokens(int32_t context_len, int32_t kv_dtype); /* head_dim 128 */
int32_t msco_paged_attention_split_tokens_for(int32_t context_len, int32_t kv_dtype, int32_t head_dim);

/* 1 when the TMA + tensor-core kernel serves this descriptor (head_dim 128, or 64 / 256 with a 16-bit
 * cache; block_size 16 / 32 / 64 / 128, at most 64 for head_dim 256), 0 when the general kernel does. */
int32_t msco_paged_attention_tma_supported(const MscoPaDesc *desc);

/* Build the launch plan from the host copy of context_lens (the reference
 * reads the same host values into its param: paged_attention_graph.cc:773-776,
 * paged_attention_pynative.cc:686-692).  Pure host work.  The plan words live in
 * a block of a pooled page-locked arena (the role of the reference's
 * TilingMemMgr, ops/framework/ms_kernels_internal/tiling_mem_mgr.cc:82-137,
 * 224-238): slabs are obtained once, blocks are recycled, so planning does not
 * call cudaHostAlloc / cudaFreeHost in the steady state. */
int msco_paged_attention_plan(const MscoPaDesc *desc, const int32_t *host_context_lens, int32_t batch,
                              MscoPaPlan **plan);
/* Re-plan in place for new lengths (the reference re-tiles when the lengths change,
 * paged_attention_graph.cc:808-856): same descriptor, new context_lens, any batch.  The plan keeps
 * its arena block (a larger one is taken only when the batch outgrows it) and its tensor maps, so a
 * decode loop that re-plans every step allocates nothing.  Launches already enqueued are unaffected
 * (they carry their plan words with them; for plans too large for that the call first waits for the
 * pending upload).  Not thread-safe against launches of the same plan object.  On failure the plan
 * must not be launched again before a successful re-plan. */
int msco_paged_attention_replan(MscoPaPlan *plan, const int32_t *host_context_lens, int32_t batch);
/* Multi-token (speculative) queries, calc_type = 1 of the operator (q_seq_len of
 * CustomASDPagedAttentionParam, paged_attention_graph.cc:758-762), planned so that the context is read ONCE
 * for all query tokens of a sequence: sequence b has host_q_seq_lens[b] consecutive rows in `query` / `out`
 * (sum of them rows in total) and ONE row of block_tables.  Runs of up to 16 / (q heads per kv head)
 * consecutive tokens (8 / ... for head_dim 256) are stacked into the q rows of one work item.  The launch
 * entry points are the same; attn_mask, when given, has one row per query token (mask_type 1 with
 * mask_batch_stride = the row length: the operator's SPEC mask).  Needs the TMA kernel (MSCO_ERR_UNSUPPORTED
 * otherwise: plan one decode row per token with msco_paged_attention_plan + msco_expand_rows_i32 instead). */
int msco_paged_attention_plan_tokens(const MscoPaDesc *desc, const int32_t *host_context_lens,
                                     const int32_t *host_q_seq_lens, int32_t num_seqs, MscoPaPlan **plan);
int msco_paged_attention_replan_tokens(MscoPaPlan *plan, const int32_t *host_context_lens,
                                       const int32_t *host_q_seq_lens, int32_t num_seqs);
/* Counters of the plan arena: [0] slabs obtained (cudaHostAlloc calls), [1] their bytes, [2] blocks
 * in use, [3] block requests served, [4] requests larger than a slab, [5] 1 if page-locked. */
void msco_plan_arena_stats(int64_t *stats /* [6] */);
size_t msco_paged_attention_workspace_bytes(const MscoPaPlan *plan);
int msco_paged_attention_plan_info(const MscoPaPlan *plan, MscoPaPlanInfo *info);
void msco_paged_attention_plan_destroy(MscoPaPlan *plan);

/* Launch.  Layouts (all contiguous):
 *   query        [batch, num_q_heads, head_dim]                      q_dtype
 *   key_cache    [num_blocks, block_size, num_kv_heads, head_dim]    kv_dtype
 *                ([num_blocks, num_kv_heads, block_size, head_dim] when desc.cache_layout == 1)
 *   value_cache  same shape as key_cache
 *   block_tables [batch, max_blocks_per_seq] int32 (device)
 *   k_descale / v_descale [num_kv_heads * head_dim] float32, k_offset / v_offset int32
 *                (quant_type == 1 only; offsets only when has_quant_offset)
 *   attn_mask    NORM [batch, 1, max_ctx], ALIBI [batch, num_q_heads, 1, max_ctx]
 *   out          [batch, num_q_heads, head_dim]                      q_dtype
 *   workspace    >= msco_paged_attention_workspace_bytes(plan), 256-byte aligned;
 *                holds two status words, the plan words, the kernel's scheduling words (work-item
 *                ticket, one arrival counter per split group) and the split partials.  It needs no
 *                initialisation: errors are tagged with a per-launch epoch and the launch zeroes the
 *                scheduling words itself (a small memset in front of the kernel).
 * Plans of up to 2304 words (about 280 sequences) travel as a kernel parameter; larger ones are
 * copied into the workspace by an async copy from the plan's pinned host memory in front of the
 * kernel: the plan must outlive the launch. */
int msco_paged_attention_launch(const MscoPaPlan *plan, const void *query, const void *key_cache,
                                const void *value_cache, const int32_t *block_tables,
                                const float *k_descale, const int32_t *k_offset,
                                const float *v_descale, const int32_t *v_offset,
                                const void *attn_mask, void *out, void *workspace,
                                size_t workspace_bytes, void *stream);

/* Multi-token (speculative) queries, calc_type = 1 of the operator (q_seq_len of
 * CustomASDPagedAttentionParam, paged_attention_graph.cc:758-762): every query token is a row of the
 * decode batch -- plan with one context length per TOKEN (its sequence's), launch with a block table
 * that has one row per token.  This helper builds that table on the device:
 * dst[i, :] = src[host_row_of[i], :] for i < out_rows (src [src_rows, cols], dst [out_rows, cols], both
 * device int32).  host_row_of is host memory (copied into device_row_of, out_rows device int32s, on
 * `stream`; it may be freed when the call returns).  The SPEC mask [tokens, max_context] is then the
 * NORM decode mask of that batch (mask_type 1, mask_batch_stride = max_context). */
int msco_expand_rows_i32(const int32_t *src, int32_t src_rows, int32_t cols, const int32_t *host_row_of,
                         int32_t out_rows, int32_t *dst, int32_t *device_row_of, void *stream);

/* Extension (the reference operator has no such output): the same launch that also writes
 * lse[batch, num_q_heads] float32 = log(sum over the context of exp(qk_scale * q.k + mask)), natural
 * logarithm, -inf for an empty context.  With it, outputs computed over different parts of a context
 * (sequence-parallel decode) are merged exactly by msco_fa_update. */
int msco_paged_attention_launch_lse(const MscoPaPlan *plan, const void *query, const void *key_cache,
                                    const void *value_cache, const int32_t *block_tables,
                                    const float *k_descale, const int32_t *k_offset, const float *v_descale,
                                    const int32_t *v_offset, const void *attn_mask, void *out, float *lse,
                                    void *workspace, size_t workspace_bytes, void *stream);

/* One decode step in one call: reshape_and_cache of `num_tokens` new rows (key / value:
 * [num_tokens, num_kv_heads * head_dim] in the query dtype; quantised on the way in when the plan's
 * quant_type is 1) followed by the attention launch above on the same caches.  Same result as the
 * two separate calls; the attention kernel is launched with programmatic stream serialisation
 * behind the scatter kernel so that its set-up overlaps the scatter's tail, and the scatter kernel
 * zeroes the attention kernel's scheduling words on its way: two kernel launches per step, the
 * split partials being merged by the attention kernel itself. */
int msco_decode_step(const MscoPaPlan *plan, const void *key, const void *value, void *key_cache,
                     void *value_cache, const int32_t *slot_mapping, int64_t num_tokens, const void *query,
                     const int32_t *block_tables, const float *k_descale, const int32_t *k_offset,
                     const float *v_descale, const int32_t *v_offset, const void *attn_mask, void *out,
                     void *workspace, size_t workspace_bytes, void *stream);

/* After the stream has been synchronised: reads the status word the kernels
 * leave in the workspace.  MSCO_OK, MSCO_ERR_TIMEOUT (a bounded wait inside
 * the kernel expired) or MSCO_ERR_OOB (a block id outside the cache was met;
 * the affected tokens were skipped).  Reads the two words with a synchronous
 * cudaMemcpy (device to host, default stream semantics).  `plan`
 * may be NULL (the status word is the first word of the workspace). */
int msco_paged_attention_status(const MscoPaPlan *plan, const void *workspace);

/* ------------------------------------------------------------------------
 * Launch without any caller-provided scratch memory.
 *
 * Has no counterpart in the reference (there the framework always hands the
 * kernel library a workspace it allocated).  It exists for callers that are
 * not in a position to allocate device memory when they need to launch:
 * code running inside a framework whose allocator they must not re-enter
 * (custom-op callbacks that may only touch the tensors they were given), hosts
 * that pre-allocate everything at start-up and forbid cudaMalloc afterwards
 * (real-time serving loops, where an allocation can stall the whole device),
 * and thin language bindings that have pointers to inputs and outputs but no
 * allocator at all.  Those callers still pass every input and the output; what
 * they cannot supply is the scratch area for the split-KV partials and the
 * uploaded plan.
 *
 * Same arguments and same result as msco_paged_attention_launch, minus
 * `workspace`: the scratch is a fixed MSCO_STATIC_SCRATCH_BYTES array that
 * lives inside the library's device image, so every GPU that loads the library
 * carries it until the process exits.  Plans whose workspace need is larger
 * are rejected with MSCO_ERR_INVALID_ARG and a message stating both sizes (use
 * msco_paged_attention_workspace_bytes(plan) to know beforehand) -- nothing is
 * launched in that case.
 *
 * The first call on each device looks up the device address of the array
 * (one cudaGetSymbolAddress, with that device current); make that first call
 * outside any stream capture.  No call allocates or frees device memory.
 * All calls on one device share the one array and it keeps whatever the last
 * call left there; each launch rewrites everything it later reads (plan words,
 * status word, partials), so nothing needs clearing by the caller -- but two
 * launches that can overlap on the GPU (different streams, or graph branches)
 * would write the same bytes at the same time: serialise them.
 * msco_paged_attention_status_static reads the status word of the last launch
 * on the current device (after synchronising the stream) with a synchronous
 * cudaMemcpy of two words out of the array.  The array's address is cached per
 * device ordinal of the calling process's primary context: a process that
 * drives one device through several CUDA contexts must use this entry point
 * from one of them only.
 * ---------------------------------------------------------------------- */
#define MSCO_STATIC_SCRATCH_BYTES (16u << 20)
int msco_paged_attention_launch_static(const MscoPaPlan *plan, const void *query, const void *key_cache,
                                       const void *value_cache, const int32_t *block_tables,
                                       const float *k_descale, const int32_t *k_offset,
                                       const float *v_descale, const int32_t *v_offset,
                                       const void *attn_mask, void *out, void *stream);
int msco_paged_attention_status_static(const MscoPaPlan *plan);

/* ------------------------------------------------------------------------
 * All-gather of per-rank outputs over NVLink peer memory (kv-head sharding).
 *
 * The reference has no multi-device code on this path; with the cache split by
 * kv head the one exchange of a step is the all-gather of each rank's
 * [batch, q_heads / N, head_dim] output.  msco_peer_allgather launches one small
 * kernel that stores the local slice into slot `rank` of every rank's gathered
 * buffer (plain peer stores), publishes `step` in every rank's flag array and
 * waits -- bounded -- until all ranks have published `step` here.  When it has
 * completed, gathered[rank] holds all slices: [world][slice_bytes].
 *
 * Set-up (once): every rank allocates its gathered buffer (world * slice_bytes)
 * and a zeroed uint32[world] flag array, exports both with msco_ipc_export,
 * exchanges the 64-byte handles and offsets with its peers by any host channel
 * and maps theirs with msco_ipc_import.  `ticket` (zeroed uint32) and `status`
 * (zeroed int32; set to MSCO_ERR_TIMEOUT if a peer never arrives) are local
 * device words.  Call with step = 1, 2, 3, ... ; alternate between two gathered
 * buffers from step to step if a consumer may still read the previous one.
 * ---------------------------------------------------------------------- */
#define MSCO_MAX_PEERS 8
#define MSCO_IPC_HANDLE_BYTES 64
typedef struct MscoGatherDesc {
  int32_t world, rank;
  void *gathered[MSCO_MAX_PEERS];     /* gathered[r]: rank r's buffer as mapped in this process   */
  uint32_t *flags[MSCO_MAX_PEERS];    /* flags[r]: rank r's uint32[world] as mapped in this process */
  int64_t slice_bytes;                /* bytes of one rank's slice; multiple of 16                 */
  unsigned int *ticket;               /* local device word, zero before the first call            */
  int32_t *status;                    /* local device word, zero before the first call            */
  uint32_t wait_polls;                /* polls (about 0.1 us apart) before the wait for a peer gives up and
                                         sets *status = MSCO_ERR_TIMEOUT; 0 = the default, 2^22 (about half a second) */
  uint32_t reserved;
  void *packets[MSCO_MAX_PEERS];      /* optional (all NULL: not used).  packets[r]: rank r's packet buffer as
                                         mapped in this process, 2 * world * slice_bytes bytes, zero before the first
                                         step.  With it msco_decode_step_gather exchanges the rows as 8-byte packets
                                         {4 data bytes, step}: the receiver sees a packet's data when it sees its step,
                                         so the exchange needs no fence, no flag and no last block -- one NVLink
                                         crossing instead of three; every thread copies the packets it waits for into
                                         its own plain gathered buffer.  flags[] are not used then. */
} MscoGatherDesc;
int msco_ipc_export(const void *dev_ptr, unsigned char *handle /* [64] */, int64_t *offset);
int msco_ipc_import(const unsigned char *handle, int64_t offset, void **dev_ptr);
int msco_ipc_release(void *dev_ptr, int64_t offset);
int msco_peer_allgather(const MscoGatherDesc *desc, const void *local_out, uint32_t step, void *stream);

/* msco_decode_step for one rank of a kv-head-sharded step, with the exchange folded in: the kernel that
 * finishes the output rows (the split merge; rows that need no merge are read back from `out`) also
 * stores every row into slot `rank` of every rank's gathered buffer, and its last block publishes `step`
 * and waits -- bounded, as above -- for the peers.  Same descriptor, flag protocol, `step` sequence and
 * status word as msco_peer_allgather, which it replaces for the step (one launch and one read-back of
 * the slice fewer); `out` still receives the local slice.  gather->slice_bytes must equal the size of
 * the plan's output (query rows x q heads x head_dim x 2).  No reference counterpart. */
int msco_decode_step_gather(const MscoPaPlan *plan, const void *key, const void *value, void *key_cache,
                            void *value_cache, const int32_t *slot_mapping, int64_t num_tokens,
                            const void *query, const int32_t *block_tables, const float *k_descale,
                            const int32_t *k_offset, const float *v_descale, const int32_t *v_offset,
                            const void *attn_mask, void *out, void *workspace, size_t workspace_bytes,
                            void *stream, const MscoGatherDesc *gather, uint32_t step);

/* Kernel timing for benchmarks.  After msco_paged_attention_profile_enable(plan, 1) every launch
 * of this plan records a pair of CUDA events directly around the attention kernel (not around the
 * plan upload or the reduce kernel) into a ring of 64 pairs owned by the plan.
 * msco_paged_attention_profile_read synchronises on the recorded pairs and returns the kernel
 * durations of the most recent launches, oldest first (at most `max_count`, at most 64), then
 * clears the ring.  Off by default; enabling it makes the plan unsuitable for stream capture. */
int msco_paged_attention_profile_enable(MscoPaPlan *plan, int32_t enable);
int msco_paged_attention_profile_read(MscoPaPlan *plan, float *kernel_ms, int32_t max_count, int32_t *count);

#ifdef __cplusplus
}
#endif
#endif /* MSCO_B200_H_ */
