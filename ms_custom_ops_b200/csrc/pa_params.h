// Kernel parameter block and host-side plan object of paged attention.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <mutex>
#include <vector>

#include "msco_b200.h"

namespace msco {

// Passed by value to every paged-attention kernel.
struct PaParams {
  const void *q;
  const void *key_cache;
  const void *value_cache;
  const int32_t *block_tables;
  const float *k_descale;
  const int32_t *k_offset;
  const float *v_descale;
  const int32_t *v_offset;
  const void *mask;
  void *out;
  float *lse;           // optional [batch, num_q_heads]: natural-log sum of exp of the scaled (+mask) scores
  const int32_t *plan;  // device copy of the plan words (unused when the words travel as a kernel parameter)
  int32_t *status;      // workspace words 0..1: [error code, launch epoch]
  uint32_t epoch;       // identifies this launch in the status words
  int32_t plan_in_param;  // the plan words are in the PlanParam kernel argument
  float *part_o;   // [total_parts, num_q_heads, head_dim] un-normalised partial outputs
  float *part_ml;  // [total_parts, num_q_heads, 2] (running max in log2 domain, running sum)
  // Scheduling words of the persistent kernel, zero when the kernel starts: sync[0] is the work-item
  // ticket, sync[kSyncHeaderWords + g] counts the splits of group g (sequence, kv head, q-row block)
  // that have stored their partial; the CTA that brings it to the split count merges the group.
  uint32_t *sync;
  int32_t fused_merge;  // the attention kernel merges the split partials itself (no reduce kernel)
  int64_t num_blocks;
  int64_t mask_batch_stride, mask_head_stride;
  int num_q_heads, num_kv_heads, head_dim, block_size, group, rows_per_item, max_blocks_per_seq;
  int mask_type, mask_dtype;
  int cache_layout;   // 0: [blocks, block_size, kv_heads, head_dim]; 1: [blocks, kv_heads, block_size, head_dim]
  float scale;        // qk_scale
  float scale_log2e;  // qk_scale * log2(e)
};

// Plans of up to kPlanParamWords words travel as a kernel parameter (no upload, no stream
// operation in front of the attention kernel); larger ones are copied into the workspace.
// Two parameter sizes: a launch with 9 KB of parameters starts about a microsecond later than one with
// 2.5 KB, so plans of up to kPlanParamWordsSmall words (about 70 sequences) use the small form.
constexpr int kPlanParamWords = 2304;
constexpr int kPlanParamWordsSmall = 640;
template <int W>
struct PlanParamT {
  int32_t w[W];
};
using PlanParam = PlanParamT<kPlanParamWords>;
using PlanParamSmall = PlanParamT<kPlanParamWordsSmall>;  // a prefix of PlanParam
constexpr size_t kPlanRegionOffset = 256;  // workspace: [status block | plan words | scheduling words | partials]
constexpr int kSyncHeaderWords = 4;        // scheduling words: [ticket, 3 unused, one counter per group]

constexpr int kKernelGeneric = 1;
constexpr int kKernelTma = 2;

}  // namespace msco

struct MscoPaPlan {
  MscoPaDesc desc;
  int batch = 0;
  int kernel = 0;
  int rows_per_item = 8;
  int grid = 0;
  int num_sms = 148;
  int nseq = 0, total_items = 0, total_parts = 0, max_splits = 0;
  bool need_reduce = false;
  int64_t kv_tokens = 0;
  // plan words: a block of the pooled pinned arena (plan_arena.h), kept across re-plans
  int32_t *host_words = nullptr;
  size_t host_capacity = 0;     // bytes of that block
  size_t plan_words = 0;
  size_t plan_bytes = 0;        // bytes uploaded per launch
  // an async copy of host_words (plans too large for the kernel parameters) may still be queued
  // when the plan is rewritten: the event is recorded behind the copy and waited for before a re-plan
  mutable cudaEvent_t upload_done = nullptr;
  mutable bool upload_pending = false;
  bool fused_merge = false;     // the attention kernel merges the split partials itself
  bool fused_merge_wanted = false;
  bool multi_token = false;     // planned from (context_lens, q_seq_lens): `batch` counts query tokens
  int num_groups = 0;           // (sequence with tokens, kv head, q-row block) triples
  size_t sync_offset = 0;       // scheduling words inside the workspace
  size_t sync_bytes = 0;
  size_t part_o_offset = 0;     // byte offsets inside the workspace
  size_t part_ml_offset = 0;
  size_t workspace_bytes = 0;
  // tensor maps of the TMA kernel, rebuilt when the cache addresses change
  mutable std::mutex tm_mutex;
  mutable const void *tm_k_ptr = nullptr;
  mutable const void *tm_v_ptr = nullptr;
  alignas(64) mutable unsigned char tm_k[128];
  alignas(64) mutable unsigned char tm_v[128];
  mutable uint32_t last_epoch = 0;  // epoch of the most recent launch (status check)
  // optional kernel timing (benchmarks): ring of event pairs recorded around the attention kernel
  static constexpr int kProfRing = 64;
  bool profile = false;
  mutable cudaEvent_t prof_ev[kProfRing][2] = {};
  mutable int64_t prof_count = 0;
};

namespace msco {
// kernel launchers (defined next to the kernels)
// `pp`: the plan words as a kernel parameter (meaningful when p.plan_in_param); `after_kernel`:
// the previous operation on the stream is a kernel of this library that triggers its dependents
// early, so the launch may use programmatic stream serialisation.
int launch_pa_generic(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, cudaStream_t stream);
int launch_pa_tma(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, cudaStream_t stream,
                  bool after_kernel);
struct GatherArgs;  // peer_gather.cuh
// `gather` != NULL: the kernel also pushes every finished row to the peers of a kv-head-sharded step
int launch_pa_reduce(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, cudaStream_t stream,
                     const GatherArgs *gather = nullptr);
// reshape_and_cache launchers that can also zero `clear_words` 32-bit words at `clear` (the attention
// kernel's scheduling words) on their way; *cleared tells whether the launched kernel does it
int launch_rac(const void *key, const void *value, void *key_cache, void *value_cache, const int32_t *slot_mapping,
               int64_t num_tokens, int64_t k_row_bytes, int64_t v_row_bytes, int64_t num_slots, int32_t *oob_count,
               cudaStream_t stream, uint32_t *clear, int clear_words, bool *cleared);
int launch_rac_quant(const void *key, const void *value, int8_t *key_cache, int8_t *value_cache,
                     const int32_t *slot_mapping, int64_t num_tokens, int64_t k_row_elems, int64_t v_row_elems,
                     int32_t in_dtype, const float *k_descale, const int32_t *k_offset, const float *v_descale,
                     const int32_t *v_offset, int64_t num_slots, int32_t *oob_count, cudaStream_t stream,
                     uint32_t *clear, int clear_words, bool *cleared);
bool pa_tma_supported(const MscoPaDesc &d);
int pa_tma_rows_per_item(const MscoPaDesc &d);
}  // namespace msco
