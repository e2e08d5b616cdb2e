// C ABI of libmsco_b200.so: error reporting, paged-attention planning and launch.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <numeric>

#include "msco_common.cuh"
#include "pa_params.h"
#include "peer_gather.cuh"
#include "plan_arena.h"

namespace msco {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace msco

using namespace msco;

extern "C" int msco_version(void) { return MSCO_ABI_VERSION; }
extern "C" const char *msco_last_error(void) { return g_err; }

// Tokens per KV split.  A function of the sequence's own length (and of the
// cache element type, fixed per call) only: the result for one request never
// depends on what else is in the batch.  A split is sized to about 256 KB of
// K/V per kv head at the short end, so that the per-split merge is amortised.
static int32_t split_tokens(int32_t context_len, int32_t token_bytes) {
  if (context_len > 65536) return 2048;
  // token rows of 128 bytes (int8 at head_dim 128, 16-bit at head_dim 64) are half the bytes, and the
  // per-item cost of those kernel variants is the larger one: contexts of up to 4096 tokens are one item,
  // longer ones are cut every 2048 tokens
  if (token_bytes <= 128) return context_len <= 4096 ? 4096 : 2048;
  if (context_len > 16384) return 1024;
  return 512;
}
extern "C" int32_t msco_paged_attention_split_tokens(int32_t context_len, int32_t kv_dtype) {
  return split_tokens(context_len, kv_dtype == MSCO_DTYPE_I8 ? 128 : 256);
}
extern "C" int32_t msco_paged_attention_split_tokens_for(int32_t context_len, int32_t kv_dtype, int32_t head_dim) {
  return split_tokens(context_len, head_dim * (kv_dtype == MSCO_DTYPE_I8 ? 1 : 2));
}

static int validate_desc(const MscoPaDesc &d) {
  if (d.q_dtype != MSCO_DTYPE_F16 && d.q_dtype != MSCO_DTYPE_BF16)
    return fail(MSCO_ERR_UNSUPPORTED, "paged_attention: query dtype must be float16/bfloat16 (full-quant int8 query is not built)");
  if (d.quant_type == 0) {
    if (d.kv_dtype != d.q_dtype)
      return fail(MSCO_ERR_INVALID_ARG, "paged_attention: in unquant mode the cache dtype must equal the query dtype");
  } else if (d.quant_type == 1) {
    if (d.kv_dtype != MSCO_DTYPE_I8)
      return fail(MSCO_ERR_INVALID_ARG, "paged_attention: in dequant mode the cache dtype must be int8");
  } else {
    return fail(MSCO_ERR_UNSUPPORTED, "paged_attention: quant_type %d is not built (0 and 1 are)", d.quant_type);
  }
  if (d.num_q_heads <= 0 || d.num_kv_heads <= 0 || d.num_q_heads % d.num_kv_heads != 0)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: q heads (%d) must be a positive multiple of kv heads (%d)",
                d.num_q_heads, d.num_kv_heads);
  if (d.head_dim <= 0 || d.head_dim > 256)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: head_dim must be in (0, 256], got %d", d.head_dim);
  if (d.block_size <= 0 || d.num_blocks <= 0 || d.max_blocks_per_seq < 0)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: bad cache geometry");
  if (d.cache_layout != 0 && d.cache_layout != 1)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: cache_layout must be 0 (block_size major) or 1 (head major)");
  if (d.cache_layout == 1 && d.quant_type != 0)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: the head-major cache layout takes no quantised cache "
                                      "(the reference requires quant_type 0 with input_layout 1)");
  if (d.mask_type < 0 || d.mask_type > 2)
    return fail(MSCO_ERR_UNSUPPORTED, "paged_attention: mask_type %d is not built (0, 1, 2 are)", d.mask_type);
  if (d.mask_type != 0 && d.mask_dtype != MSCO_DTYPE_F16 && d.mask_dtype != MSCO_DTYPE_BF16 &&
      d.mask_dtype != MSCO_DTYPE_F32)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: mask dtype must be float16/bfloat16/float32");
  return MSCO_OK;
}

namespace {

// SM count of the current device, looked up once per device ordinal (148 when there is none).
int current_sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();  // no device (planning only): keep the B200 default
    return 148;
  }
  if (dev >= 0 && dev < 64) {
    const int c = cached[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
    (void)cudaGetLastError();
    return 148;
  }
  if (dev >= 0 && dev < 64) cached[dev].store(sms, std::memory_order_relaxed);
  return sms;
}

// Fills `pl` (descriptor already set) for one vector of context lengths.  The plan words live in a
// block of the pinned arena that the plan keeps across calls: a re-plan with a batch of the same size
// class touches no allocator at all.
// `q_lens` (NULL for a decode batch: one query token per sequence) gives the number of query tokens of
// every sequence (multi-token / speculative queries); `num` is the number of sequences.  Runs of up to
// rows / group consecutive tokens of a sequence become one plan entry whose q rows are stacked into one
// work item, so the context is read once for all of them.
int fill_plan(MscoPaPlan *pl, const int32_t *host_context_lens, const int32_t *q_lens, int32_t num) {
  const MscoPaDesc &d = pl->desc;
  const int64_t cap = (int64_t)d.max_blocks_per_seq * d.block_size;
  int64_t tokens = 0;
  int max_q = 1;
  for (int b = 0; b < num; ++b) {
    if (host_context_lens[b] < 0)
      return fail(MSCO_ERR_INVALID_ARG, "paged_attention_plan: context_lens[%d] = %d is negative", b,
                  host_context_lens[b]);
    if (host_context_lens[b] > cap)
      return fail(MSCO_ERR_INVALID_ARG,
                  "paged_attention_plan: context_lens[%d] = %d exceeds the block table (%d blocks of %d)", b,
                  host_context_lens[b], d.max_blocks_per_seq, d.block_size);
    if (q_lens != nullptr) {
      if (q_lens[b] < 0) return fail(MSCO_ERR_INVALID_ARG, "paged_attention_plan: q_seq_lens[%d] = %d is negative", b, q_lens[b]);
      tokens += q_lens[b];
      max_q = std::max(max_q, q_lens[b]);
    }
  }
  if (tokens > 0x7fffffffLL) return fail(MSCO_ERR_INVALID_ARG, "paged_attention_plan: too many query tokens");
  const bool mt = q_lens != nullptr;
  const int batch = mt ? (int)tokens : num;  // rows of query / out
  pl->batch = batch;
  pl->multi_token = mt;
  const int g = d.num_q_heads / d.num_kv_heads;
  // query tokens stacked into one item: as many as the item's q rows hold
  int tpi = 1;
  pl->rows_per_item = pl->kernel == kKernelTma ? pa_tma_rows_per_item(d) : 8;
  if (mt && pl->kernel == kKernelTma) {
    const int rows_max = d.head_dim == 256 ? 8 : 16;
    tpi = std::max(1, std::min(max_q, rows_max / g));
    if (tpi > 1) pl->rows_per_item = tpi * g > 8 ? 16 : 8;
  }
  const int nqb = (g + pl->rows_per_item - 1) / pl->rows_per_item;
  const int items_per_split = d.num_kv_heads * nqb;
  pl->num_sms = current_sm_count();

  // entries with work, longest first (stable), so that the big items lead the work list
  struct Entry { int b, len, qtok0, ntok; };
  static thread_local std::vector<Entry> entries;
  entries.clear();
  int qbase = 0, empty_rows = 0;
  for (int b = 0; b < num; ++b) {
    const int ql = mt ? q_lens[b] : 1;
    if (host_context_lens[b] > 0) {
      for (int t0 = 0; t0 < ql; t0 += tpi) entries.push_back({b, host_context_lens[b], mt ? qbase + t0 : b, std::min(tpi, ql - t0)});
    } else {
      empty_rows += ql;
    }
    qbase += ql;
  }
  std::stable_sort(entries.begin(), entries.end(), [](const Entry &a, const Entry &b) { return a.len > b.len; });
  const int nseq = (int)entries.size();
  pl->nseq = nseq;
  pl->plan_words = kPlanHeaderWords + (size_t)(nseq + 1) + 5 * (size_t)nseq + 2 * (size_t)batch + (mt ? 2 * (size_t)nseq : 0);
  pl->plan_bytes = pl->plan_words * 4;
  if (pl->upload_pending) {  // an async copy out of the old words may still be queued
    MSCO_CUDA_CHECK(cudaEventSynchronize(pl->upload_done));
    pl->upload_pending = false;
  }
  if (pl->host_words == nullptr || pl->host_capacity < pl->plan_bytes) {
    if (pl->host_words != nullptr) PlanArena::Instance().Free(pl->host_words, pl->host_capacity);
    pl->host_capacity = 0;
    pl->host_words = static_cast<int32_t *>(PlanArena::Instance().Alloc(pl->plan_bytes, &pl->host_capacity));
    if (pl->host_words == nullptr) return fail(MSCO_ERR_INTERNAL, "paged_attention_plan: out of host memory");
  }
  int32_t *w = pl->host_words;
  memset(w, 0, pl->plan_bytes);
  int32_t *item_base = w + kPlanHeaderWords;
  int32_t *seq_idx = item_base + nseq + 1, *seq_len = seq_idx + nseq, *chunk = seq_len + nseq;
  int32_t *nsplit = chunk + nseq, *part_base = nsplit + nseq;
  int32_t *b_nsplit = part_base + nseq, *b_part_base = b_nsplit + batch;
  int32_t *qtok0 = b_part_base + batch, *qntok = qtok0 + nseq;
  int64_t items = 0, parts = 0, kv_tokens = 0;
  int max_splits = 0;
  const bool fused = pl->kernel == kKernelTma && pl->fused_merge_wanted;
  for (int s = 0; s < nseq; ++s) {
    const Entry &e = entries[s];
    const int c = msco_paged_attention_split_tokens_for(e.len, d.kv_dtype, d.head_dim);
    const int ns = (e.len + c - 1) / c;
    item_base[s] = (int32_t)items;
    seq_idx[s] = e.b; seq_len[s] = e.len; chunk[s] = c; nsplit[s] = ns;
    part_base[s] = (int32_t)parts;
    if (mt) { qtok0[s] = e.qtok0; qntok[s] = e.ntok; }
    // per output row (the reduce kernel's view): splits and first partial.  When the attention kernel
    // merges its partials itself the reduce kernel only zero-fills the rows of empty sequences, so every
    // other row is marked as written.
    // (partials of a run of stacked tokens are token-major: token t, split s -> parts + t * ns + s)
    for (int t = 0; t < e.ntok; ++t) {
      b_nsplit[e.qtok0 + t] = fused ? 1 : ns;
      b_part_base[e.qtok0 + t] = (int32_t)(parts + (int64_t)t * ns);
    }
    items += (int64_t)ns * items_per_split;
    if (ns > 1) parts += (int64_t)ns * e.ntok;
    max_splits = std::max(max_splits, ns);
    kv_tokens += e.len;
    if (items > 0x7fffffffLL || parts > 0x7fffffffLL)
      return fail(MSCO_ERR_INVALID_ARG, "paged_attention_plan: too many work items");
  }
  item_base[nseq] = (int32_t)items;
  w[0] = 0; w[1] = nseq; w[2] = (int32_t)items; w[3] = (int32_t)parts; w[4] = batch; w[5] = items_per_split;
  w[6] = mt ? 1 : 0;
  pl->total_items = (int)items;
  pl->total_parts = (int)parts;
  pl->max_splits = max_splits;
  pl->kv_tokens = kv_tokens;
  // the TMA kernel merges its split partials itself (the CTA that stores the last partial of a group
  // does it); the reduce kernel is then only needed to zero the rows of empty sequences
  pl->fused_merge = fused;
  const bool has_empty = mt ? empty_rows > 0 : nseq < batch;
  pl->need_reduce = pl->fused_merge ? has_empty : (parts > 0 || has_empty);
  pl->grid = pl->kernel == kKernelTma ? (int)std::min<int64_t>(items, pl->num_sms) : (int)items;
  pl->num_groups = pl->fused_merge ? nseq * items_per_split : 0;
  pl->sync_offset = align_up(kPlanRegionOffset + pl->plan_bytes, 256);
  // the TMA kernel always takes its work items by the ticket in the first scheduling word
  pl->sync_bytes = pl->kernel == kKernelTma ? align_up((size_t)(kSyncHeaderWords + pl->num_groups) * 4, 256) : 0;
  pl->part_o_offset = pl->sync_offset + pl->sync_bytes;
  const size_t part_o_bytes = (size_t)parts * d.num_q_heads * d.head_dim * 4;
  pl->part_ml_offset = align_up(pl->part_o_offset + part_o_bytes, 256);
  pl->workspace_bytes = align_up(pl->part_ml_offset + (size_t)parts * d.num_q_heads * 2 * 4, 256);
  return MSCO_OK;
}

int new_plan(const MscoPaDesc *desc, const int32_t *lens, const int32_t *q_lens, int32_t num, MscoPaPlan **out_plan) {
  if (desc == nullptr || out_plan == nullptr || num < 0 || (num > 0 && lens == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_plan: NULL argument");
  *out_plan = nullptr;
  int rc = validate_desc(*desc);
  if (rc != MSCO_OK) return rc;
  const MscoPaDesc &d = *desc;
  const bool tma_ok = pa_tma_supported(d);
  if (d.kernel == kKernelTma && !tma_ok)
    return fail(MSCO_ERR_UNSUPPORTED,
                "paged_attention_plan: the TMA kernel needs head_dim 128 (or 64 / 256 with a 16-bit cache) and "
                "block_size 16/32/64/128 (at most 64 for head_dim 256)");
  const int kernel = (d.kernel == kKernelGeneric || !tma_ok) ? kKernelGeneric : kKernelTma;
  if (q_lens != nullptr && kernel != kKernelTma)
    return fail(MSCO_ERR_UNSUPPORTED,
                "paged_attention_plan_tokens: stacked query tokens need the TMA kernel; for this shape plan one decode "
                "row per query token instead (msco_paged_attention_plan + msco_expand_rows_i32)");
  MscoPaPlan *pl = new (std::nothrow) MscoPaPlan();
  if (pl == nullptr) return fail(MSCO_ERR_INTERNAL, "paged_attention_plan: out of host memory");
  pl->desc = d;
  pl->kernel = kernel;
  // MSCO_PA_FUSED_MERGE=1: the attention kernel merges its split partials itself (the CTA that stores a
  // group's last partial does it) instead of leaving them to the reduce kernel: one launch less per step,
  // paid for with a device-scope fence and an atomic per multi-split item
  if (const char *e = getenv("MSCO_PA_FUSED_MERGE")) pl->fused_merge_wanted = atoi(e) != 0;
  rc = fill_plan(pl, lens, q_lens, num);
  if (rc != MSCO_OK) {
    msco_paged_attention_plan_destroy(pl);
    return rc;
  }
  *out_plan = pl;
  return MSCO_OK;
}

}  // namespace

extern "C" int32_t msco_paged_attention_tma_supported(const MscoPaDesc *desc) {
  return (desc != nullptr && validate_desc(*desc) == MSCO_OK && desc->kernel != kKernelGeneric &&
          pa_tma_supported(*desc)) ? 1 : 0;
}

extern "C" int msco_paged_attention_plan(const MscoPaDesc *desc, const int32_t *host_context_lens,
                                         int32_t batch, MscoPaPlan **out_plan) {
  return new_plan(desc, host_context_lens, nullptr, batch, out_plan);
}

extern "C" int msco_paged_attention_plan_tokens(const MscoPaDesc *desc, const int32_t *host_context_lens,
                                                const int32_t *host_q_seq_lens, int32_t num_seqs,
                                                MscoPaPlan **out_plan) {
  if (num_seqs > 0 && host_q_seq_lens == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_plan_tokens: NULL q_seq_lens");
  static const int32_t none = 0;
  return new_plan(desc, host_context_lens, host_q_seq_lens != nullptr ? host_q_seq_lens : &none, num_seqs, out_plan);
}

extern "C" int msco_paged_attention_replan(MscoPaPlan *plan, const int32_t *host_context_lens, int32_t batch) {
  if (plan == nullptr || batch < 0 || (batch > 0 && host_context_lens == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_replan: NULL argument");
  return fill_plan(plan, host_context_lens, nullptr, batch);
}

extern "C" int msco_paged_attention_replan_tokens(MscoPaPlan *plan, const int32_t *host_context_lens,
                                                  const int32_t *host_q_seq_lens, int32_t num_seqs) {
  if (plan == nullptr || num_seqs < 0 || (num_seqs > 0 && (host_context_lens == nullptr || host_q_seq_lens == nullptr)))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_replan_tokens: NULL argument");
  if (plan->kernel != kKernelTma)
    return fail(MSCO_ERR_UNSUPPORTED, "paged_attention_replan_tokens: stacked query tokens need the TMA kernel");
  static const int32_t none = 0;
  return fill_plan(plan, host_context_lens, num_seqs > 0 ? host_q_seq_lens : &none, num_seqs);
}

extern "C" void msco_plan_arena_stats(int64_t *stats /* [6] */) {
  if (stats == nullptr) return;
  PlanArenaStats st;
  PlanArena::Instance().Stats(&st);
  stats[0] = st.slabs; stats[1] = st.slab_bytes; stats[2] = st.blocks_in_use;
  stats[3] = st.block_allocs; stats[4] = st.oversize_allocs; stats[5] = st.pinned;
}

extern "C" size_t msco_paged_attention_workspace_bytes(const MscoPaPlan *plan) {
  return plan ? plan->workspace_bytes : 0;
}

extern "C" int msco_paged_attention_plan_info(const MscoPaPlan *plan, MscoPaPlanInfo *info) {
  if (plan == nullptr || info == nullptr) return fail(MSCO_ERR_INVALID_ARG, "plan_info: NULL argument");
  info->kernel = plan->kernel;
  info->grid = plan->grid;
  info->work_items = plan->total_items;
  info->partials = plan->total_parts;
  info->max_splits = plan->max_splits;
  info->rows_per_item = plan->rows_per_item;
  info->workspace_bytes = (int64_t)plan->workspace_bytes;
  info->kv_tokens = plan->kv_tokens;
  return MSCO_OK;
}

extern "C" int msco_paged_attention_profile_enable(MscoPaPlan *plan, int32_t enable) {
  if (plan == nullptr) return fail(MSCO_ERR_INVALID_ARG, "profile_enable: NULL plan");
  if (enable && plan->prof_ev[0][0] == nullptr) {
    for (int i = 0; i < MscoPaPlan::kProfRing; ++i)
      for (int j = 0; j < 2; ++j) MSCO_CUDA_CHECK(cudaEventCreate(&plan->prof_ev[i][j]));
  }
  plan->profile = enable != 0;
  plan->prof_count = 0;
  return MSCO_OK;
}

extern "C" int msco_paged_attention_profile_read(MscoPaPlan *plan, float *kernel_ms, int32_t max_count,
                                                 int32_t *count) {
  if (plan == nullptr || kernel_ms == nullptr || count == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "profile_read: NULL argument");
  const int64_t have = std::min<int64_t>(plan->prof_count, MscoPaPlan::kProfRing);
  const int64_t n = std::min<int64_t>(have, max_count);
  for (int64_t i = 0; i < n; ++i) {
    const int64_t idx = (plan->prof_count - n + i) % MscoPaPlan::kProfRing;
    MSCO_CUDA_CHECK(cudaEventSynchronize(plan->prof_ev[idx][1]));
    MSCO_CUDA_CHECK(cudaEventElapsedTime(&kernel_ms[i], plan->prof_ev[idx][0], plan->prof_ev[idx][1]));
  }
  *count = (int32_t)n;
  plan->prof_count = 0;
  return MSCO_OK;
}

extern "C" void msco_paged_attention_plan_destroy(MscoPaPlan *plan) {
  if (plan == nullptr) return;
  if (plan->prof_ev[0][0] != nullptr)
    for (int i = 0; i < MscoPaPlan::kProfRing; ++i)
      for (int j = 0; j < 2; ++j) cudaEventDestroy(plan->prof_ev[i][j]);
  if (plan->upload_done != nullptr) {
    if (plan->upload_pending) cudaEventSynchronize(plan->upload_done);
    cudaEventDestroy(plan->upload_done);
  }
  if (plan->host_words != nullptr) PlanArena::Instance().Free(plan->host_words, plan->host_capacity);
  delete plan;
}

namespace {

// Launch epochs: every launch gets a fresh 32-bit tag; a kernel that reports an error writes the
// tag next to the code, so stale words in a reused workspace are never mistaken for a new error
// and nothing has to be cleared in front of a launch.
std::atomic<uint32_t> g_epoch{(uint32_t)std::chrono::steady_clock::now().time_since_epoch().count() | 1u};

// (workspace, epoch) of recent launches, for status queries that come without the plan
std::mutex g_recent_mu;
struct Recent { const void *ws; uint32_t epoch; };
Recent g_recent[64] = {};
unsigned g_recent_next = 0;

void remember_launch(const void *ws, uint32_t epoch) {
  std::lock_guard<std::mutex> g(g_recent_mu);
  for (auto &r : g_recent)
    if (r.ws == ws) { r.epoch = epoch; return; }
  g_recent[g_recent_next++ % 64] = {ws, epoch};
}
bool recall_launch(const void *ws, uint32_t *epoch) {
  std::lock_guard<std::mutex> g(g_recent_mu);
  for (auto &r : g_recent)
    if (r.ws == ws) { *epoch = r.epoch; return true; }
  return false;
}

int pa_launch_impl(const MscoPaPlan *plan, const void *query, const void *key_cache, const void *value_cache,
                   const int32_t *block_tables, const float *k_descale, const int32_t *k_offset,
                   const float *v_descale, const int32_t *v_offset, const void *attn_mask, void *out,
                   void *workspace, size_t workspace_bytes, void *stream, bool after_kernel, float *lse = nullptr,
                   bool sync_cleared = false, const GatherArgs *gather = nullptr) {
  if (plan == nullptr) return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: NULL plan");
  if (plan->batch == 0) return MSCO_OK;
  const MscoPaDesc &d = plan->desc;
  if (query == nullptr || key_cache == nullptr || value_cache == nullptr || block_tables == nullptr ||
      out == nullptr || workspace == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: NULL tensor");
  if (workspace_bytes < plan->workspace_bytes)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: workspace too small (%zu < %zu)", workspace_bytes,
                plan->workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: workspace must be 256-byte aligned");
  if (d.quant_type == 1 && (k_descale == nullptr || v_descale == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: k_descale / v_descale are required when quant_type = 1");
  if (d.quant_type == 1 && d.has_quant_offset && (k_offset == nullptr || v_offset == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: k_offset / v_offset are required when has_quant_offset");
  if (d.mask_type != 0 && attn_mask == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch: attn_mask is required when mask_type != 0");
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  PaParams p;
  memset(&p, 0, sizeof(p));
  p.q = query; p.key_cache = key_cache; p.value_cache = value_cache; p.block_tables = block_tables;
  if (d.quant_type == 1) {
    p.k_descale = k_descale; p.v_descale = v_descale;
    if (d.has_quant_offset) { p.k_offset = k_offset; p.v_offset = v_offset; }
  }
  p.mask = d.mask_type ? attn_mask : nullptr;
  p.out = out;
  p.lse = lse;
  char *ws = static_cast<char *>(workspace);
  p.status = reinterpret_cast<int32_t *>(ws);
  p.plan = reinterpret_cast<const int32_t *>(ws + kPlanRegionOffset);
  p.sync = reinterpret_cast<uint32_t *>(ws + plan->sync_offset);
  p.fused_merge = plan->fused_merge ? 1 : 0;
  p.part_o = reinterpret_cast<float *>(ws + plan->part_o_offset);
  p.part_ml = reinterpret_cast<float *>(ws + plan->part_ml_offset);
  p.num_blocks = d.num_blocks;
  p.mask_batch_stride = d.mask_batch_stride; p.mask_head_stride = d.mask_head_stride;
  p.num_q_heads = d.num_q_heads; p.num_kv_heads = d.num_kv_heads; p.head_dim = d.head_dim;
  p.block_size = d.block_size; p.group = d.num_q_heads / d.num_kv_heads;
  p.rows_per_item = plan->rows_per_item; p.max_blocks_per_seq = d.max_blocks_per_seq;
  p.mask_type = d.mask_type; p.mask_dtype = d.mask_dtype;
  p.cache_layout = d.cache_layout;
  p.scale = d.qk_scale;
  p.scale_log2e = d.qk_scale * 1.4426950408889634f;
  p.epoch = g_epoch.fetch_add(2u);
  plan->last_epoch = p.epoch;
  remember_launch(workspace, p.epoch);

  // small plans ride in the kernel parameters; larger ones are uploaded in front of the kernel
  static thread_local PlanParam pp;
  p.plan_in_param = plan->plan_words <= (size_t)kPlanParamWords ? 1 : 0;
  if (p.plan_in_param) {
    memcpy(pp.w, plan->host_words, plan->plan_bytes);
  } else {
    MSCO_CUDA_CHECK(cudaMemcpyAsync(ws + kPlanRegionOffset, plan->host_words, plan->plan_bytes,
                                    cudaMemcpyHostToDevice, st));
    // a re-plan rewrites host_words: it waits for this event first
    if (plan->upload_done == nullptr)
      MSCO_CUDA_CHECK(cudaEventCreateWithFlags(&plan->upload_done, cudaEventDisableTiming));
    MSCO_CUDA_CHECK(cudaEventRecord(plan->upload_done, st));
    plan->upload_pending = true;
    after_kernel = false;  // a copy now sits between the previous kernel and ours
  }
  // the scheduling words (work-item ticket, per-group arrival counters) start at zero: either the
  // kernel in front of us cleared them on its way (fused decode step) or a small memset does
  if (plan->sync_bytes != 0 && plan->total_items > 0 && !sync_cleared) {
    MSCO_CUDA_CHECK(cudaMemsetAsync(ws + plan->sync_offset, 0, plan->sync_bytes, st));
    after_kernel = false;
  }
  cudaEvent_t *pe = nullptr;
  if (plan->profile && plan->total_items > 0) {
    pe = plan->prof_ev[plan->prof_count % MscoPaPlan::kProfRing];
    MSCO_CUDA_CHECK(cudaEventRecord(pe[0], st));
    after_kernel = false;
  }
  int rc = plan->kernel == kKernelTma ? launch_pa_tma(plan, p, pp, st, after_kernel)
                                      : launch_pa_generic(plan, p, pp, st);
  if (rc != MSCO_OK) return rc;
  if (pe != nullptr) {
    MSCO_CUDA_CHECK(cudaEventRecord(pe[1], st));
    ++plan->prof_count;
  }
  // with a gather the finishing kernel runs even when no row needs a merge: it is the exchange then
  if (plan->need_reduce || gather != nullptr) rc = launch_pa_reduce(plan, p, pp, st, gather);
  return rc;
}

}  // namespace

extern "C" int msco_paged_attention_launch(const MscoPaPlan *plan, const void *query, const void *key_cache,
                                           const void *value_cache, const int32_t *block_tables,
                                           const float *k_descale, const int32_t *k_offset,
                                           const float *v_descale, const int32_t *v_offset,
                                           const void *attn_mask, void *out, void *workspace,
                                           size_t workspace_bytes, void *stream) {
  return pa_launch_impl(plan, query, key_cache, value_cache, block_tables, k_descale, k_offset, v_descale, v_offset,
                        attn_mask, out, workspace, workspace_bytes, stream, false);
}

// ---------------------------------------------------------------------------------------------
// Multi-token (speculative) queries: every query token becomes a row of the decode batch that shares
// the block table of its sequence.  This builds the per-token block table on the device.
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(256)
expand_rows_kernel(const int32_t *__restrict__ src, const int32_t *__restrict__ row_of, int32_t *__restrict__ dst,
                   int out_rows, int cols) {
  const int64_t total = (int64_t)out_rows * cols;
  for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * 256) {
    const int r = (int)(idx / cols);
    dst[idx] = __ldg(src + (int64_t)__ldg(row_of + r) * cols + (idx - (int64_t)r * cols));
  }
}
}  // namespace

extern "C" int msco_expand_rows_i32(const int32_t *src, int32_t src_rows, int32_t cols, const int32_t *host_row_of,
                                    int32_t out_rows, int32_t *dst, int32_t *device_row_of, void *stream) {
  if (src_rows < 0 || cols < 0 || out_rows < 0) return fail(MSCO_ERR_INVALID_ARG, "expand_rows: negative size");
  if (out_rows == 0 || cols == 0) return MSCO_OK;
  if (src == nullptr || host_row_of == nullptr || dst == nullptr || device_row_of == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "expand_rows: NULL argument");
  for (int32_t i = 0; i < out_rows; ++i)
    if (host_row_of[i] < 0 || host_row_of[i] >= src_rows)
      return fail(MSCO_ERR_INVALID_ARG, "expand_rows: row %d of the output names source row %d of %d", i,
                  host_row_of[i], src_rows);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // pageable source: staged before the call returns, the caller may free it right away
  MSCO_CUDA_CHECK(cudaMemcpyAsync(device_row_of, host_row_of, (size_t)out_rows * sizeof(int32_t),
                                  cudaMemcpyHostToDevice, st));
  const int64_t total = (int64_t)out_rows * cols;
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, 148 * 8));
  expand_rows_kernel<<<grid, 256, 0, st>>>(src, device_row_of, dst, out_rows, cols);
  MSCO_CUDA_CHECK(cudaGetLastError());
  return MSCO_OK;
}

// The same launch with a second output: lse[batch, num_q_heads] (float32), the natural-log sum of
// exp over the context of the scaled (and masked) scores -- what fa_update needs to merge outputs
// computed over different parts of a context.  -inf for an empty context.
extern "C" int msco_paged_attention_launch_lse(const MscoPaPlan *plan, const void *query, const void *key_cache,
                                               const void *value_cache, const int32_t *block_tables,
                                               const float *k_descale, const int32_t *k_offset,
                                               const float *v_descale, const int32_t *v_offset,
                                               const void *attn_mask, void *out, float *lse, void *workspace,
                                               size_t workspace_bytes, void *stream) {
  if (lse == nullptr) return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch_lse: NULL lse");
  return pa_launch_impl(plan, query, key_cache, value_cache, block_tables, k_descale, k_offset, v_descale, v_offset,
                        attn_mask, out, workspace, workspace_bytes, stream, false, lse);
}

// One decode step in one call: scatter the new token rows, then attention.  The attention kernel
// is launched with programmatic stream serialisation behind the scatter kernel, so its set-up
// overlaps the scatter's tail; it waits for the scatter's writes before it reads the cache.
namespace {
int decode_step_impl(const MscoPaPlan *plan, const void *key, const void *value, void *key_cache,
                                void *value_cache, const int32_t *slot_mapping, int64_t num_tokens,
                                const void *query, const int32_t *block_tables, const float *k_descale,
                                const int32_t *k_offset, const float *v_descale, const int32_t *v_offset,
                                const void *attn_mask, void *out, void *workspace, size_t workspace_bytes,
                                void *stream, const GatherArgs *gather) {
  if (plan == nullptr) return fail(MSCO_ERR_INVALID_ARG, "decode_step: NULL plan");
  const MscoPaDesc &d = plan->desc;
  const int64_t row = (int64_t)d.num_kv_heads * d.head_dim;
  const int64_t slots = d.num_blocks * d.block_size;
  if (plan->batch != 0 && (workspace == nullptr || workspace_bytes < plan->workspace_bytes))
    return fail(MSCO_ERR_INVALID_ARG, "decode_step: workspace too small (%zu < %zu)", workspace_bytes,
                plan->workspace_bytes);
  // the scatter kernel also zeroes the attention kernel's scheduling words, which saves the memset
  // (and the launch boundary it would put between the two kernels)
  uint32_t *clear = nullptr;
  int clear_words = 0;
  if (plan->batch != 0 && plan->sync_bytes != 0 && plan->total_items > 0) {
    clear = reinterpret_cast<uint32_t *>(static_cast<char *>(workspace) + plan->sync_offset);
    clear_words = (int)(plan->sync_bytes / 4);
  }
  bool cleared = false;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  if (d.quant_type == 1) {
    rc = launch_rac_quant(key, value, static_cast<int8_t *>(key_cache), static_cast<int8_t *>(value_cache),
                          slot_mapping, num_tokens, row, row, d.q_dtype, k_descale,
                          d.has_quant_offset ? k_offset : nullptr, v_descale,
                          d.has_quant_offset ? v_offset : nullptr, slots, nullptr, st, clear, clear_words, &cleared);
  } else if (d.cache_layout == 1) {
    rc = msco_reshape_and_cache_bnsd(key, value, key_cache, value_cache, slot_mapping, num_tokens, d.num_kv_heads,
                                     (int64_t)d.head_dim * 2, (int64_t)d.head_dim * 2, d.block_size, slots, nullptr,
                                     stream);
  } else {
    rc = launch_rac(key, value, key_cache, value_cache, slot_mapping, num_tokens, row * 2, row * 2, slots, nullptr, st,
                    clear, clear_words, &cleared);
  }
  if (rc != MSCO_OK) return rc;
  return pa_launch_impl(plan, query, key_cache, value_cache, block_tables, k_descale, k_offset, v_descale, v_offset,
                        attn_mask, out, workspace, workspace_bytes, stream, num_tokens > 0, nullptr, cleared, gather);
}
}  // namespace

extern "C" int msco_decode_step(const MscoPaPlan *plan, const void *key, const void *value, void *key_cache,
                                void *value_cache, const int32_t *slot_mapping, int64_t num_tokens,
                                const void *query, const int32_t *block_tables, const float *k_descale,
                                const int32_t *k_offset, const float *v_descale, const int32_t *v_offset,
                                const void *attn_mask, void *out, void *workspace, size_t workspace_bytes,
                                void *stream) {
  return decode_step_impl(plan, key, value, key_cache, value_cache, slot_mapping, num_tokens, query, block_tables,
                          k_descale, k_offset, v_descale, v_offset, attn_mask, out, workspace, workspace_bytes, stream,
                          nullptr);
}

extern "C" int msco_decode_step_gather(const MscoPaPlan *plan, const void *key, const void *value, void *key_cache,
                                       void *value_cache, const int32_t *slot_mapping, int64_t num_tokens,
                                       const void *query, const int32_t *block_tables, const float *k_descale,
                                       const int32_t *k_offset, const float *v_descale, const int32_t *v_offset,
                                       const void *attn_mask, void *out, void *workspace, size_t workspace_bytes,
                                       void *stream, const MscoGatherDesc *gather, uint32_t step) {
  if (plan == nullptr) return fail(MSCO_ERR_INVALID_ARG, "decode_step_gather: NULL plan");
  if (plan->batch == 0) return fail(MSCO_ERR_INVALID_ARG, "decode_step_gather: an empty batch has nothing to gather");
  GatherArgs g;
  const int rc = fill_gather_args(gather, step, "decode_step_gather", &g);
  if (rc != MSCO_OK) return rc;
  return decode_step_impl(plan, key, value, key_cache, value_cache, slot_mapping, num_tokens, query, block_tables,
                          k_descale, k_offset, v_descale, v_offset, attn_mask, out, workspace, workspace_bytes, stream,
                          &g);
}


extern "C" int msco_paged_attention_status(const MscoPaPlan *plan, const void *workspace) {
  // plan may be NULL: the epoch of the last launch that used this workspace is remembered
  if (workspace == nullptr) return fail(MSCO_ERR_INVALID_ARG, "paged_attention_status: NULL workspace");
  if (plan != nullptr && plan->batch == 0) return MSCO_OK;
  uint32_t epoch = 0;
  if (plan != nullptr) epoch = plan->last_epoch;
  else if (!recall_launch(workspace, &epoch)) return MSCO_OK;  // nothing was launched with it
  int32_t words[2] = {0, 0};
  MSCO_CUDA_CHECK(cudaMemcpy(words, workspace, sizeof(words), cudaMemcpyDeviceToHost));
  if ((uint32_t)words[1] != epoch) return MSCO_OK;  // no kernel of that launch reported anything
  if (words[0] == kStatusTimeout) return fail(MSCO_ERR_TIMEOUT, "paged_attention: a bounded wait inside the kernel expired");
  if (words[0] == kStatusOob) return fail(MSCO_ERR_OOB, "paged_attention: a block id outside the cache was met");
  return MSCO_OK;
}

// ---------------------------------------------------------------------------------------------
// Launch without caller-provided scratch: the workspace is a fixed array in the device image.
// ---------------------------------------------------------------------------------------------
namespace {

// Scratch of msco_paged_attention_launch_static.  In host code this name is only a handle for
// cudaGetSymbolAddress -- it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[MSCO_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void *g_static_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch(void **ptr) {
  int dev = -1;
  MSCO_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(MSCO_ERR_INTERNAL, "launch_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> g(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void *p = nullptr;
    MSCO_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return fail(MSCO_ERR_CUDA, "launch_static: cudaGetSymbolAddress returned a NULL address");
    g_static_ptr[dev] = p;
  }
  *ptr = g_static_ptr[dev];
  return MSCO_OK;
}

}  // namespace

extern "C" int msco_paged_attention_launch_static(const MscoPaPlan *plan, const void *query,
                                                  const void *key_cache, const void *value_cache,
                                                  const int32_t *block_tables, const float *k_descale,
                                                  const int32_t *k_offset, const float *v_descale,
                                                  const int32_t *v_offset, const void *attn_mask, void *out,
                                                  void *stream) {
  if (plan == nullptr) return fail(MSCO_ERR_INVALID_ARG, "paged_attention_launch_static: NULL plan");
  if (plan->workspace_bytes > (size_t)MSCO_STATIC_SCRATCH_BYTES)
    return fail(MSCO_ERR_INVALID_ARG,
                "paged_attention_launch_static: this plan needs %zu bytes of scratch but the built-in scratch "
                "holds %zu; use msco_paged_attention_launch with a caller-provided workspace",
                plan->workspace_bytes, (size_t)MSCO_STATIC_SCRATCH_BYTES);
  void *ws = nullptr;
  const int rc = static_scratch(&ws);
  if (rc != MSCO_OK) return rc;
  return msco_paged_attention_launch(plan, query, key_cache, value_cache, block_tables, k_descale, k_offset,
                                     v_descale, v_offset, attn_mask, out, ws, (size_t)MSCO_STATIC_SCRATCH_BYTES,
                                     stream);
}

extern "C" int msco_paged_attention_status_static(const MscoPaPlan *plan) {
  void *ws = nullptr;
  const int rc = static_scratch(&ws);
  if (rc != MSCO_OK) return rc;
  return msco_paged_attention_status(plan, ws);
}
