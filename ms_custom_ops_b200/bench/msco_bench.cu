// Standalone C++ benchmark of the paged-KV decode path through the thin C ABI (msco_b200.h):
// no Python, no PyTorch.  Builds a synthetic decode workload in GPU memory (counter-based generator)
// and steps it the way a serving loop does: every step appends one token to every sequence
// (context_lens + 1, slot_mapping moves to the new position, block tables already hold the blocks
// reserved for the growth), re-plans in place (msco_paged_attention_replan) and issues one
// msco_decode_step (cache scatter + attention).  Prints one JSON line:
//   value / ms_per_step          device-timed loop, everything resident in HBM (CUDA events, median of --repeats loops)
//   attention_kernel_ms, kernel_gbs, frac_of_peak, frac_of_8tbs   the attention kernel alone (event pairs around it)
//   e2e_ms_per_step / e2e_value  the same step with the inputs in PINNED HOST memory: one packed host->device
//                                copy (query | new K rows | new V rows | slots | block tables), the step, the
//                                device->host copy of the output, the host waits -- serial, what one batch of
//                                autoregressive decode can do
//
//   msco_bench [--config c1|c2|c3|c4|c5] [--batch N] [--q-heads N] [--kv-heads N] [--head-dim 64|128|256]
//              [--block-size N] [--len-lo N] [--len-hi N] [--loguniform] [--int8] [--fp16]
//              [--steps 50] [--warmup 5] [--repeats 5] [--seed 2] [--peak-gbs 6553.6] [--dump FILE]
//
// --config presets are the five benchmark configurations (c1 st-style fp16 batch 4; c2 8B-shaped bf16
// batch 64, lengths U[2048, 8192]; c3 int8 KV batch 128, 64 q heads, U[1024, 4096]; c4 bf16 batch 32,
// 64 q heads, log-uniform [512, 131072]; c5 decode bf16 batch 256, U[128, 2048]).
// Lengths are drawn as stated; block tables are a shuffled assignment of a block pool sized to the
// tokens + 10 % (+ the blocks the decode loop grows into); Q / K / V / new rows ~ N(0, 1) (int8 caches:
// N(0, 1) quantised per channel with scales uniform in [0.01, 0.05]).
// --dump FILE writes the state of one extra step (lengths, tables, slots, query, new rows, scales, both
// caches after the step, and the output) so that a checker outside this program can recompute the step.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <random>
#include <string>
#include <vector>

#include "msco_b200.h"

#define CK(x)                                                                              \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      fprintf(stderr, "%s failed: %s (%s:%d)\n", #x, cudaGetErrorString(e_), __FILE__, __LINE__); \
      exit(2);                                                                             \
    }                                                                                      \
  } while (0)
#define MS(x)                                                                \
  do {                                                                       \
    int r_ = (x);                                                            \
    if (r_ != MSCO_OK) {                                                     \
      fprintf(stderr, "%s failed (%d): %s\n", #x, r_, msco_last_error());    \
      exit(3);                                                               \
    }                                                                        \
  } while (0)

__device__ __forceinline__ uint64_t splitmix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ float normal_at(uint64_t seed, uint64_t i) {  // Box-Muller on two counters
  const uint64_t a = splitmix(seed ^ (2 * i)), b = splitmix(seed ^ (2 * i + 1));
  const float u1 = ((a >> 40) + 1) * (1.0f / 16777217.0f), u2 = (b >> 40) * (1.0f / 16777216.0f);
  return sqrtf(-2.f * logf(u1)) * cospif(2.f * u2);
}
template <typename T> __device__ T cvt(float v);
template <> __device__ __half cvt<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __nv_bfloat16 cvt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __global__ void fill_normal(T *p, size_t n, uint64_t seed) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    p[i] = cvt<T>(normal_at(seed, i));
}
__global__ void fill_normal_q8(int8_t *p, size_t n, uint64_t seed, const float *descale, int channels) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float q = rintf(normal_at(seed, i) / descale[i % channels]);
    p[i] = (int8_t)fminf(fmaxf(q, -128.f), 127.f);
  }
}
__global__ void fill_uniform(float *p, size_t n, uint64_t seed, float lo, float hi) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    p[i] = lo + (hi - lo) * (splitmix(seed ^ i) >> 40) * (1.0f / 16777216.0f);
}

static void dump_section(FILE *f, const char *name, const void *host, size_t bytes) {
  char tag[32];
  memset(tag, 0, sizeof(tag));
  strncpy(tag, name, sizeof(tag) - 1);
  const uint64_t n = bytes;
  fwrite(tag, 1, sizeof(tag), f);
  fwrite(&n, 8, 1, f);
  fwrite(host, 1, bytes, f);
}
static void dump_device(FILE *f, const char *name, const void *dev, size_t bytes) {
  std::vector<char> h(bytes);
  CK(cudaMemcpy(h.data(), dev, bytes, cudaMemcpyDeviceToHost));
  dump_section(f, name, h.data(), bytes);
}

int main(int argc, char **argv) {
  int batch = 64, hq = 32, hkv = 8, d = 128, bs = 128, len_lo = 2048, len_hi = 8192, steps = 50, warmup = 5, repeats = 5;
  uint64_t seed = 2;
  bool int8 = false, fp16 = false, loguniform = false;
  double peak_gbs = 6553.6;
  std::string config = "c2", dump;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() { return (i + 1 < argc) ? atoi(argv[++i]) : 0; };
    if (a == "--config") {
      config = (i + 1 < argc) ? argv[++i] : "c2";
      if (config == "c1") { batch = 4; hq = 32; len_lo = 1; len_hi = 1024; fp16 = true; seed = 0; }
      else if (config == "c2") { batch = 64; hq = 32; len_lo = 2048; len_hi = 8192; }
      else if (config == "c3") { batch = 128; hq = 64; len_lo = 1024; len_hi = 4096; int8 = true; seed = 3; }
      else if (config == "c4") { batch = 32; hq = 64; len_lo = 512; len_hi = 131072; loguniform = true; seed = 4; }
      else if (config == "c5") { batch = 256; hq = 32; len_lo = 128; len_hi = 2048; seed = 5; }
      else { fprintf(stderr, "unknown config %s\n", config.c_str()); return 1; }
    }
    else if (a == "--batch") batch = next(); else if (a == "--q-heads") hq = next(); else if (a == "--kv-heads") hkv = next();
    else if (a == "--head-dim") d = next(); else if (a == "--block-size") bs = next();
    else if (a == "--len-lo") len_lo = next(); else if (a == "--len-hi") len_hi = next();
    else if (a == "--steps") steps = next(); else if (a == "--warmup") warmup = next(); else if (a == "--repeats") repeats = next();
    else if (a == "--seed") seed = (uint64_t)next(); else if (a == "--int8") int8 = true; else if (a == "--fp16") fp16 = true;
    else if (a == "--loguniform") loguniform = true;
    else if (a == "--peak-gbs") peak_gbs = (i + 1 < argc) ? atof(argv[++i]) : peak_gbs;
    else if (a == "--dump") dump = (i + 1 < argc) ? argv[++i] : "";
    else { fprintf(stderr, "unknown argument %s\n", a.c_str()); return 1; }
  }
  warmup = std::max(warmup, 3);
  repeats = std::max(repeats, 1);
  const int nprof = std::min(steps, 64);
  const int total_steps = warmup + repeats * steps + nprof + (3 + steps) + 4;  // every step the loop will ever issue

  // ---- lengths, block tables (with the blocks the loop grows into), slots of every step ----
  std::mt19937_64 rng(seed);
  std::vector<int32_t> lens0(batch);
  for (auto &l : lens0) {
    if (loguniform) {
      const double u = std::log((double)len_lo) + (std::log((double)len_hi) - std::log((double)len_lo)) * ((rng() >> 11) * (1.0 / 9007199254740992.0));
      l = std::min<int32_t>((int32_t)std::floor(std::exp(u)), len_hi);
    } else {
      l = len_lo + (int32_t)(rng() % (uint64_t)(len_hi - len_lo + 1));
    }
  }
  int64_t blocks_now = 0, blocks_later = 0, kv_tokens0 = 0;
  int width = 1;
  for (int b = 0; b < batch; ++b) {
    blocks_now += (lens0[b] + bs - 1) / bs;
    blocks_later += (lens0[b] + total_steps + bs - 1) / bs;
    width = std::max(width, (lens0[b] + total_steps + bs - 1) / bs);
    kv_tokens0 += lens0[b];
  }
  const int64_t nb_pool = (int64_t)std::ceil(blocks_now * 1.1) + 1;
  const int64_t nb = nb_pool + (blocks_later - blocks_now);  // fresh blocks for the growth are appended to the pool
  std::vector<int32_t> pool(nb_pool);
  std::iota(pool.begin(), pool.end(), 0);
  std::shuffle(pool.begin(), pool.end(), rng);
  std::vector<int32_t> tables((size_t)batch * width, 0);
  size_t next_block = 0;
  int64_t next_fresh = nb_pool;
  for (int b = 0; b < batch; ++b) {
    const int now = (lens0[b] + bs - 1) / bs, later = (lens0[b] + total_steps + bs - 1) / bs;
    for (int j = 0; j < now; ++j) tables[(size_t)b * width + j] = pool[next_block++];
    for (int j = now; j < later; ++j) tables[(size_t)b * width + j] = (int32_t)next_fresh++;
  }
  auto slot_of = [&](int b, int step) {  // slot of sequence b's newest token at `step` (its length: lens0 + step)
    const int64_t last = (int64_t)lens0[b] + step - 1;
    return last < 0 ? -1 : (int32_t)((int64_t)tables[(size_t)b * width + last / bs] * bs + last % bs);
  };
  std::vector<int32_t> slots_all((size_t)(total_steps + 1) * batch);
  for (int s = 0; s <= total_steps; ++s)
    for (int b = 0; b < batch; ++b) slots_all[(size_t)s * batch + b] = slot_of(b, s);

  const size_t c = (size_t)hkv * d, cache_elems = (size_t)nb * bs * c;
  const int es = 2, kes = int8 ? 1 : 2;
  const size_t q_bytes = (size_t)batch * hq * d * es, row_bytes = (size_t)batch * c * es;
  void *q, *key, *val, *kc, *vc, *out;
  int32_t *d_tables, *d_slots_all;
  float *kd = nullptr, *vd = nullptr;
  CK(cudaMalloc(&q, q_bytes));
  CK(cudaMalloc(&out, q_bytes));
  CK(cudaMalloc(&key, row_bytes));
  CK(cudaMalloc(&val, row_bytes));
  CK(cudaMalloc(&kc, cache_elems * kes));
  CK(cudaMalloc(&vc, cache_elems * kes));
  CK(cudaMalloc(&d_tables, tables.size() * 4));
  CK(cudaMalloc(&d_slots_all, slots_all.size() * 4));
  CK(cudaMemcpy(d_tables, tables.data(), tables.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_slots_all, slots_all.data(), slots_all.size() * 4, cudaMemcpyHostToDevice));
  const int G = 148 * 8, B = 256;
  auto fill16 = [&](void *p, size_t n, uint64_t s) {
    if (fp16) fill_normal<__half><<<G, B>>>((__half *)p, n, s); else fill_normal<__nv_bfloat16><<<G, B>>>((__nv_bfloat16 *)p, n, s);
  };
  fill16(q, (size_t)batch * hq * d, seed * 7 + 1);
  fill16(key, (size_t)batch * c, seed * 7 + 2);
  fill16(val, (size_t)batch * c, seed * 7 + 3);
  if (int8) {
    CK(cudaMalloc(&kd, c * 4));
    CK(cudaMalloc(&vd, c * 4));
    fill_uniform<<<8, B>>>(kd, c, seed * 7 + 4, 0.01f, 0.05f);
    fill_uniform<<<8, B>>>(vd, c, seed * 7 + 5, 0.01f, 0.05f);
    fill_normal_q8<<<G, B>>>((int8_t *)kc, cache_elems, seed * 7 + 6, kd, (int)c);
    fill_normal_q8<<<G, B>>>((int8_t *)vc, cache_elems, seed * 7 + 7, vd, (int)c);
  } else {
    fill16(kc, cache_elems, seed * 7 + 6);
    fill16(vc, cache_elems, seed * 7 + 7);
  }
  CK(cudaDeviceSynchronize());

  MscoPaDesc desc;
  memset(&desc, 0, sizeof(desc));
  desc.q_dtype = fp16 ? MSCO_DTYPE_F16 : MSCO_DTYPE_BF16;
  desc.kv_dtype = int8 ? MSCO_DTYPE_I8 : desc.q_dtype;
  desc.num_q_heads = hq; desc.num_kv_heads = hkv; desc.head_dim = d; desc.block_size = bs;
  desc.num_blocks = nb; desc.max_blocks_per_seq = width; desc.qk_scale = 1.0f / std::sqrt((float)d);
  desc.quant_type = int8 ? 1 : 0;
  // the partial count grows with the lengths: size the workspace for the last step
  std::vector<int32_t> lens(batch);
  for (int b = 0; b < batch; ++b) lens[b] = lens0[b] + total_steps;
  MscoPaPlan *plan = nullptr;
  MS(msco_paged_attention_plan(&desc, lens.data(), batch, &plan));
  const size_t ws_bytes = std::max<size_t>(msco_paged_attention_workspace_bytes(plan), 256);
  void *ws;
  CK(cudaMalloc(&ws, ws_bytes));
  cudaStream_t st;
  CK(cudaStreamCreate(&st));

  int cur = 0;  // index of the next step
  auto step_from = [&](const void *q_, const void *key_, const void *val_, const int32_t *slots_, const int32_t *tables_) {
    for (int b = 0; b < batch; ++b) lens[b] = lens0[b] + cur;
    MS(msco_paged_attention_replan(plan, lens.data(), batch));
    MS(msco_decode_step(plan, key_, val_, kc, vc, slots_, batch, q_, tables_, kd, nullptr, vd, nullptr, nullptr, out, ws,
                        ws_bytes, st));
    ++cur;
  };
  auto step = [&]() { step_from(q, key, val, d_slots_all + (size_t)cur * batch, d_tables); };

  for (int i = 0; i < warmup; ++i) step();
  CK(cudaStreamSynchronize(st));
  MS(msco_paged_attention_status(plan, ws));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  std::vector<double> loop_ms;
  const int first_timed = cur;
  for (int r = 0; r < repeats; ++r) {
    CK(cudaStreamSynchronize(st));
    CK(cudaEventRecord(e0, st));
    for (int i = 0; i < steps; ++i) step();
    CK(cudaEventRecord(e1, st));
    CK(cudaStreamSynchronize(st));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    loop_ms.push_back(ms / steps);
  }
  std::sort(loop_ms.begin(), loop_ms.end());
  const double step_ms = loop_ms[loop_ms.size() / 2];

  // the attention kernel alone
  MS(msco_paged_attention_profile_enable(plan, 1));
  const int first_prof = cur;
  for (int i = 0; i < nprof; ++i) step();
  CK(cudaStreamSynchronize(st));
  float kms[64];
  int32_t nk = 0;
  MS(msco_paged_attention_profile_read(plan, kms, 64, &nk));
  MS(msco_paged_attention_profile_enable(plan, 0));
  double kavg = 0;
  for (int i = 0; i < nk; ++i) kavg += kms[i];
  kavg = nk ? kavg / nk : 0;
  MscoPaPlanInfo info;
  MS(msco_paged_attention_plan_info(plan, &info));
  const double tokens_prof = (double)kv_tokens0 + (double)batch * (first_prof + (nprof - 1) / 2.0);
  const double bytes = tokens_prof * 2 * hkv * d * kes + (double)batch * hq * d * 4 + (int8 ? 2.0 * c * 4 : 0.0);

  // ---- end to end, serial, inputs in pinned host memory ----
  size_t offs[5], total = 0;
  const size_t sizes[5] = {q_bytes, row_bytes, row_bytes, (size_t)batch * 4, tables.size() * 4};
  for (int i = 0; i < 5; ++i) { offs[i] = total; total += (sizes[i] + 255) / 256 * 256; }
  char *h_stage, *d_stage, *h_out;
  CK(cudaHostAlloc((void **)&h_stage, total, cudaHostAllocDefault));
  CK(cudaHostAlloc((void **)&h_out, q_bytes, cudaHostAllocDefault));
  CK(cudaMalloc((void **)&d_stage, total));
  CK(cudaMemcpy(h_stage + offs[0], q, q_bytes, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(h_stage + offs[1], key, row_bytes, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(h_stage + offs[2], val, row_bytes, cudaMemcpyDeviceToHost));
  memcpy(h_stage + offs[4], tables.data(), tables.size() * 4);
  auto e2e_step = [&]() {
    memcpy(h_stage + offs[3], slots_all.data() + (size_t)cur * batch, (size_t)batch * 4);
    CK(cudaMemcpyAsync(d_stage, h_stage, total, cudaMemcpyHostToDevice, st));
    step_from(d_stage + offs[0], d_stage + offs[1], d_stage + offs[2], (const int32_t *)(d_stage + offs[3]),
              (const int32_t *)(d_stage + offs[4]));
    CK(cudaMemcpyAsync(h_out, out, q_bytes, cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));  // the step's result is read on the host
  };
  for (int i = 0; i < 3; ++i) e2e_step();
  int64_t arena0[6], arena1[6];
  msco_plan_arena_stats(arena0);
  CK(cudaEventRecord(e0, st));
  for (int i = 0; i < steps; ++i) e2e_step();
  CK(cudaEventRecord(e1, st));
  CK(cudaStreamSynchronize(st));
  msco_plan_arena_stats(arena1);
  float e2e_total = 0.f;
  CK(cudaEventElapsedTime(&e2e_total, e0, e1));
  const double e2e_ms = e2e_total / steps;
  MS(msco_paged_attention_status(plan, ws));

  if (!dump.empty()) {
    // one more step whose state is written out for an external checker
    const int s = cur;
    step();
    CK(cudaStreamSynchronize(st));
    FILE *f = fopen(dump.c_str(), "wb");
    if (f == nullptr) { fprintf(stderr, "cannot open %s\n", dump.c_str()); return 4; }
    const int32_t hdr[12] = {batch, hq, hkv, d, bs, (int32_t)nb, width, int8 ? 1 : 0, fp16 ? 1 : 0, s, 0, 0};
    dump_section(f, "header", hdr, sizeof(hdr));
    for (int b = 0; b < batch; ++b) lens[b] = lens0[b] + s;
    dump_section(f, "context_lens", lens.data(), lens.size() * 4);
    dump_section(f, "block_tables", tables.data(), tables.size() * 4);
    dump_section(f, "slot_mapping", slots_all.data() + (size_t)s * batch, (size_t)batch * 4);
    dump_device(f, "query", q, q_bytes);
    dump_device(f, "key", key, row_bytes);
    dump_device(f, "value", val, row_bytes);
    if (int8) {
      dump_device(f, "k_descale", kd, c * 4);
      dump_device(f, "v_descale", vd, c * 4);
    }
    dump_device(f, "key_cache", kc, cache_elems * kes);
    dump_device(f, "value_cache", vc, cache_elems * kes);
    dump_device(f, "out", out, q_bytes);
    fclose(f);
  }

  printf("{\"harness\": \"msco_bench\", \"metric\": \"paged-attn decode tokens/s\", \"config\": \"%s\", \"value\": %.1f, "
         "\"unit\": \"tokens/s\", \"ms_per_step\": %.5f, \"loops\": %d, \"steps\": %d, \"warmup\": %d, "
         "\"attention_kernel_ms\": %.5f, \"kernel_gbs\": %.1f, \"frac_of_peak\": %.4f, \"peak_gbs\": %.1f, "
         "\"frac_of_8tbs\": %.4f, \"algorithmic_bytes\": %.0f, \"e2e_value\": %.1f, \"e2e_ms_per_step\": %.5f, "
         "\"e2e_mode\": \"serial, pinned host buffers, one packed upload, output downloaded, host waits\", "
         "\"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu, \"pinned_slabs_added_in_e2e_loop\": %lld, "
         "\"launch\": \"real decode loop: lengths + 1 per step, re-plan in place, msco_decode_step (2 kernels)\", "
         "\"batch\": %d, \"q_heads\": %d, \"kv_heads\": %d, \"head_dim\": %d, \"block_size\": %d, \"kv_tokens\": %lld, "
         "\"kv\": \"%s\", \"kernel\": %d, \"work_items\": %d, \"split_partials\": %d, \"grid\": %d, \"first_timed_step\": %d}\n",
         config.c_str(), batch / step_ms * 1e3, step_ms, repeats, steps, warmup, kavg, kavg > 0 ? bytes / kavg / 1e6 : 0.0,
         kavg > 0 ? bytes / kavg / 1e6 / peak_gbs : 0.0, peak_gbs, kavg > 0 ? bytes / kavg / 1e6 / 8000.0 : 0.0, bytes,
         batch / e2e_ms * 1e3, e2e_ms, total, q_bytes, (long long)(arena1[0] - arena0[0]), batch, hq, hkv, d, bs,
         (long long)(kv_tokens0 + (int64_t)batch * first_timed), int8 ? "int8" : (fp16 ? "fp16" : "bf16"), info.kernel,
         info.work_items, info.partials, info.grid, first_timed);
  msco_paged_attention_plan_destroy(plan);
  return 0;
}
