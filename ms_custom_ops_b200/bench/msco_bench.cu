// Standalone C++ benchmark of the paged-KV decode path through the thin C ABI (msco_b200.h):
// no Python, no PyTorch.  Builds a synthetic decode step in GPU memory (counter-based generator),
// runs reshape_and_cache + paged attention `steps` times with CUDA events and prints one JSON line.
//
//   msco_bench [--batch 64] [--q-heads 32] [--kv-heads 8] [--len-lo 2048] [--len-hi 8192]
//              [--int8] [--fp16] [--steps 50] [--warmup 5] [--seed 2]
//
// Lengths are uniform in [len-lo, len-hi]; block tables are a shuffled assignment of a block pool
// sized to the tokens + 10 %; Q / K / V / new rows ~ N(0, 1) (int8 caches: N(0,1) quantised per
// channel with scales uniform in [0.01, 0.05]).
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

int main(int argc, char **argv) {
  int batch = 64, hq = 32, hkv = 8, d = 128, bs = 128, len_lo = 2048, len_hi = 8192, steps = 50, warmup = 5;
  uint64_t seed = 2;
  bool int8 = false, fp16 = false;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() { return (i + 1 < argc) ? atoi(argv[++i]) : 0; };
    if (a == "--batch") batch = next(); else if (a == "--q-heads") hq = next(); else if (a == "--kv-heads") hkv = next();
    else if (a == "--len-lo") len_lo = next(); else if (a == "--len-hi") len_hi = next();
    else if (a == "--steps") steps = next(); else if (a == "--warmup") warmup = next();
    else if (a == "--seed") seed = (uint64_t)next(); else if (a == "--int8") int8 = true; else if (a == "--fp16") fp16 = true;
    else { fprintf(stderr, "unknown argument %s\n", a.c_str()); return 1; }
  }
  std::mt19937_64 rng(seed);
  std::vector<int32_t> lens(batch);
  int64_t blocks_needed = 0, kv_tokens = 0;
  for (auto &l : lens) {
    l = len_lo + (int32_t)(rng() % (uint64_t)(len_hi - len_lo + 1));
    blocks_needed += (l + bs - 1) / bs;
    kv_tokens += l;
  }
  const int64_t nb = (int64_t)std::ceil(blocks_needed * 1.1) + 1;
  std::vector<int32_t> pool(nb);
  std::iota(pool.begin(), pool.end(), 0);
  std::shuffle(pool.begin(), pool.end(), rng);
  const int width = (*std::max_element(lens.begin(), lens.end()) + bs - 1) / bs;
  std::vector<int32_t> tables((size_t)batch * width, 0), slots(batch);
  size_t next_block = 0;
  for (int b = 0; b < batch; ++b) {
    const int need = (lens[b] + bs - 1) / bs;
    for (int j = 0; j < need; ++j) tables[(size_t)b * width + j] = pool[next_block++];
    slots[b] = tables[(size_t)b * width + (lens[b] - 1) / bs] * bs + (lens[b] - 1) % bs;
  }
  const size_t c = (size_t)hkv * d, cache_elems = (size_t)nb * bs * c;
  const int es = 2, kes = int8 ? 1 : 2;
  void *q, *key, *val, *kc, *vc, *out;
  int32_t *d_tables, *d_slots;
  float *kd = nullptr, *vd = nullptr;
  CK(cudaMalloc(&q, (size_t)batch * hq * d * es));
  CK(cudaMalloc(&out, (size_t)batch * hq * d * es));
  CK(cudaMalloc(&key, (size_t)batch * c * es));
  CK(cudaMalloc(&val, (size_t)batch * c * es));
  CK(cudaMalloc(&kc, cache_elems * kes));
  CK(cudaMalloc(&vc, cache_elems * kes));
  CK(cudaMalloc(&d_tables, tables.size() * 4));
  CK(cudaMalloc(&d_slots, slots.size() * 4));
  CK(cudaMemcpy(d_tables, tables.data(), tables.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(d_slots, slots.data(), slots.size() * 4, cudaMemcpyHostToDevice));
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
  MscoPaPlan *plan = nullptr;
  MS(msco_paged_attention_plan(&desc, lens.data(), batch, &plan));
  MscoPaPlanInfo info;
  MS(msco_paged_attention_plan_info(plan, &info));
  void *ws;
  CK(cudaMalloc(&ws, std::max<size_t>(msco_paged_attention_workspace_bytes(plan), 256)));
  cudaStream_t st;
  CK(cudaStreamCreate(&st));
  auto step = [&]() {
    if (int8) MS(msco_reshape_and_cache_quant(key, val, (int8_t *)kc, (int8_t *)vc, d_slots, batch, c, c, desc.q_dtype, kd, nullptr, vd, nullptr, nb * bs, nullptr, st));
    else MS(msco_reshape_and_cache(key, val, kc, vc, d_slots, batch, c * es, c * es, nb * bs, nullptr, st));
    MS(msco_paged_attention_launch(plan, q, kc, vc, d_tables, kd, nullptr, vd, nullptr, nullptr, out, ws,
                                   msco_paged_attention_workspace_bytes(plan) < 256 ? 256 : msco_paged_attention_workspace_bytes(plan), st));
  };
  for (int i = 0; i < std::max(warmup, 3); ++i) step();
  CK(cudaStreamSynchronize(st));
  MS(msco_paged_attention_status(plan, ws));
  MS(msco_paged_attention_profile_enable(plan, 1));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e0, st));
  for (int i = 0; i < steps; ++i) step();
  CK(cudaEventRecord(e1, st));
  CK(cudaStreamSynchronize(st));
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, e0, e1));
  float kms[64];
  int32_t nk = 0;
  MS(msco_paged_attention_profile_read(plan, kms, 64, &nk));
  double kavg = 0;
  for (int i = 0; i < nk; ++i) kavg += kms[i];
  kavg = nk ? kavg / nk : 0;
  const double bytes = (double)kv_tokens * 2 * hkv * d * kes + (double)batch * hq * d * 4 + (int8 ? 2.0 * c * 4 : 0.0);
  const double step_ms = ms / steps;
  printf("{\"harness\": \"msco_bench\", \"metric\": \"paged-attn decode tokens/s\", \"value\": %.1f, \"unit\": \"tokens/s\", "
         "\"ms_per_step\": %.5f, \"attention_kernel_ms\": %.5f, \"kernel_gbs\": %.1f, \"frac_of_8tbs\": %.4f, "
         "\"algorithmic_bytes\": %.0f, \"batch\": %d, \"q_heads\": %d, \"kv_heads\": %d, \"kv_tokens\": %lld, "
         "\"kv\": \"%s\", \"work_items\": %d, \"grid\": %d, \"steps\": %d}\n",
         batch / step_ms * 1e3, step_ms, kavg, kavg > 0 ? bytes / kavg / 1e6 : 0.0, kavg > 0 ? bytes / kavg / 1e6 / 8000.0 : 0.0,
         bytes, batch, hq, hkv, (long long)kv_tokens, int8 ? "int8" : (fp16 ? "fp16" : "bf16"), info.work_items, info.grid, steps);
  msco_paged_attention_plan_destroy(plan);
  return 0;
}
