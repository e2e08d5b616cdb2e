// paged_cache_load for B200: gather the token rows of every sequence out of the paged K/V cache
// into contiguous [sum_tokens, heads * head_dim] tensors -- the inverse data movement of
// reshape_and_cache, same block-table indexing.
//
// HBM-bound byte movement.  The tokens of one cache block are contiguous in the cache
// ([block_size, heads, head_dim]) and in the output, so the unit of work is one (sequence, block)
// pair = one contiguous copy of up to block_size rows, K and V in different CTAs (grid.y).
// Algorithmic bytes per gathered token: (k_row_bytes + v_row_bytes) read + the same written.
//
// Where a row lands is decided on the device, by a one-CTA prologue kernel, so that no host copy of
// the lengths is needed: an exclusive scan of the valid tokens of all (sequence, block) pairs.
// Blocks with a negative id contribute no rows and the rows behind them move up, the rows left over
// at the end of the output are zero (tests/st/test_custom_paged_cache_load.py:35-76).
#include <algorithm>

#include "msco_common.cuh"

namespace msco {
namespace {

constexpr int kPclThreads = 256;
constexpr int kPclOffsetThreads = 1024;
constexpr int kPclHeaderWords = 16;  // ws[0] = rows written; the rest reserved
constexpr int kPclZeroCtas = 32;     // CTAs (per K / V) that clear the rows nothing was gathered into

__device__ __forceinline__ uint4 ld_nc16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_cs16(uint4 *p, const uint4 &v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <typename V> __device__ __forceinline__ V pcl_ld(const V *p) { return __ldg(p); }
template <> __device__ __forceinline__ uint4 pcl_ld<uint4>(const uint4 *p) { return ld_nc16(p); }
template <typename V> __device__ __forceinline__ void pcl_st(V *p, const V &v) { *p = v; }
template <> __device__ __forceinline__ void pcl_st<uint4>(uint4 *p, const uint4 &v) { st_cs16(p, v); }
template <typename V> __device__ __forceinline__ V pcl_zero() { return V(0); }
template <> __device__ __forceinline__ uint4 pcl_zero<uint4>() { return make_uint4(0u, 0u, 0u, 0u); }

struct SeqSpan {
  int len;  // tokens of the sequence (0 for a malformed length)
  int off;  // first block-table column
  bool bad;
};

// seq_lens holds lengths [batch] or, in cumulative mode, running sums [batch + 1];
// seq_starts (optional) is a token position whose block is the first one read
__device__ __forceinline__ SeqSpan seq_span(const int32_t *seq_lens, const int32_t *seq_starts, int i, int cumsum,
                                            int block_size) {
  SeqSpan s;
  s.len = cumsum ? __ldg(seq_lens + i + 1) - __ldg(seq_lens + i) : __ldg(seq_lens + i);
  s.bad = s.len < 0;
  if (s.bad) s.len = 0;
  int start = seq_starts != nullptr ? __ldg(seq_starts + i) : 0;
  if (start < 0) {
    s.bad = true;
    start = 0;
  }
  s.off = start / block_size;
  return s;
}

// rows block j of sequence i contributes: 0 for a negative id (skipped, as in the golden) and for a
// column or id out of range (counted in *bad)
__device__ __forceinline__ int block_rows(const int32_t *row_table, const SeqSpan &s, int j, int max_blocks,
                                          int block_size, int num_blocks, int *bad) {
  const int col = s.off + j;
  if (col >= max_blocks) {
    ++*bad;
    return 0;
  }
  const int id = __ldg(row_table + col);
  if (id < 0) return 0;
  if (id >= num_blocks) {
    ++*bad;
    return 0;
  }
  return min(block_size, s.len - j * block_size);
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
  for (int sh = 16; sh > 0; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
  return v;
}
__device__ __forceinline__ int warp_inclusive_scan(int v, int lane) {
#pragma unroll
  for (int sh = 1; sh < 32; sh <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, v, sh);
    if (lane >= sh) v += o;
  }
  return v;
}

// ws: [0] rows written in total, [16 .. 16 + batch) first output row of each sequence,
//     then dest[batch][max_blocks]: first output row of each (sequence, block), -1 = nothing to copy
__global__ void __launch_bounds__(kPclOffsetThreads)
pcl_offsets_kernel(const int32_t *__restrict__ block_tables, const int32_t *__restrict__ seq_lens,
                   const int32_t *__restrict__ seq_starts, int batch, int max_blocks, int block_size,
                   int num_blocks, int cumsum, int32_t *__restrict__ ws, int32_t *oob_count) {
  // the copy kernel is launched with programmatic stream serialisation: let it become resident
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kPclOffsetThreads / 32;
  int32_t *base = ws + kPclHeaderWords;
  int32_t *dest = base + batch;

  for (int i = warp; i < batch; i += kWarps) {
    const SeqSpan s = seq_span(seq_lens, seq_starts, i, cumsum, block_size);
    const int nblk = (s.len + block_size - 1) / block_size;
    const int32_t *row = block_tables + (int64_t)i * max_blocks;
    int rows = 0, bad = (s.bad && lane == 0) ? 1 : 0;
    for (int j = lane; j < nblk; j += 32) rows += block_rows(row, s, j, max_blocks, block_size, num_blocks, &bad);
    rows = warp_sum(rows);
    bad = warp_sum(bad);
    if (lane == 0) {
      base[i] = rows;
      if (bad != 0 && oob_count != nullptr) atomicAdd(oob_count, bad);
    }
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int i0 = 0; i0 < batch; i0 += 32) {
      const int i = i0 + lane;
      const int v = i < batch ? base[i] : 0;
      const int incl = warp_inclusive_scan(v, lane);
      if (i < batch) base[i] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) ws[0] = carry;
  }
  __syncthreads();
  for (int i = warp; i < batch; i += kWarps) {
    const SeqSpan s = seq_span(seq_lens, seq_starts, i, cumsum, block_size);
    const int nblk = (s.len + block_size - 1) / block_size;
    const int32_t *row = block_tables + (int64_t)i * max_blocks;
    const int first = base[i];
    int carry = 0, bad = 0;
    for (int j0 = 0; j0 < max_blocks; j0 += 32) {
      const int j = j0 + lane;
      const int n = j < nblk ? block_rows(row, s, j, max_blocks, block_size, num_blocks, &bad) : 0;
      const int incl = warp_inclusive_scan(n, lane);
      if (j < max_blocks) dest[(int64_t)i * max_blocks + j] = n > 0 ? first + carry + incl - n : -1;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
}

// V = copy granule (16, 2 or 1 bytes); rows are counted in granules.
template <typename V, int UNROLL>
__global__ void __launch_bounds__(kPclThreads)
pcl_copy_kernel(const V *__restrict__ key_cache, const V *__restrict__ value_cache,
                const int32_t *__restrict__ block_tables, const int32_t *__restrict__ seq_lens,
                const int32_t *__restrict__ seq_starts, V *__restrict__ key_out, V *__restrict__ value_out,
                int batch, int max_blocks, int block_size, int cumsum, int64_t k_row, int64_t v_row,
                int64_t sum_tokens, const int32_t *ws, int32_t *oob_count) {
  const bool is_v = blockIdx.y != 0;
  const int64_t row = is_v ? v_row : k_row;
  const V *cache = is_v ? value_cache : key_cache;
  V *out = is_v ? value_out : key_out;
  const int pairs = batch * max_blocks;
  // everything above is independent of the offsets kernel; its results are read below
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if ((int)blockIdx.x >= pairs) {
    // rows no block was gathered into (only when block ids were negative or out of range)
    const int64_t begin = (int64_t)__ldcg(ws) * row, end = sum_tokens * row;
    const int z = blockIdx.x - pairs;
    for (int64_t u = begin + (int64_t)z * kPclThreads + threadIdx.x; u < end; u += (int64_t)kPclZeroCtas * kPclThreads)
      pcl_st<V>(out + u, pcl_zero<V>());
    return;
  }
  const int32_t *dest = ws + kPclHeaderWords + batch;
  const int d = __ldcg(dest + blockIdx.x);  // written by the grid just waited for: read through L2
  if (d < 0) return;
  const int i = blockIdx.x / max_blocks, j = blockIdx.x - i * max_blocks;
  const SeqSpan s = seq_span(seq_lens, seq_starts, i, cumsum, block_size);
  const int id = __ldg(block_tables + (int64_t)i * max_blocks + s.off + j);
  int n = min(block_size, s.len - j * block_size);
  if ((int64_t)d + n > sum_tokens) {  // the output is shorter than the lengths say: never write past it
    if (threadIdx.x == 0 && oob_count != nullptr) atomicAdd(oob_count, 1);
    n = (int)max((int64_t)0, sum_tokens - d);
  }
  const V *src = cache + (int64_t)id * block_size * row;
  V *dst = out + (int64_t)d * row;
  const int64_t cnt = (int64_t)n * row;
  for (int64_t c0 = threadIdx.x; c0 < cnt; c0 += (int64_t)kPclThreads * UNROLL) {
    V r[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t c = c0 + (int64_t)u * kPclThreads;
      if (c < cnt) r[u] = pcl_ld<V>(src + c);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t c = c0 + (int64_t)u * kPclThreads;
      if (c < cnt) pcl_st<V>(dst + c, r[u]);
    }
  }
}

template <typename V, int UNROLL>
cudaError_t launch_copy(const void *kc, const void *vc, const int32_t *tables, const int32_t *lens,
                        const int32_t *starts, void *ko, void *vo, int batch, int max_blocks, int block_size,
                        int cumsum, int64_t k_row_bytes, int64_t v_row_bytes, int64_t sum_tokens,
                        const int32_t *ws, int32_t *oob_count, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(batch * max_blocks + kPclZeroCtas), 2, 1);
  cfg.blockDim = dim3(kPclThreads, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int64_t k_row = k_row_bytes / (int64_t)sizeof(V), v_row = v_row_bytes / (int64_t)sizeof(V);
  return cudaLaunchKernelEx(&cfg, pcl_copy_kernel<V, UNROLL>, (const V *)kc, (const V *)vc, tables, lens, starts,
                            (V *)ko, (V *)vo, batch, max_blocks, block_size, cumsum, k_row, v_row, sum_tokens, ws,
                            oob_count);
}

}  // namespace
}  // namespace msco

using namespace msco;

extern "C" size_t msco_paged_cache_load_workspace_bytes(int32_t batch, int32_t max_blocks_per_seq) {
  if (batch < 0 || max_blocks_per_seq < 0) return 0;
  return ((size_t)kPclHeaderWords + (size_t)batch + (size_t)batch * (size_t)max_blocks_per_seq) * sizeof(int32_t);
}

extern "C" int msco_paged_cache_load(const void *key_cache, const void *value_cache, const int32_t *block_tables,
                                     const int32_t *seq_lens, const int32_t *seq_starts, void *key_out,
                                     void *value_out, int32_t batch, int32_t max_blocks_per_seq,
                                     int32_t block_size, int32_t num_blocks, int64_t k_row_bytes,
                                     int64_t v_row_bytes, int64_t sum_tokens, int32_t seq_lens_cumsum,
                                     void *workspace, size_t workspace_bytes, int32_t *oob_count, void *stream) {
  if (batch < 0 || max_blocks_per_seq < 0 || block_size < 0 || num_blocks < 0 || k_row_bytes < 0 ||
      v_row_bytes < 0 || sum_tokens < 0)
    return fail(MSCO_ERR_INVALID_ARG, "paged_cache_load: negative size");
  // zero-sized inputs: the reference skips execution (paged_cache_load_graph.cc:80-97)
  if (batch == 0 || max_blocks_per_seq == 0 || block_size == 0 || num_blocks == 0 || sum_tokens == 0 ||
      (k_row_bytes == 0 && v_row_bytes == 0))
    return MSCO_OK;
  if (key_cache == nullptr || value_cache == nullptr || block_tables == nullptr || seq_lens == nullptr ||
      key_out == nullptr || value_out == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "paged_cache_load: caches, block_tables, seq_lens and outputs must not be NULL");
  if ((int64_t)batch * max_blocks_per_seq > (int64_t)0x7fffff00)
    return fail(MSCO_ERR_INVALID_ARG, "paged_cache_load: block table too large");
  if (sum_tokens > (int64_t)INT32_MAX)
    return fail(MSCO_ERR_INVALID_ARG, "paged_cache_load: too many tokens");
  const size_t need = msco_paged_cache_load_workspace_bytes(batch, max_blocks_per_seq);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 3) != 0)
    return fail(MSCO_ERR_INVALID_ARG, "paged_cache_load: workspace too small (%zu < %zu)", workspace_bytes, need);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t *ws = static_cast<int32_t *>(workspace);
  pcl_offsets_kernel<<<1, kPclOffsetThreads, 0, st>>>(block_tables, seq_lens, seq_starts, batch, max_blocks_per_seq,
                                                      block_size, num_blocks, seq_lens_cumsum ? 1 : 0, ws, oob_count);
  MSCO_CUDA_CHECK(cudaGetLastError());
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(key_cache) | reinterpret_cast<uintptr_t>(value_cache) |
                         reinterpret_cast<uintptr_t>(key_out) | reinterpret_cast<uintptr_t>(value_out);
  const int cs = seq_lens_cumsum ? 1 : 0;
  cudaError_t e;
  if (k_row_bytes % 16 == 0 && v_row_bytes % 16 == 0 && (ptrs & 15) == 0) {
    e = launch_copy<uint4, 8>(key_cache, value_cache, block_tables, seq_lens, seq_starts, key_out, value_out, batch,
                              max_blocks_per_seq, block_size, cs, k_row_bytes, v_row_bytes, sum_tokens, ws,
                              oob_count, st);
  } else if (k_row_bytes % 2 == 0 && v_row_bytes % 2 == 0 && (ptrs & 1) == 0) {
    e = launch_copy<uint16_t, 8>(key_cache, value_cache, block_tables, seq_lens, seq_starts, key_out, value_out,
                                 batch, max_blocks_per_seq, block_size, cs, k_row_bytes, v_row_bytes, sum_tokens, ws,
                                 oob_count, st);
  } else {
    e = launch_copy<uint8_t, 8>(key_cache, value_cache, block_tables, seq_lens, seq_starts, key_out, value_out,
                                batch, max_blocks_per_seq, block_size, cs, k_row_bytes, v_row_bytes, sum_tokens, ws,
                                oob_count, st);
  }
  MSCO_CUDA_CHECK(e);
  return MSCO_OK;
}
