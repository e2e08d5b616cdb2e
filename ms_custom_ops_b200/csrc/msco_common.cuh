// Shared device/host helpers for libmsco_b200.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "msco_b200.h"

namespace msco {

// ---- host-side error plumbing --------------------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define MSCO_CUDA_CHECK(expr)                                                            \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      return ::msco::fail(MSCO_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                          cudaGetErrorString(_e), __FILE__, __LINE__);                   \
    }                                                                                    \
  } while (0)

inline int dtype_size(int dt) {
  switch (dt) {
    case MSCO_DTYPE_F16:
    case MSCO_DTYPE_BF16: return 2;
    case MSCO_DTYPE_I8: return 1;
    case MSCO_DTYPE_F32:
    case MSCO_DTYPE_I32: return 4;
    case MSCO_DTYPE_I64: return 8;
    default: return 0;
  }
}

// ---- device plan layout (int32 words at the start of the PA workspace) ----
// [0] unused  [1] nseq  [2] total_items  [3] total_parts  [4] batch  [5] items_per_split
// [6] 1 when the entries carry query-token ranges (multi-token queries)  [7] pad
// then: item_base[nseq+1], seq_idx[nseq], seq_len[nseq], chunk[nseq], nsplit[nseq], part_base[nseq],
//       b_nsplit[batch], b_part_base[batch], and with [6] set: qtok0[nseq], qntok[nseq]
// An "entry" (nseq of them) is one sequence of a decode batch, or -- multi-token queries -- a run of up to
// rows_per_item / group consecutive query tokens of one sequence, whose q rows are stacked into one item.
constexpr int kPlanHeaderWords = 8;
constexpr int kStatusTimeout = MSCO_ERR_TIMEOUT;
constexpr int kStatusOob = MSCO_ERR_OOB;

struct PlanView {
  const int32_t *base;
  int nseq, total_items, total_parts, batch, multi_token;
  const int32_t *item_base, *seq_idx, *seq_len, *chunk, *nsplit, *part_base, *b_nsplit, *b_part_base;
  const int32_t *qtok0, *qntok;  // multi-token queries only
};

__host__ __device__ inline PlanView make_plan_view(const int32_t *w) {
  PlanView v;
  v.base = w;
  v.nseq = w[1];
  v.total_items = w[2];
  v.total_parts = w[3];
  v.batch = w[4];
  v.multi_token = w[6];
  const int32_t *p = w + kPlanHeaderWords;
  v.item_base = p; p += v.nseq + 1;
  v.seq_idx = p; p += v.nseq;
  v.seq_len = p; p += v.nseq;
  v.chunk = p; p += v.nseq;
  v.nsplit = p; p += v.nseq;
  v.part_base = p; p += v.nseq;
  v.b_nsplit = p; p += v.batch;
  v.b_part_base = p; p += v.batch;
  v.qtok0 = p; p += v.nseq;
  v.qntok = p;
  return v;
}

// One unit of attention work: the q rows [row0, row0+nrows) of kv head `kvh`
// of sequence `b` against KV tokens [tok0, tok1).
struct WorkItem {
  int b, kvh, row0, nrows, tok0, tok1, nsplit, part;
  int grp;    // index of the (sequence, kv head, q-row block) group: one arrival counter per group
  int part0;  // partial row of the group's first token and first split: token t, split s -> part0 + t * nsplit + s
  int qtok0;  // first query token (row of query / out) of the item; the sequence index b for a decode batch
  int ntok;   // query tokens stacked into the item (1 for a decode batch): q row r is token r / group
};

#ifdef __CUDACC__
// Error report of a kernel: the code and the epoch of the launch that hit it (the host compares
// the epoch, so the words never need clearing).
__device__ __forceinline__ void report_status(int32_t *status, uint32_t epoch, int code) {
  status[1] = (int32_t)epoch;
  atomicExch(status, code);
}

// ---- dtype conversion ------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<int8_t>(int8_t v) { return (float)v; }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// pack two floats into one 32-bit register of 16-bit values (lo = a, hi = b)
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

// ---- work-item decode (serial; any thread) ---------------------------------
// `item_base_smem`, when given, is a shared-memory copy of pv.item_base[0 .. nseq]: the binary
// search then costs no global-memory round trips (each would be ~0.6 us of dependent latency).
__device__ __forceinline__ WorkItem decode_item(const PlanView &pv, int t, int num_kv_heads, int g,
                                                int rows_per_item, const int32_t *item_base_smem = nullptr) {
  int lo = 0, hi = pv.nseq;  // find s with item_base[s] <= t < item_base[s+1]
  if (item_base_smem != nullptr) {
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (item_base_smem[mid] <= t) lo = mid; else hi = mid;
    }
  } else {
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (__ldg(pv.item_base + mid) <= t) lo = mid; else hi = mid;
    }
  }
  const int s = lo;
  const int nqb = (g + rows_per_item - 1) / rows_per_item;
  const int nps = num_kv_heads * nqb;
  const int r = t - (item_base_smem != nullptr ? item_base_smem[s] : __ldg(pv.item_base + s));
  const int split = r / nps, hh = r - split * nps;
  WorkItem w;
  w.kvh = hh / nqb;
  const int qb = hh - w.kvh * nqb;
  w.row0 = qb * rows_per_item;
  w.nrows = min(rows_per_item, g - w.row0);
  w.b = __ldg(pv.seq_idx + s);
  const int len = __ldg(pv.seq_len + s), c = __ldg(pv.chunk + s);
  w.nsplit = __ldg(pv.nsplit + s);
  w.tok0 = split * c;
  w.tok1 = min(len, w.tok0 + c);
  w.part0 = __ldg(pv.part_base + s);
  w.grp = s * nps + hh;
  w.qtok0 = w.b;
  w.ntok = 1;
  if (pv.multi_token) {
    w.qtok0 = __ldg(pv.qtok0 + s);
    w.ntok = __ldg(pv.qntok + s);
    if (w.ntok > 1) w.nrows = w.ntok * g;  // one row block holds the whole run (the planner sees to it)
  }
  w.part = w.part0 + split;  // of the item's first token
  return w;
}

// ---- PTX wrappers: mbarrier, TMA, ldmatrix, mma ----------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a
// hardware-defined short time), so a lost arrival can never hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 24)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// Tiled TMA load of a 3-D box (no multicast), completion on an mbarrier.
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tmap, int x, int y, int z,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
// Untiled bulk copy global -> shared (16-byte aligned addresses, size % 16 == 0).
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// D(16x8,f32) += A(16x16) * B(16x8); A/B fp16 or bf16
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
#endif  // __CUDACC__

}  // namespace msco
