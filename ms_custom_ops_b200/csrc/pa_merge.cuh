// Merge of the split-KV partials of one output row (head_dim 64 / 128 / 256), shared by the reduce kernel and by
// the attention kernel's own epilogue so that both produce the same bits.
//
// The partials hold, per split s, the running maximum m_s (log2 domain), the running sum l_s and the
// un-normalised output O_s.  In split order:
//   M = max_s m_s,   out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s
// which is the log-sum-exp merge of the reference's fa_update golden
// (tests/st/test_asd_faupdate.py:34-59) written for un-normalised partials.
#pragma once

#include "msco_common.cuh"
#include "pa_params.h"

namespace msco {

__device__ __forceinline__ float merge_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// One warp merges output row `row` (= query token * num_q_heads + hq): `ns` >= 2 splits whose partial rows
// are base, base + 1, ..., base + ns - 1.
// D = head_dim (64, 128 or 256): a lane owns D / 32 consecutive columns.
// All loads bypass L1 (ld.global.cg): the partials may have been written by other SMs of the same grid.
// PREFETCH = 0: the partial rows are loaded inside the accumulation loop (16-fold unrolled): the form for
// the attention kernel's own epilogue, where registers are short.  PREFETCH = 16 or 32 (the merge kernel):
// the rows are requested in batches of that many before the first is used, and the first batch goes out
// before anything else -- it does not depend on the maxima of pass 1 -- so a row of up to PREFETCH splits
// costs two dependent round trips (maxima, then nothing: the rows are already on their way) instead of
// three or more.  Same accumulation order in every form: the same bits.
template <typename TQ, int D, int PREFETCH = 0>
__device__ __forceinline__ void merge_row(const PaParams &p, int64_t row, int hq, int ns, int base, int lane) {
  static_assert(D == 64 || D == 128 || D == 256, "head_dim 64, 128 or 256");
  static_assert(PREFETCH == 0 || PREFETCH == 16 || PREFETCH == 32, "batches of 16 or 32 rows");
  constexpr int kCols = D / 32;  // columns per lane: 2, 4 or 8
  constexpr int kBatch = PREFETCH > 0 ? PREFETCH : 1;
  constexpr float kNegBig = -1.0e30f;
  constexpr float kLn2f = 0.6931471805599453f;
  const int64_t hq_stride = p.num_q_heads;
  [[maybe_unused]] float vb[kBatch][kCols];
  [[maybe_unused]] auto load_batch = [&](int s_first, int cnt) {  // partial rows s_first .. s_first + cnt - 1
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (u < cnt) {
        const float *src = p.part_o + ((int64_t)(base + s_first + u) * hq_stride + hq) * D + lane * kCols;
        if (kCols == 2) {
          const float2 t = __ldcg(reinterpret_cast<const float2 *>(src));
          vb[u][0] = t.x; vb[u][1] = t.y;
        } else {
#pragma unroll
          for (int c = 0; c < kCols; c += 4) {
            const float4 t = __ldcg(reinterpret_cast<const float4 *>(src + c));
            vb[u][c] = t.x; vb[u][c + 1] = t.y; vb[u][c + 2] = t.z; vb[u][c + 3] = t.w;
          }
        }
      }
    }
  };
  if constexpr (PREFETCH > 0) load_batch(0, min(PREFETCH, ns));
  // pass 1: M = max_s m_s (lanes stride over the splits)
  float M = kNegBig;
  for (int s = lane; s < ns; s += 32) M = fmaxf(M, __ldcg(p.part_ml + ((int64_t)(base + s) * hq_stride + hq) * 2));
  M = merge_warp_max(M);
  const int kvh = hq / p.group;
  float L = 0.f;
  float acc[kCols];
#pragma unroll
  for (int c = 0; c < kCols; ++c) acc[c] = 0.f;
  // splits in blocks of 32 (weights in registers), accumulated in split order: bit-reproducible
  for (int s0 = 0; s0 < ns; s0 += 32) {
    float f_mine = 0.f, l_mine = 0.f;
    if (s0 + lane < ns) {
      const float2 ml =
          __ldcg(reinterpret_cast<const float2 *>(p.part_ml + ((int64_t)(base + s0 + lane) * hq_stride + hq) * 2));
      f_mine = exp2f(ml.x - M);
      l_mine = ml.y;
    }
    const int cnt = min(32, ns - s0);
    if constexpr (PREFETCH > 0) {
      for (int j0 = 0; j0 < cnt; j0 += PREFETCH) {
        const int n = min(PREFETCH, cnt - j0);
        if (s0 + j0 > 0) load_batch(s0 + j0, n);  // (the first batch is on its way since the start)
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          if (u < n) {  // warp-uniform
            const float f = __shfl_sync(0xffffffffu, f_mine, j0 + u);
            const float lj = __shfl_sync(0xffffffffu, l_mine, j0 + u);
            L = fmaf(lj, f, L);
#pragma unroll
            for (int c = 0; c < kCols; ++c) acc[c] = fmaf(vb[u][c], f, acc[c]);
          }
        }
      }
    } else {
      // 16 partial rows in flight per lane: the loop is a chain of L2 round trips otherwise
#pragma unroll 16
      for (int j = 0; j < cnt; ++j) {
        const float f = __shfl_sync(0xffffffffu, f_mine, j);
        const float lj = __shfl_sync(0xffffffffu, l_mine, j);
        const float *src = p.part_o + ((int64_t)(base + s0 + j) * hq_stride + hq) * D + lane * kCols;
        float v[kCols];
        if (kCols == 2) {
          const float2 t = __ldcg(reinterpret_cast<const float2 *>(src));
          v[0] = t.x; v[1] = t.y;
        } else {
#pragma unroll
          for (int c = 0; c < kCols; c += 4) {
            const float4 t = __ldcg(reinterpret_cast<const float4 *>(src + c));
            v[c] = t.x; v[c + 1] = t.y; v[c + 2] = t.z; v[c + 3] = t.w;
          }
        }
        L = fmaf(lj, f, L);
#pragma unroll
        for (int c = 0; c < kCols; ++c) acc[c] = fmaf(v[c], f, acc[c]);
      }
    }
  }
  const float inv = 1.f / L;
  float r[kCols];
#pragma unroll
  for (int c = 0; c < kCols; ++c) r[c] = acc[c] * inv;
  if (p.v_descale != nullptr) {
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
      const int d = lane * kCols + c;
      if (p.v_offset != nullptr) r[c] += (float)__ldg(p.v_offset + kvh * D + d);
      r[c] *= __ldg(p.v_descale + kvh * D + d);
    }
  }
  TQ *dst = static_cast<TQ *>(p.out) + row * D + lane * kCols;
  if (kCols == 2) {
    *reinterpret_cast<uint32_t *>(dst) = pack2<TQ>(r[0], r[1]);
  } else {
#pragma unroll
    for (int c = 0; c < kCols; c += 4) {
      uint2 pk;
      pk.x = pack2<TQ>(r[c], r[c + 1]);
      pk.y = pack2<TQ>(r[c + 2], r[c + 3]);
      *reinterpret_cast<uint2 *>(dst + c) = pk;
    }
  }
  if (lane == 0 && p.lse != nullptr) p.lse[row] = (M + log2f(L)) * kLn2f;
}

}  // namespace msco
