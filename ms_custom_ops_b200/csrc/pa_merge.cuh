// Merge of the split-KV partials of one output row (head_dim 128), shared by the reduce kernel and by
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

// One warp merges row (b, hq): `ns` >= 2 splits whose partial rows start at part index `base`.
// All loads bypass L1 (ld.global.cg): the partials may have been written by other SMs of the same grid.
template <typename TQ>
__device__ __forceinline__ void merge_row_d128(const PaParams &p, int b, int hq, int ns, int base, int lane) {
  constexpr float kNegBig = -1.0e30f;
  constexpr float kLn2f = 0.6931471805599453f;
  const int64_t hq_stride = p.num_q_heads;
  const int64_t row = (int64_t)b * p.num_q_heads + hq;
  // pass 1: M = max_s m_s (lanes stride over the splits)
  float M = kNegBig;
  for (int s = lane; s < ns; s += 32) M = fmaxf(M, __ldcg(p.part_ml + ((int64_t)(base + s) * hq_stride + hq) * 2));
  M = merge_warp_max(M);
  const int kvh = hq / p.group;
  float L = 0.f;
  // lane owns 4 consecutive head-dim columns; splits in blocks of 32 (weights in registers)
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < ns; s0 += 32) {
    float f_mine = 0.f, l_mine = 0.f;
    if (s0 + lane < ns) {
      const float2 ml =
          __ldcg(reinterpret_cast<const float2 *>(p.part_ml + ((int64_t)(base + s0 + lane) * hq_stride + hq) * 2));
      f_mine = exp2f(ml.x - M);
      l_mine = ml.y;
    }
    const int cnt = min(32, ns - s0);
#pragma unroll 8
    for (int j = 0; j < cnt; ++j) {  // split order: bit-reproducible
      const float f = __shfl_sync(0xffffffffu, f_mine, j);
      const float lj = __shfl_sync(0xffffffffu, l_mine, j);
      const float4 v =
          __ldcg(reinterpret_cast<const float4 *>(p.part_o + ((int64_t)(base + s0 + j) * hq_stride + hq) * 128) + lane);
      L = fmaf(lj, f, L);
      acc.x = fmaf(v.x, f, acc.x); acc.y = fmaf(v.y, f, acc.y);
      acc.z = fmaf(v.z, f, acc.z); acc.w = fmaf(v.w, f, acc.w);
    }
  }
  const float inv = 1.f / L;
  float r0 = acc.x * inv, r1 = acc.y * inv, r2 = acc.z * inv, r3 = acc.w * inv;
  if (p.v_descale != nullptr) {
    const float4 vs = __ldg(reinterpret_cast<const float4 *>(p.v_descale + kvh * 128) + lane);
    if (p.v_offset != nullptr) {
      const int4 vo = __ldg(reinterpret_cast<const int4 *>(p.v_offset + kvh * 128) + lane);
      r0 += (float)vo.x; r1 += (float)vo.y; r2 += (float)vo.z; r3 += (float)vo.w;
    }
    r0 *= vs.x; r1 *= vs.y; r2 *= vs.z; r3 *= vs.w;
  }
  uint2 pk;
  pk.x = pack2<TQ>(r0, r1);
  pk.y = pack2<TQ>(r2, r3);
  *reinterpret_cast<uint2 *>(static_cast<TQ *>(p.out) + row * 128 + lane * 4) = pk;
  if (lane == 0 && p.lse != nullptr) p.lse[row] = (M + log2f(L)) * kLn2f;
}

}  // namespace msco
