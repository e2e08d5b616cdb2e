// Paged-attention decode for B200: persistent TMA-fed split-KV kernel.
//
// HBM-bound: every K/V byte of the context is read exactly once.  One
// persistent CTA per SM walks a static round-robin list of work items
// (sequence, kv head, q-row block, KV split).  A producer warp streams
// 128-token K and V tiles of the paged cache into a ring of shared-memory
// stages with tiled TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no
// multicast) that complete on mbarriers; the stream runs ahead across item
// boundaries, so the memory pipe never drains between items.  Eight consumer
// warps each own 16 of the tile's 128 tokens and keep an independent online
// softmax state (m, l, O) for the padded GQA group (M = 16 rows):
//   S = Q K^T  and  O += P V  as mma.sync m16n8k16 micro-tiles, fp32 accumulate,
//   K fragments by ldmatrix, V fragments by ldmatrix.trans,
//   int8 KV: bytes -> fp16 in registers (xor 0x80, byte-permute into
//   0x6400|u = 1024+u, subtract 1152), k_descale folded into Q once per item,
//   v_descale / v_offset applied once to the output.
// At the end of an item the eight states are merged through shared memory and
// either written as the final output (one split) or as an fp32 partial
// (m, l, O) for the reduce kernel.
//
// Algorithmic bytes per context token: 2 * head_dim * sizeof(kv) per kv head.
#include <cuda.h>

#include <type_traits>

#include "msco_common.cuh"
#include "pa_params.h"

namespace msco {
namespace {

constexpr int kD = 128;               // head_dim of this kernel
constexpr int kTile = 128;            // tokens per tile
constexpr int kConsumerWarps = 8;     // 16 tokens of the tile each
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kMergeStride = 136;     // floats per merged row (bank-conflict padding)
constexpr int kQSlotBytes = 16 * kD * 2;
constexpr float kNeg = -1.0e30f;
constexpr uint32_t kWaitLimit = 1u << 24;

template <bool KV8, bool G16> struct Cfg {
  static constexpr int kRowBytes = KV8 ? kD : 2 * kD;       // one token row of one head
  static constexpr int kStageBytes = kTile * kRowBytes;     // 16 KB (int8) / 32 KB (16-bit)
  static constexpr int kStages = KV8 ? 8 : (G16 ? 4 : 5);
  static constexpr int kRows = G16 ? 16 : 8;
  static constexpr int kMergeBytes = kConsumerWarps * kRows * kMergeStride * 4;
  static constexpr int kOffQ = kStages * kStageBytes;
  static constexpr int kOffMerge = kOffQ + 2 * kQSlotBytes;
  static constexpr int kOffMl = kOffMerge + kMergeBytes;           // [warp][16][2] floats
  static constexpr int kOffDesc = kOffMl + kConsumerWarps * 16 * 2 * 4;  // 2 x WorkItem (8 ints)
  static constexpr int kOffBar = kOffDesc + 2 * 8 * 4;             // mbarriers
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static constexpr int kDynSmem = kSmemBytes + 1024;               // slack for 1024-byte alignment
};

// int8x4 (already xor-ed with 0x80808080) -> two fp16x2 registers holding the
// signed values of byte pairs (sel picks which bytes).
__device__ __forceinline__ uint32_t bytes_to_half2(uint32_t x, uint32_t sel) {
  uint32_t h;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(h) : "r"(x), "r"(0x64646464u), "r"(sel));
  // h = {1024 + u_lo, 1024 + u_hi} as fp16x2; remove 1024 + 128
  const uint32_t bias = 0x64806480u;  // fp16 1152.0 twice
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(h), "r"(bias));
  return r;
}

template <typename T, bool KV8, bool G16>
__global__ void __launch_bounds__(kThreads, 1)
pa_tma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, PaParams p) {
  using C = Cfg<KV8, G16>;
  // fp16 arithmetic for int8 KV (integers up to 255 are exact in fp16, not in bf16)
  using MT = typename std::conditional<KV8, __half, T>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C::kOffBar);
  uint64_t *full = bars, *empty = bars + C::kStages;
  uint64_t *qfull = bars + 2 * C::kStages, *qempty = qfull + 2;
  int *desc = reinterpret_cast<int *>(smem + C::kOffDesc);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kConsumerWarps);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qfull[i], 1);
      mbar_init(&qempty[i], kConsumerWarps);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const PlanView pv = make_plan_view(p.plan);
  const int total = pv.total_items;
  const int rpi = C::kRows;

  if (warp == kConsumerWarps) {
    // ======================= producer warp =======================
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
    }
    uint32_t st = 0, ph = 0;
    const int bs = p.block_size;
    const int bpt = kTile / bs;  // cache blocks per tile
    int qi = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++qi) {
      const WorkItem w = decode_item(pv, t, p.num_kv_heads, p.group, rpi);
      const int qs = qi & 1;
      const uint32_t qph = (qi >> 1) & 1;
      if (!mbar_wait(&qempty[qs], qph ^ 1, kWaitLimit)) {
        atomicExch(p.plan, kStatusTimeout);
        return;
      }
      if (lane == 0) {
        int *d = desc + qs * 8;
        d[0] = w.b; d[1] = w.kvh; d[2] = w.row0; d[3] = w.nrows;
        d[4] = w.tok0; d[5] = w.tok1; d[6] = w.nsplit; d[7] = w.part;
        const uint32_t qbytes = (uint32_t)w.nrows * kD * 2;
        mbar_arrive_expect_tx(&qfull[qs], qbytes);
        const char *qsrc = static_cast<const char *>(p.q) +
                           ((int64_t)w.b * p.num_q_heads + w.kvh * p.group + w.row0) * (kD * 2);
        bulk_load(smem + C::kOffQ + qs * kQSlotBytes, qsrc, qbytes, &qfull[qs]);
      }
      const int ntok = w.tok1 - w.tok0;
      const int nblk_item = (ntok + bs - 1) / bs;
      const int32_t *trow = p.block_tables + (int64_t)w.b * p.max_blocks_per_seq + w.tok0 / bs;
      int tile = 0;
      for (int blk0 = 0; blk0 < nblk_item; blk0 += 32) {
        // 32 block ids per batch, one per lane; a batch holds whole tiles (bpt divides 32)
        int my_id = 0;
        if (blk0 + lane < nblk_item) {
          my_id = __ldg(trow + blk0 + lane);
          if (my_id < 0 || my_id >= p.num_blocks) {
            atomicExch(p.plan, kStatusOob);
            my_id = 0;  // stay inside the cache; the result of this item is undefined
          }
        }
        const int nblk_batch = min(32, nblk_item - blk0);
        for (int jb = 0; jb < nblk_batch; jb += bpt, ++tile) {
          const int nv = min(kTile, ntok - tile * kTile);  // valid tokens of this tile
          const int nb_tile = (nv + bs - 1) / bs;
#pragma unroll 1
          for (int op = 0; op < 2; ++op) {
            if (!mbar_wait(&empty[st], ph ^ 1, kWaitLimit)) {
              atomicExch(p.plan, kStatusTimeout);
              return;
            }
            uint8_t *dst = smem + st * C::kStageBytes;
            if (lane == 0) mbar_arrive_expect_tx(&full[st], (uint32_t)(nb_tile * bs * C::kRowBytes));
            for (int j = 0; j < nb_tile; ++j) {
              const int id = __shfl_sync(0xffffffffu, my_id, jb + j);
              if (lane == 0) {
                const CUtensorMap *tm = op == 0 ? &tm_k : &tm_v;
                const int z = id * bs;
                if (KV8) {
                  tma_load_3d(dst + j * bs * 128, tm, 0, w.kvh, z, &full[st]);
                } else {
                  tma_load_3d(dst + j * bs * 128, tm, 0, w.kvh, z, &full[st]);
                  tma_load_3d(dst + kTile * 128 + j * bs * 128, tm, 64, w.kvh, z, &full[st]);
                }
              }
            }
            if (++st == C::kStages) { st = 0; ph ^= 1; }
          }
        }
      }
    }
    return;
  }

  // ======================= consumer warps =======================
  const int gid = lane >> 2, q4 = lane & 3;
  const int t0 = warp * 16;                 // this warp's token rows inside a tile
  const int mat = lane >> 3, mr = lane & 7; // ldmatrix: matrix id and row supplied by this lane
  const uint32_t stage0 = smem_u32(smem);
  float *mbuf = reinterpret_cast<float *>(smem + C::kOffMerge);
  float2 *mlbuf = reinterpret_cast<float2 *>(smem + C::kOffMl);
  // per-lane byte offsets of the ldmatrix rows (swizzle: 16-byte chunk ^= row & 7)
  const uint32_t k_row_off = (uint32_t)(t0 + (mat >> 1) * 8 + mr) * 128u;  // K: matrices 2,3 = tokens +8
  const uint32_t v_row_off = (uint32_t)(t0 + (mat & 1) * 8 + mr) * 128u;   // V: matrices 1,3 = tokens +8
  const int tid = threadIdx.x;

  uint32_t st = 0, ph = 0;
  int qi = 0;
  for (int t = blockIdx.x; t < total; t += gridDim.x, ++qi) {
    const int qs = qi & 1;
    const uint32_t qph = (qi >> 1) & 1;
    if (!mbar_wait(&qfull[qs], qph, kWaitLimit)) {
      atomicExch(p.plan, kStatusTimeout);
      return;
    }
    const int *dsc = desc + qs * 8;
    const int b = dsc[0], kvh = dsc[1], row0 = dsc[2], nrows = dsc[3];
    const int tok0 = dsc[4], tok1 = dsc[5], nsplit = dsc[6], part = dsc[7];

    // ---- Q fragments (A operand, 16 x 128), rows >= nrows are zero ----
    uint32_t qa[8][4];
    {
      const T *qsm = reinterpret_cast<const T *>(smem + C::kOffQ + qs * kQSlotBytes);
      const bool vlo = gid < nrows, vhi = G16 && (gid + 8 < nrows);
      const T *qlo = qsm + gid * kD, *qhi = qsm + (gid + 8) * kD;
      if (!KV8) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int c = 16 * ks + 2 * q4;
          qa[ks][0] = vlo ? *reinterpret_cast<const uint32_t *>(qlo + c) : 0u;
          qa[ks][1] = vhi ? *reinterpret_cast<const uint32_t *>(qhi + c) : 0u;
          qa[ks][2] = vlo ? *reinterpret_cast<const uint32_t *>(qlo + c + 8) : 0u;
          qa[ks][3] = vhi ? *reinterpret_cast<const uint32_t *>(qhi + c + 8) : 0u;
        }
      } else {
        // int8 K: the contraction index inside each 16-wide group is permuted so that the four
        // bytes a lane gets from ldmatrix (d = 16ks + 4q4 .. +3) are its two B registers; Q uses
        // the same permutation.  k_descale is folded into Q here.
        const float *ksc = p.k_descale + kvh * kD;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int c = 16 * ks + 4 * q4;
          const float4 sc = __ldg(reinterpret_cast<const float4 *>(ksc + c));
          float lo[4] = {0.f, 0.f, 0.f, 0.f}, hi[4] = {0.f, 0.f, 0.f, 0.f};
          if (vlo) {
            lo[0] = to_f32<T>(qlo[c]) * sc.x; lo[1] = to_f32<T>(qlo[c + 1]) * sc.y;
            lo[2] = to_f32<T>(qlo[c + 2]) * sc.z; lo[3] = to_f32<T>(qlo[c + 3]) * sc.w;
          }
          if (vhi) {
            hi[0] = to_f32<T>(qhi[c]) * sc.x; hi[1] = to_f32<T>(qhi[c + 1]) * sc.y;
            hi[2] = to_f32<T>(qhi[c + 2]) * sc.z; hi[3] = to_f32<T>(qhi[c + 3]) * sc.w;
          }
          qa[ks][0] = pack2<__half>(lo[0], lo[1]);
          qa[ks][1] = pack2<__half>(hi[0], hi[1]);
          qa[ks][2] = pack2<__half>(lo[2], lo[3]);
          qa[ks][3] = pack2<__half>(hi[2], hi[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&qempty[qs]);

    float m_lo = kNeg, m_hi = kNeg, l_lo = 0.f, l_hi = 0.f;  // l_*: this thread's share of the row sum
    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    const int ntiles = (tok1 - tok0 + kTile - 1) / kTile;
    for (int ti = 0; ti < ntiles; ++ti) {
      const int nv = min(kTile, tok1 - tok0 - ti * kTile);
      const bool active = t0 < nv;  // warp-uniform: any of this warp's 16 tokens valid
      // ---------------- S = Q K^T ----------------
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      if (!mbar_wait(&full[st], ph, kWaitLimit)) {
        atomicExch(p.plan, kStatusTimeout);
        return;
      }
      if (active) {
        const uint32_t kbase = stage0 + st * C::kStageBytes + k_row_off;
        if (!KV8) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t cc = (uint32_t)(2 * (ks & 3) + (mat & 1));
            const uint32_t addr = kbase + (uint32_t)(ks >> 2) * (kTile * 128) + ((cc ^ (uint32_t)mr) << 4);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(addr, b0, b1, b2, b3);
            mma16816<MT>(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
            mma16816<MT>(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t cc = (uint32_t)(2 * i + (mat & 1));
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(kbase + ((cc ^ (uint32_t)mr) << 4), r0, r1, r2, r3);
            r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
            mma16816<MT>(s[0], qa[2 * i][0], qa[2 * i][1], qa[2 * i][2], qa[2 * i][3],
                         bytes_to_half2(r0, 0x5140u), bytes_to_half2(r0, 0x5342u));
            mma16816<MT>(s[0], qa[2 * i + 1][0], qa[2 * i + 1][1], qa[2 * i + 1][2], qa[2 * i + 1][3],
                         bytes_to_half2(r1, 0x5140u), bytes_to_half2(r1, 0x5342u));
            mma16816<MT>(s[1], qa[2 * i][0], qa[2 * i][1], qa[2 * i][2], qa[2 * i][3],
                         bytes_to_half2(r2, 0x5140u), bytes_to_half2(r2, 0x5342u));
            mma16816<MT>(s[1], qa[2 * i + 1][0], qa[2 * i + 1][1], qa[2 * i + 1][2], qa[2 * i + 1][3],
                         bytes_to_half2(r3, 0x5140u), bytes_to_half2(r3, 0x5342u));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
      if (++st == C::kStages) { st = 0; ph ^= 1; }

      // ---------------- online softmax ----------------
      uint32_t pa[4] = {0u, 0u, 0u, 0u};
      if (active) {
        const float c = p.scale_log2e;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[j][e] *= c;
        if (nv < t0 + 16) {  // tail: mask tokens at or beyond the end of the range
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (t0 + 8 * j + 2 * q4 + (e & 1) >= nv) s[j][e] = kNeg;
        }
        {
          float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float mnew = fmaxf(m_lo, mx);
          const float alpha = fast_exp2(m_lo - mnew);
          m_lo = mnew;
          const float p0 = fast_exp2(s[0][0] - mnew), p1 = fast_exp2(s[0][1] - mnew);
          const float p2 = fast_exp2(s[1][0] - mnew), p3 = fast_exp2(s[1][1] - mnew);
          l_lo = l_lo * alpha + (p0 + p1) + (p2 + p3);
          pa[0] = pack2<MT>(p0, p1);
          pa[2] = pack2<MT>(p2, p3);
          if (alpha != 1.f) {
#pragma unroll
            for (int i = 0; i < 16; ++i) { o[i][0] *= alpha; o[i][1] *= alpha; }
          }
        }
        if (G16) {
          float mx = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float mnew = fmaxf(m_hi, mx);
          const float alpha = fast_exp2(m_hi - mnew);
          m_hi = mnew;
          const float p0 = fast_exp2(s[0][2] - mnew), p1 = fast_exp2(s[0][3] - mnew);
          const float p2 = fast_exp2(s[1][2] - mnew), p3 = fast_exp2(s[1][3] - mnew);
          l_hi = l_hi * alpha + (p0 + p1) + (p2 + p3);
          pa[1] = pack2<MT>(p0, p1);
          pa[3] = pack2<MT>(p2, p3);
          if (alpha != 1.f) {
#pragma unroll
            for (int i = 0; i < 16; ++i) { o[i][2] *= alpha; o[i][3] *= alpha; }
          }
        }
      }

      // ---------------- O += P V ----------------
      if (!mbar_wait(&full[st], ph, kWaitLimit)) {
        atomicExch(p.plan, kStatusTimeout);
        return;
      }
      if (active) {
        uint8_t *vst = smem + st * C::kStageBytes;
        if (nv < t0 + 16) {
          // rows past the end of the range may hold anything (also NaN): zero them so that
          // 0 * garbage cannot reach the accumulators
          constexpr int kChunks = C::kRowBytes / 16;
          for (int idx = lane; idx < 16 * kChunks; idx += 32) {
            const int r = idx / kChunks, ch = idx - r * kChunks;
            if (t0 + r >= nv) {
              uint8_t *dst = KV8 ? vst + (t0 + r) * 128 + ch * 16
                                 : vst + (ch >> 3) * (kTile * 128) + (t0 + r) * 128 + (ch & 7) * 16;
              *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
          }
          fence_proxy_async();
          __syncwarp();
        }
        const uint32_t vbase = stage0 + st * C::kStageBytes + v_row_off;
        if (!KV8) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t c16 = (uint32_t)(2 * i + (mat >> 1));
            const uint32_t addr = vbase + (c16 >> 3) * (kTile * 128) + (((c16 & 7) ^ (uint32_t)mr) << 4);
            uint32_t v0, v1, v2, v3;
            ldmatrix_x4_trans(addr, v0, v1, v2, v3);
            mma16816<MT>(o[2 * i], pa[0], pa[1], pa[2], pa[3], v0, v1);
            mma16816<MT>(o[2 * i + 1], pa[0], pa[1], pa[2], pa[3], v2, v3);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t cc = (uint32_t)(2 * i + (mat >> 1));
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4_trans(vbase + ((cc ^ (uint32_t)mr) << 4), r0, r1, r2, r3);
            r0 ^= 0x80808080u; r1 ^= 0x80808080u; r2 ^= 0x80808080u; r3 ^= 0x80808080u;
            // bytes 0,2 = even column of the 16-wide group, bytes 1,3 = odd column
            mma16816<MT>(o[4 * i + 0], pa[0], pa[1], pa[2], pa[3], bytes_to_half2(r0, 0x5240u), bytes_to_half2(r1, 0x5240u));
            mma16816<MT>(o[4 * i + 1], pa[0], pa[1], pa[2], pa[3], bytes_to_half2(r0, 0x5341u), bytes_to_half2(r1, 0x5341u));
            mma16816<MT>(o[4 * i + 2], pa[0], pa[1], pa[2], pa[3], bytes_to_half2(r2, 0x5240u), bytes_to_half2(r3, 0x5240u));
            mma16816<MT>(o[4 * i + 3], pa[0], pa[1], pa[2], pa[3], bytes_to_half2(r2, 0x5341u), bytes_to_half2(r3, 0x5341u));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
      if (++st == C::kStages) { st = 0; ph ^= 1; }
    }

    // ---------------- merge the eight warps' states ----------------
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    if (G16) {
      l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
      l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    }
    if (q4 == 0) {
      mlbuf[warp * 16 + gid] = make_float2(m_lo, l_lo);
      if (G16) mlbuf[warp * 16 + gid + 8] = make_float2(m_hi, l_hi);
    }
    named_bar_sync(1, kConsumerThreads);
    {
      float Mlo = kNeg, Mhi = kNeg;
#pragma unroll
      for (int w2 = 0; w2 < kConsumerWarps; ++w2) {
        Mlo = fmaxf(Mlo, mlbuf[w2 * 16 + gid].x);
        if (G16) Mhi = fmaxf(Mhi, mlbuf[w2 * 16 + gid + 8].x);
      }
      const float flo = fast_exp2(m_lo - Mlo), fhi = G16 ? fast_exp2(m_hi - Mhi) : 0.f;
      float *rlo = mbuf + (warp * C::kRows + gid) * kMergeStride;
      float *rhi = mbuf + (warp * C::kRows + (G16 ? gid + 8 : 0)) * kMergeStride;
      if (!KV8) {
#pragma unroll
        for (int jn = 0; jn < 16; ++jn) {
          const int d = 8 * jn + 2 * q4;
          *reinterpret_cast<float2 *>(rlo + d) = make_float2(o[jn][0] * flo, o[jn][1] * flo);
          if (G16) *reinterpret_cast<float2 *>(rhi + d) = make_float2(o[jn][2] * fhi, o[jn][3] * fhi);
        }
      } else {
#pragma unroll
        for (int cg = 0; cg < 8; ++cg) {
          const int d = 16 * cg + 4 * q4;  // even tile -> d, d+2; odd tile -> d+1, d+3
          *reinterpret_cast<float4 *>(rlo + d) =
              make_float4(o[2 * cg][0] * flo, o[2 * cg + 1][0] * flo, o[2 * cg][1] * flo, o[2 * cg + 1][1] * flo);
          if (G16)
            *reinterpret_cast<float4 *>(rhi + d) =
                make_float4(o[2 * cg][2] * fhi, o[2 * cg + 1][2] * fhi, o[2 * cg][3] * fhi, o[2 * cg + 1][3] * fhi);
        }
      }
    }
    named_bar_sync(1, kConsumerThreads);
    {
      const int c4 = (tid & 31) * 4;  // four consecutive head-dim columns
#pragma unroll
      for (int rr = 0; rr < C::kRows / 8; ++rr) {
        const int row = (tid >> 5) + 8 * rr;
        if (row < nrows) {
          float M = kNeg;
#pragma unroll
          for (int w2 = 0; w2 < kConsumerWarps; ++w2) M = fmaxf(M, mlbuf[w2 * 16 + row].x);
          float L = 0.f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int w2 = 0; w2 < kConsumerWarps; ++w2) {
            const float2 ml = mlbuf[w2 * 16 + row];
            L = fmaf(ml.y, fast_exp2(ml.x - M), L);
            const float4 v = *reinterpret_cast<const float4 *>(mbuf + (w2 * C::kRows + row) * kMergeStride + c4);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          const int hq = kvh * p.group + row0 + row;
          if (nsplit == 1) {
            const float inv = 1.f / L;
            float r0 = acc.x * inv, r1 = acc.y * inv, r2 = acc.z * inv, r3 = acc.w * inv;
            if (KV8) {
              const float4 vs = __ldg(reinterpret_cast<const float4 *>(p.v_descale + kvh * kD + c4));
              if (p.v_offset != nullptr) {
                const int4 vo = __ldg(reinterpret_cast<const int4 *>(p.v_offset + kvh * kD + c4));
                r0 += (float)vo.x; r1 += (float)vo.y; r2 += (float)vo.z; r3 += (float)vo.w;
              }
              r0 *= vs.x; r1 *= vs.y; r2 *= vs.z; r3 *= vs.w;
            }
            uint2 pk;
            pk.x = pack2<T>(r0, r1);
            pk.y = pack2<T>(r2, r3);
            *reinterpret_cast<uint2 *>(static_cast<T *>(p.out) + ((int64_t)b * p.num_q_heads + hq) * kD + c4) = pk;
          } else {
            const int64_t prow = (int64_t)part * p.num_q_heads + hq;
            *reinterpret_cast<float4 *>(p.part_o + prow * kD + c4) = acc;
            if ((tid & 31) == 0) *reinterpret_cast<float2 *>(p.part_ml + prow * 2) = make_float2(M, L);
          }
        }
      }
    }
    named_bar_sync(1, kConsumerThreads);  // merge buffers are reused by the next item
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// View of one cache as [tokens = num_blocks * block_size][kv heads][head_dim]; a box is one head's
// rows of one cache block (block_size tokens) and 128 bytes of the head dimension.
int make_cache_tmap(CUtensorMap *tm, const void *cache, const MscoPaDesc &d) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return fail(MSCO_ERR_CUDA, "paged_attention: cuTensorMapEncodeTiled is not available");
  const bool kv8 = d.kv_dtype == MSCO_DTYPE_I8;
  const int es = kv8 ? 1 : 2;
  const cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)d.num_kv_heads,
                              (cuuint64_t)d.num_blocks * (cuuint64_t)d.block_size};
  const cuuint64_t strides[2] = {(cuuint64_t)kD * es, (cuuint64_t)d.num_kv_heads * kD * es};
  const cuuint32_t box[3] = {(cuuint32_t)(kv8 ? 128 : 64), 1u, (cuuint32_t)(d.block_size < kTile ? d.block_size : kTile)};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt = kv8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : (d.kv_dtype == MSCO_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  const CUresult r = enc(tm, dt, 3, const_cast<void *>(cache), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MSCO_ERR_CUDA, "paged_attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return MSCO_OK;
}

template <typename T, bool KV8, bool G16>
int launch_one(const MscoPaPlan *plan, const PaParams &p, const CUtensorMap &tk, const CUtensorMap &tv,
               cudaStream_t stream) {
  using C = Cfg<KV8, G16>;
  static_assert(C::kDynSmem <= 232448, "shared memory budget of one SM exceeded");
  auto kfn = pa_tma_kernel<T, KV8, G16>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kDynSmem);
  });
  if (attr_err != cudaSuccess)
    return fail(MSCO_ERR_CUDA, "paged_attention: cudaFuncSetAttribute failed: %s", cudaGetErrorString(attr_err));
  kfn<<<dim3(plan->grid), dim3(kThreads), C::kDynSmem, stream>>>(tk, tv, p);
  MSCO_CUDA_CHECK(cudaGetLastError());
  return MSCO_OK;
}

}  // namespace

bool pa_tma_supported(const MscoPaDesc &d) {
  const int bs = d.block_size;
  const bool bs_ok = bs == 16 || bs == 32 || bs == 64 || bs == 128;
  return d.head_dim == kD && bs_ok && d.mask_type == 0 && d.num_blocks * (int64_t)bs < (1ll << 31);
}

int launch_pa_tma(const MscoPaPlan *plan, const PaParams &p, cudaStream_t stream) {
  if (plan->total_items == 0) return MSCO_OK;
  if ((reinterpret_cast<uintptr_t>(p.q) & 15) || (reinterpret_cast<uintptr_t>(p.key_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(p.value_cache) & 15) || (reinterpret_cast<uintptr_t>(p.out) & 7))
    return fail(MSCO_ERR_INVALID_ARG, "paged_attention: query / caches must be 16-byte aligned");
  CUtensorMap tk, tv;
  {
    std::lock_guard<std::mutex> g(plan->tm_mutex);
    if (plan->tm_k_ptr != p.key_cache) {
      int rc = make_cache_tmap(reinterpret_cast<CUtensorMap *>(plan->tm_k), p.key_cache, plan->desc);
      if (rc != MSCO_OK) return rc;
      plan->tm_k_ptr = p.key_cache;
    }
    if (plan->tm_v_ptr != p.value_cache) {
      int rc = make_cache_tmap(reinterpret_cast<CUtensorMap *>(plan->tm_v), p.value_cache, plan->desc);
      if (rc != MSCO_OK) return rc;
      plan->tm_v_ptr = p.value_cache;
    }
    tk = *reinterpret_cast<const CUtensorMap *>(plan->tm_k);
    tv = *reinterpret_cast<const CUtensorMap *>(plan->tm_v);
  }
  const bool kv8 = plan->desc.kv_dtype == MSCO_DTYPE_I8;
  const bool g16 = plan->rows_per_item == 16;
  const bool f16 = plan->desc.q_dtype == MSCO_DTYPE_F16;
#define MSCO_GO(T, A, B) return launch_one<T, A, B>(plan, p, tk, tv, stream)
  if (f16) {
    if (kv8) { if (g16) MSCO_GO(__half, true, true); else MSCO_GO(__half, true, false); }
    else     { if (g16) MSCO_GO(__half, false, true); else MSCO_GO(__half, false, false); }
  } else {
    if (kv8) { if (g16) MSCO_GO(__nv_bfloat16, true, true); else MSCO_GO(__nv_bfloat16, true, false); }
    else     { if (g16) MSCO_GO(__nv_bfloat16, false, true); else MSCO_GO(__nv_bfloat16, false, false); }
  }
#undef MSCO_GO
}

}  // namespace msco
