// reshape_and_cache for B200: scatter new K/V token rows into the paged cache.
//
// HBM-bound byte movement.  One warp moves the K row and the V row of one
// token with 16-byte loads that are all issued before the first store, so a
// resident SM keeps hundreds of KB in flight.  Algorithmic bytes per valid
// token: (k_row_bytes + v_row_bytes) read + the same written + 4 (slot).
#include <algorithm>

#include "msco_common.cuh"
#include "pa_params.h"

namespace msco {
namespace {

constexpr int kRacThreads = 256;
constexpr int kRacWarps = kRacThreads / 32;

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// 16-byte path.  k16 / v16 = 16-byte chunks per row (v16 == 0: key only).
// UNROLL chunks per lane are loaded before any is stored.  Warps stride over the tokens (the grid
// is sized to the SM count for large inputs), so every SM stays busy until the last token.
__device__ __forceinline__ void st_stream16(uint4 *p, const uint4 &v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int UNROLL, bool CS>
__global__ void __launch_bounds__(kRacThreads)
rac_scatter16_kernel(const uint4 *__restrict__ key, const uint4 *__restrict__ value,
                     uint4 *__restrict__ key_cache, uint4 *__restrict__ value_cache,
                     const int32_t *__restrict__ slot_mapping, int64_t num_tokens, int k16, int v16,
                     int64_t num_slots, int32_t *oob_count, uint32_t *__restrict__ clear, int clear_words) {
  // launched with programmatic stream serialisation itself: the grid may be resident before the
  // kernels in front of it (the previous decode step) have finished; nothing is read or written
  // before they have (a no-op behind an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // a kernel launched behind this one with programmatic stream serialisation (the attention kernel
  // of a fused decode step) may start its set-up now; it waits for this grid before reading the cache
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // scheduling words of that attention kernel: zeroed here, on the way
  for (int i = blockIdx.x * kRacThreads + threadIdx.x; i < clear_words; i += gridDim.x * kRacThreads) clear[i] = 0u;
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * kRacWarps;
  const int total = k16 + v16;  // K chunks then V chunks, one flat index space
  for (int64_t tok = (int64_t)blockIdx.x * kRacWarps + (threadIdx.x >> 5); tok < num_tokens; tok += nwarps) {
    const int64_t slot = __ldg(slot_mapping + tok);
    if (slot < 0) continue;  // padding token: nothing is written
    if (slot >= num_slots) {
      if (lane == 0 && oob_count != nullptr) atomicAdd(oob_count, 1);
      continue;
    }
    const uint4 *ks = key + tok * k16;
    uint4 *kd = key_cache + slot * k16;
    const uint4 *vs = value + tok * v16;
    uint4 *vd = value_cache + slot * v16;
    for (int c0 = lane; c0 < total; c0 += 32 * UNROLL) {
      uint4 r[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + 32 * u;
        if (c < total) r[u] = (c < k16) ? ld_stream16(ks + c) : ld_stream16(vs + (c - k16));
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + 32 * u;
        if (c < total) {
          uint4 *dst = (c < k16) ? kd + c : vd + (c - k16);
          if (CS) st_stream16(dst, r[u]); else *dst = r[u];
        }
      }
    }
  }
}

// 2-byte path for rows or pointers that are not 16-byte aligned.
__global__ void __launch_bounds__(kRacThreads)
rac_scatter2_kernel(const uint16_t *__restrict__ key, const uint16_t *__restrict__ value,
                    uint16_t *__restrict__ key_cache, uint16_t *__restrict__ value_cache,
                    const int32_t *__restrict__ slot_mapping, int64_t num_tokens, int k2, int v2,
                    int64_t num_slots, int32_t *oob_count) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * kRacWarps + (threadIdx.x >> 5);
  if (tok >= num_tokens) return;
  const int64_t slot = __ldg(slot_mapping + tok);
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (lane == 0 && oob_count != nullptr) atomicAdd(oob_count, 1);
    return;
  }
  for (int c = lane; c < k2; c += 32) key_cache[slot * k2 + c] = key[tok * k2 + c];
  for (int c = lane; c < v2; c += 32) value_cache[slot * v2 + c] = value[tok * v2 + c];
}

// 1-byte path (int8 rows of odd length)
__global__ void __launch_bounds__(kRacThreads)
rac_scatter1_kernel(const uint8_t *__restrict__ key, const uint8_t *__restrict__ value,
                    uint8_t *__restrict__ key_cache, uint8_t *__restrict__ value_cache,
                    const int32_t *__restrict__ slot_mapping, int64_t num_tokens, int k1, int v1,
                    int64_t num_slots, int32_t *oob_count) {
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * kRacWarps + (threadIdx.x >> 5);
  if (tok >= num_tokens) return;
  const int64_t slot = __ldg(slot_mapping + tok);
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (lane == 0 && oob_count != nullptr) atomicAdd(oob_count, 1);
    return;
  }
  for (int c = lane; c < k1; c += 32) key_cache[slot * k1 + c] = key[tok * k1 + c];
  for (int c = lane; c < v1; c += 32) value_cache[slot * v1 + c] = value[tok * v1 + c];
}

// ---- head-major cache blocks ("BNSD": [num_blocks, heads, block_size, head_dim]) --------------------
// The layout of the reference's reshape_and_cache_npd (cache shapes
// ops/ascendc/ms_glue/reshape_and_cache_npd/reshape_and_cache_npd.md:24-25; addressing
// ops/ascendc/aclnn_src/reshape_and_cache_npd/op_kernel/reshape_and_cache_npd.cpp:167-173): the rows of
// one head of one block are contiguous, so the token row is split by head and head h of slot s lands at
// ((s / block_size * heads + h) * block_size + s % block_size) * head_bytes.  G = bytes per copy granule.
template <typename G, int UNROLL>
__global__ void __launch_bounds__(kRacThreads)
rac_scatter_bnsd_kernel(const G *__restrict__ key, const G *__restrict__ value, G *__restrict__ key_cache,
                        G *__restrict__ value_cache, const int32_t *__restrict__ slot_mapping, int64_t num_tokens,
                        int heads, int kg, int vg, int block_size, int64_t num_slots, int32_t *oob_count) {
  // kg / vg: granules per head row of K / V (vg == 0: key only)
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * kRacWarps;
  const int ktot = heads * kg, total = heads * (kg + vg);
  for (int64_t tok = (int64_t)blockIdx.x * kRacWarps + (threadIdx.x >> 5); tok < num_tokens; tok += nwarps) {
    const int64_t slot = __ldg(slot_mapping + tok);
    if (slot < 0) continue;  // padding token: nothing is written
    if (slot >= num_slots) {
      if (lane == 0 && oob_count != nullptr) atomicAdd(oob_count, 1);
      continue;
    }
    const int64_t blk = slot / block_size, off = slot - blk * block_size;
    const G *ks = key + tok * (int64_t)ktot;
    const G *vs = value + tok * (int64_t)(heads * vg);
    for (int c0 = lane; c0 < total; c0 += 32 * UNROLL) {
      G r[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + 32 * u;
        if (c < total) r[u] = (c < ktot) ? ks[c] : vs[c - ktot];
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int c = c0 + 32 * u;
        if (c < total) {
          const bool is_k = c < ktot;
          const int cc = is_k ? c : c - ktot, per = is_k ? kg : vg;
          const int h = cc / per, g = cc - h * per;
          G *dst = (is_k ? key_cache : value_cache) + ((blk * heads + h) * block_size + off) * per + g;
          *dst = r[u];
        }
      }
    }
  }
}

// ---- quantising scatter ------------------------------------------------------
// q = saturate_int8(rint(float(x) / descale[c]) - offset[c]); IEEE division,
// round-half-to-even, NaN -> 0: bit-identical to float32 numpy arithmetic.
__device__ __forceinline__ int quant_one(float x, float d, float off) {
  float q = rintf(__fdiv_rn(x, d));
  q = __fsub_rn(q, off);
  if (q != q) q = 0.f;
  q = fminf(fmaxf(q, -128.f), 127.f);
  return (int)q;
}

template <typename T>
__device__ __forceinline__ void quant_row8(const T *__restrict__ src, int8_t *__restrict__ dst,
                                           const float *__restrict__ descale,
                                           const int32_t *__restrict__ offset, int elems, int lane) {
  // 8 elements per lane per step: one 16-byte load, one 8-byte store
  for (int e = lane * 8; e < elems; e += 32 * 8) {
    uint4 raw = ld_stream16(src + e);
    const T *x = reinterpret_cast<const T *>(&raw);
    const float4 d0 = __ldg(reinterpret_cast<const float4 *>(descale + e));
    const float4 d1 = __ldg(reinterpret_cast<const float4 *>(descale + e + 4));
    float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (offset != nullptr) {
      const int4 o0 = __ldg(reinterpret_cast<const int4 *>(offset + e));
      const int4 o1 = __ldg(reinterpret_cast<const int4 *>(offset + e + 4));
      o[0] = (float)o0.x; o[1] = (float)o0.y; o[2] = (float)o0.z; o[3] = (float)o0.w;
      o[4] = (float)o1.x; o[5] = (float)o1.y; o[6] = (float)o1.z; o[7] = (float)o1.w;
    }
    const float d[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= (uint32_t)(quant_one(to_f32<T>(x[i]), d[i], o[i]) & 0xff) << (8 * i);
      hi |= (uint32_t)(quant_one(to_f32<T>(x[i + 4]), d[i + 4], o[i + 4]) & 0xff) << (8 * i);
    }
    *reinterpret_cast<uint2 *>(dst + e) = make_uint2(lo, hi);
  }
}

template <typename T>
__device__ __forceinline__ void quant_row1(const T *__restrict__ src, int8_t *__restrict__ dst,
                                           const float *__restrict__ descale,
                                           const int32_t *__restrict__ offset, int elems, int lane) {
  for (int e = lane; e < elems; e += 32) {
    const float off = offset ? (float)__ldg(offset + e) : 0.f;
    dst[e] = (int8_t)quant_one(to_f32<T>(src[e]), __ldg(descale + e), off);
  }
}

// Four warps per token (K low half, K high half, V low half, V high half of the row): a decode
// step has only `batch` tokens, so the work of one token is spread to keep the kernel short.
constexpr int kQuantParts = 4;

template <typename T, bool VEC>
__global__ void __launch_bounds__(kRacThreads)
rac_scatter_quant_kernel(const T *__restrict__ key, const T *__restrict__ value,
                         int8_t *__restrict__ key_cache, int8_t *__restrict__ value_cache,
                         const int32_t *__restrict__ slot_mapping, int64_t num_tokens, int k_elems,
                         int v_elems, const float *__restrict__ k_descale,
                         const int32_t *__restrict__ k_offset, const float *__restrict__ v_descale,
                         const int32_t *__restrict__ v_offset, int64_t num_slots, int32_t *oob_count) {
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * kRacWarps + (threadIdx.x >> 5);
  const int64_t tok = unit / kQuantParts;
  const int part = (int)(unit - tok * kQuantParts);
  if (tok >= num_tokens) return;
  const int64_t slot = __ldg(slot_mapping + tok);
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (lane == 0 && part == 0 && oob_count != nullptr) atomicAdd(oob_count, 1);
    return;
  }
  const bool is_v = part >= 2;
  const int elems = is_v ? v_elems : k_elems;
  if (elems == 0) return;
  // split the row at a multiple of 8 elements so that both halves keep the vector alignment
  const int half = ((elems / 2) + 7) & ~7;
  const int e0 = (part & 1) ? min(half, elems) : 0, e1 = (part & 1) ? elems : min(half, elems);
  if (e0 >= e1) return;
  const T *src = (is_v ? value + tok * v_elems : key + tok * k_elems) + e0;
  int8_t *dst = (is_v ? value_cache + slot * v_elems : key_cache + slot * k_elems) + e0;
  const float *ds = (is_v ? v_descale : k_descale) + e0;
  const int32_t *of = is_v ? v_offset : k_offset;
  if (of != nullptr) of += e0;
  if (VEC) quant_row8<T>(src, dst, ds, of, e1 - e0, lane);
  else quant_row1<T>(src, dst, ds, of, e1 - e0, lane);
}

// Fast path of the quantising scatter for rows of up to 1024 channels (K and V alike).
// Warps stride over the tokens and each warp owns whole K rows or whole V rows, so a lane's channels
// never change: the reciprocals of the scales and the offsets are loaded once into registers.
//
// rint(x / d) without a division, exactly: with r = fl(1 / d) and e = x * r (the exact product),
//   z = fma(x, r, M), M = 1.5 * 2^23   rounds e to the nearest integer (ties to even) for |e| < 2^22,
//   q = z - M                          is that integer, t = fma(x, r, -q) = e - q its distance to e.
// e differs from x / d by at most |e| * 2^-24 (r is a correctly rounded normal number), and the
// correctly rounded quotient from x / d by at most half an ulp: together less than |q| * 2^-23 * 1.01.
// So |t| <= 0.49995 - q^2 * 2^-30 puts fl(x / d) strictly within 0.5 of q, i.e. rint(fl(x / d)) = q:
// below |q| = 256 the constant margin (5e-5 > 3.1e-5) covers the error, from 256 on the quadratic
// term does (q^2 * 2^-30 >= |q| * 2^-22).  The threshold turns negative at |q| = 23170, so whatever
// passes also fits 16 bits.  Everything else -- ties, huge quotients, NaN, and through r = NaN the
// channels whose scale is zero-like, huge or not finite or whose offset exceeds 8192 -- fails the test
// (the comparison is false for NaN) and takes the IEEE division (quant_exact).  The test is this
// tight on purpose: one lane that fails it sends its whole warp through the division for that group
// of eight, and with 0.013 % of the values failing that happens in 3 % of the groups.
// z - offset is still an integer in M's binade, so the low 16 bits of its bit pattern are the
// two's-complement value: two of them are packed into one register, clamped to [-128, 127] with one
// 16-bit SIMD max and one min, and the low bytes of four halves are gathered with one byte permute.
// Per element: 5 instructions on the FMA pipe, under 4 on the ALU pipe (the unpacking of the 16-bit
// input, one compare, 1.75 for clamp and pack); no conversion instruction; bit-identical to the
// division everywhere.
constexpr float kQMagic = 12582912.f;
constexpr float kQAccept = 0.49995f;          // |t| up to here (minus the quadratic term) is no tie
constexpr float kQQuad = 9.313225746154785e-10f;  // 2^-30
constexpr float kQMaxOffset = 8192.f;
// one element: the bit pattern of M + q - offset; `ok` is cleared when the element needs the division
// (`&`, not `&&`: a compare that feeds the predicate of the next one, no branch per element)
template <bool HAS_OFF>
__device__ __forceinline__ uint32_t quant_fast(float x, float r, float off, bool &ok) {
  const float z = fmaf(x, r, kQMagic);
  const float q = z - kQMagic;
  const float t = fmaf(x, r, -q);
  const float thr = fmaf(q * q, -kQQuad, kQAccept);
  ok = ok & (fabsf(t) <= thr);
  return __float_as_uint(HAS_OFF ? z - off : z);
}
// the eight 16-bit values of a 16-byte load as float32 (bfloat16: one shift or one mask each)
template <typename T> __device__ __forceinline__ void unpack8(const uint4 &raw, float (&x)[8]);
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4 &raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void unpack8<__half>(const uint4 &raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    x[2 * i] = f.x;
    x[2 * i + 1] = f.y;
  }
}
// the same element by the IEEE division, for the groups the fast test does not cover
template <bool HAS_OFF>
__device__ __forceinline__ uint32_t quant_exact(float x, float d, float off) {
  float v = rintf(__fdiv_rn(x, d));
  if (HAS_OFF) v = __fsub_rn(v, off);
  if (v != v) v = 0.f;
  v = fminf(fmaxf(v, -128.f), 127.f);
  return __float_as_uint(v + kQMagic);
}
// low 16 bits of four words, each clamped to [-128, 127] as a signed 16-bit value -> four bytes
// (measured: the packed 16-bit min / max are single instructions here; the float clamp costs one more per element)
__device__ __forceinline__ uint32_t clamp_pack4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
  uint32_t h01, h23, o;
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(h01) : "r"(w0), "r"(w1));
  asm("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(h23) : "r"(w2), "r"(w3));
  asm("max.s16x2 %0, %0, %1;" : "+r"(h01) : "r"(0xff80ff80u));
  asm("min.s16x2 %0, %0, %1;" : "+r"(h01) : "r"(0x007f007fu));
  asm("max.s16x2 %0, %0, %1;" : "+r"(h23) : "r"(0xff80ff80u));
  asm("min.s16x2 %0, %0, %1;" : "+r"(h23) : "r"(0x007f007fu));
  asm("prmt.b32 %0, %1, %2, 0x6420;" : "=r"(o) : "r"(h01), "r"(h23));
  return o;
}
// A whole group of eight by the division: ONE out-of-line call, so that the rare path costs the common
// one a single branch and no argument set-up (scales and offsets are re-read from global memory here).
template <typename T, bool HAS_OFF>
__device__ __noinline__ uint2 quant_group_exact(uint4 raw, const float *__restrict__ ds, const int32_t *__restrict__ of) {
  float x[8];
  unpack8<T>(raw, x);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = quant_exact<HAS_OFF>(x[i], __ldg(ds + i), HAS_OFF ? (float)__ldg(of + i) : 0.f);
  return make_uint2(clamp_pack4(w[0], w[1], w[2], w[3]), clamp_pack4(w[4], w[5], w[6], w[7]));
}
// reciprocal of a channel's scale for the fast test, NaN (= always take the division) when the
// reciprocal would not be a correctly rounded normal number or the offset is beyond the 16-bit argument
__device__ __forceinline__ float quant_reciprocal(float d, float off) {
  const float ad = fabsf(d);
  const bool plain = ad >= 1.1754944e-38f && ad <= 4.2535296e37f && fabsf(off) <= kQMaxOffset;  // [2^-126, 2^125]
  return plain ? __frcp_rn(d) : __int_as_float(0x7fc00000);
}

// One warp quantises whole K rows or whole V rows (fixed per warp), striding over the tokens.  The
// reciprocal scales (and offsets) of all channels sit in shared memory, filled once per block AFTER
// the warps' first rows have been requested, in a layout that makes a lane's eight values two
// conflict-free 16-byte reads; a warp requests its next row before it stores the current one.  Few
// registers per thread, so four blocks (32 warps) are resident per SM: with one warp converting while
// the others wait for memory, that occupancy -- not a deep per-warp prefetch -- is what keeps both the
// memory system and the arithmetic pipes busy (measured: 2 rows in flight per warp at 16 warps per SM
// 26.5 us, this form 24.4 us, the same loop without any arithmetic 20.8 us, for 16384 tokens).
constexpr int kQuantFastBlocksPerSm = 4;
template <typename T, bool HAS_OFF>
__global__ void __launch_bounds__(kRacThreads, kQuantFastBlocksPerSm)
rac_scatter_quant_fast_kernel(const T *__restrict__ key, const T *__restrict__ value,
                              int8_t *__restrict__ key_cache, int8_t *__restrict__ value_cache,
                              const int32_t *__restrict__ slot_mapping, int64_t num_tokens, int elems,
                              const float *__restrict__ k_descale, const int32_t *__restrict__ k_offset,
                              const float *__restrict__ v_descale, const int32_t *__restrict__ v_offset,
                              int64_t num_slots, int32_t *oob_count, bool has_v,
                              uint32_t *__restrict__ clear, int clear_words) {
  // [K | V][16-byte group of a lane: it * 2 + half][lane]
  __shared__ float4 rs[2][8][32];
  __shared__ float4 os[HAS_OFF ? 2 : 1][HAS_OFF ? 8 : 1][HAS_OFF ? 32 : 1];
  asm volatile("griddepcontrol.wait;" ::: "memory");               // see rac_scatter16_kernel
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (int i = blockIdx.x * kRacThreads + threadIdx.x; i < clear_words; i += gridDim.x * kRacThreads) clear[i] = 0u;
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * kRacWarps + (threadIdx.x >> 5);
  const int64_t nunits = (int64_t)gridDim.x * kRacWarps;
  const bool is_v = has_v && (unit & 1);
  const int64_t first = has_v ? unit >> 1 : unit, stride = has_v ? nunits >> 1 : nunits;
  const float *ds = is_v ? v_descale : k_descale;
  const int32_t *of = is_v ? v_offset : k_offset;
  const T *src_base = is_v ? value : key;
  int8_t *dst_base = is_v ? value_cache : key_cache;

  uint4 raw[4];
  int64_t slot = -1;
  auto fetch = [&](int64_t tok) {
    slot = -1;
    if (tok < num_tokens) {
      slot = __ldg(slot_mapping + tok);
      if (slot >= num_slots) {
        if (lane == 0 && !is_v && oob_count != nullptr) atomicAdd(oob_count, 1);
        slot = -1;
      }
      // the row is fetched before the slot is known to be valid: rows of padding tokens are
      // readable memory, and waiting for the slot would serialise two memory latencies
      const T *src = src_base + tok * elems + lane * 8;
#pragma unroll
      for (int it = 0; it < 4; ++it)
        if (lane * 8 + it * 256 < elems) raw[it] = ld_stream16(src + it * 256);
    }
  };
  fetch(first);
  // the tables, while the first rows are on their way
  for (int i = threadIdx.x; i < (has_v ? 2 : 1) * 8 * 32; i += kRacThreads) {
    const int kv = i >> 8, j = (i >> 5) & 7, ln = i & 31;
    const int e = ln * 8 + (j >> 1) * 256 + (j & 1) * 4;
    float4 d4 = make_float4(1.f, 1.f, 1.f, 1.f);
    int4 o4 = make_int4(0, 0, 0, 0);
    if (e < elems) {
      d4 = __ldg(reinterpret_cast<const float4 *>((kv ? v_descale : k_descale) + e));
      if (HAS_OFF) o4 = __ldg(reinterpret_cast<const int4 *>((kv ? v_offset : k_offset) + e));
    }
    rs[kv][j][ln] = make_float4(quant_reciprocal(d4.x, (float)o4.x), quant_reciprocal(d4.y, (float)o4.y),
                                quant_reciprocal(d4.z, (float)o4.z), quant_reciprocal(d4.w, (float)o4.w));
    if (HAS_OFF) os[kv][j][ln] = make_float4((float)o4.x, (float)o4.y, (float)o4.z, (float)o4.w);
  }
  __syncthreads();
  const int kv = is_v ? 1 : 0;
  for (int64_t tok = first; tok < num_tokens; tok += stride) {
    const int64_t slot_cur = slot;
    uint32_t out[8];
    if (slot_cur >= 0) {
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int e = lane * 8 + it * 256;
        if (e < elems) {
          float x[8];
          unpack8<T>(raw[it], x);
          const float4 ra = rs[kv][it * 2][lane], rb = rs[kv][it * 2 + 1][lane];
          const float r[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};
          float o[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (HAS_OFF) {
            const float4 oa = os[kv][it * 2][lane], ob = os[kv][it * 2 + 1][lane];
            o[0] = oa.x; o[1] = oa.y; o[2] = oa.z; o[3] = oa.w;
            o[4] = ob.x; o[5] = ob.y; o[6] = ob.z; o[7] = ob.w;
          }
          uint32_t w[8];
          bool ok = true;
#pragma unroll
          for (int i = 0; i < 8; ++i) w[i] = quant_fast<HAS_OFF>(x[i], r[i], o[i], ok);
          // rare: a tie, a huge quotient, an odd scale somewhere in these eight (of any lane: the vote
          // keeps the branch warp-uniform, and the division gives the same bits where the test passed)
          if (__any_sync(__activemask(), !ok)) {
            const uint2 ex = quant_group_exact<T, HAS_OFF>(raw[it], ds + e, HAS_OFF ? of + e : nullptr);
            out[2 * it] = ex.x;
            out[2 * it + 1] = ex.y;
          } else {
            out[2 * it] = clamp_pack4(w[0], w[1], w[2], w[3]);
            out[2 * it + 1] = clamp_pack4(w[4], w[5], w[6], w[7]);
          }
        }
      }
    }
    fetch(tok + stride);  // the next row's loads go out before this row's stores
    if (slot_cur >= 0) {
      int8_t *dst = dst_base + slot_cur * elems + lane * 8;
#pragma unroll
      for (int it = 0; it < 4; ++it)
        if (lane * 8 + it * 256 < elems)
          asm volatile("st.global.cs.v2.u32 [%0], {%1,%2};" ::"l"(dst + it * 256), "r"(out[2 * it]), "r"(out[2 * it + 1])
                       : "memory");
    }
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Launch with programmatic stream serialisation: the grid may become resident while the kernel in
// front of it on the stream drains (the kernel itself waits, griddepcontrol.wait, before it touches
// memory), which hides the launch latency between two decode steps.
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace
}  // namespace msco

using namespace msco;

extern "C" int msco_reshape_and_cache(const void *key, const void *value, void *key_cache, void *value_cache,
                                      const int32_t *slot_mapping, int64_t num_tokens, int64_t k_row_bytes,
                                      int64_t v_row_bytes, int64_t num_slots, int32_t *oob_count,
                                      void *stream) {
  bool cleared = false;
  return launch_rac(key, value, key_cache, value_cache, slot_mapping, num_tokens, k_row_bytes, v_row_bytes, num_slots,
                    oob_count, static_cast<cudaStream_t>(stream), nullptr, 0, &cleared);
}

int msco::launch_rac(const void *key, const void *value, void *key_cache, void *value_cache,
                     const int32_t *slot_mapping, int64_t num_tokens, int64_t k_row_bytes, int64_t v_row_bytes,
                     int64_t num_slots, int32_t *oob_count, cudaStream_t st, uint32_t *clear, int clear_words,
                     bool *cleared) {
  *cleared = false;
  if (num_tokens < 0 || k_row_bytes < 0 || v_row_bytes < 0 || num_slots < 0)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache: negative size");
  // zero-sized inputs: the reference skips execution (reshape_and_cache.cc:90-119)
  if (num_tokens == 0 || k_row_bytes == 0 || num_slots == 0) return MSCO_OK;
  const bool has_v = (value != nullptr) || (value_cache != nullptr);
  if (has_v && (value == nullptr || value_cache == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache: value and value_cache must be given together");
  if (!has_v) v_row_bytes = 0;
  if (key == nullptr || key_cache == nullptr || slot_mapping == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache: key, key_cache and slot_mapping must not be NULL");
  if (k_row_bytes > (int64_t)INT32_MAX || v_row_bytes > (int64_t)INT32_MAX)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache: row too large");
  const int64_t blocks64 = (num_tokens + kRacWarps - 1) / kRacWarps;
  if (blocks64 > 0x7fffffffLL) return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache: too many tokens");
  const dim3 grid((unsigned)blocks64), block(kRacThreads);
  // the 16-byte kernel strides over tokens: at most four resident CTAs per SM
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      sm_count = n;
    else
      sm_count = 148;
  }
  // measured on B200 (16384 tokens of 2 x 2 KB): 16 CTAs per SM in the grid, streaming stores and
  // eight 16-byte loads in flight per lane reach 0.85 of the measured copy bandwidth
  const dim3 grid16((unsigned)std::min<int64_t>(blocks64, (int64_t)sm_count * 16));
  const bool vec = (k_row_bytes % 16 == 0) && (v_row_bytes % 16 == 0) && aligned16(key) && aligned16(key_cache) &&
                   (!has_v || (aligned16(value) && aligned16(value_cache)));
  if (vec) {
    const int k16 = (int)(k_row_bytes / 16), v16 = (int)(v_row_bytes / 16);
    if (k16 + v16 > 128) {
      MSCO_CUDA_CHECK(launch_overlapped(rac_scatter16_kernel<8, true>, grid16, block, st,
          (const uint4 *)key, (const uint4 *)value, (uint4 *)key_cache, (uint4 *)value_cache, slot_mapping,
          num_tokens, k16, v16, num_slots, oob_count, clear, clear_words));
    } else {
      MSCO_CUDA_CHECK(launch_overlapped(rac_scatter16_kernel<4, true>, grid16, block, st,
          (const uint4 *)key, (const uint4 *)value, (uint4 *)key_cache, (uint4 *)value_cache, slot_mapping,
          num_tokens, k16, v16, num_slots, oob_count, clear, clear_words));
    }
    *cleared = clear_words > 0;
  } else if (k_row_bytes % 2 == 0 && v_row_bytes % 2 == 0 && (((uintptr_t)key | (uintptr_t)key_cache |
             (uintptr_t)value | (uintptr_t)value_cache) & 1) == 0) {
    rac_scatter2_kernel<<<grid, block, 0, st>>>((const uint16_t *)key, (const uint16_t *)value,
                                                (uint16_t *)key_cache, (uint16_t *)value_cache, slot_mapping,
                                                num_tokens, (int)(k_row_bytes / 2), (int)(v_row_bytes / 2),
                                                num_slots, oob_count);
  } else {
    rac_scatter1_kernel<<<grid, block, 0, st>>>((const uint8_t *)key, (const uint8_t *)value,
                                                (uint8_t *)key_cache, (uint8_t *)value_cache, slot_mapping,
                                                num_tokens, (int)k_row_bytes, (int)v_row_bytes, num_slots,
                                                oob_count);
  }
  MSCO_CUDA_CHECK(cudaGetLastError());
  return MSCO_OK;
}

extern "C" int msco_reshape_and_cache_quant(const void *key, const void *value, int8_t *key_cache,
                                            int8_t *value_cache, const int32_t *slot_mapping,
                                            int64_t num_tokens, int64_t k_row_elems, int64_t v_row_elems,
                                            int32_t in_dtype, const float *k_descale, const int32_t *k_offset,
                                            const float *v_descale, const int32_t *v_offset, int64_t num_slots,
                                            int32_t *oob_count, void *stream) {
  bool cleared = false;
  return launch_rac_quant(key, value, key_cache, value_cache, slot_mapping, num_tokens, k_row_elems, v_row_elems,
                          in_dtype, k_descale, k_offset, v_descale, v_offset, num_slots, oob_count,
                          static_cast<cudaStream_t>(stream), nullptr, 0, &cleared);
}

extern "C" int msco_copy_device(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return MSCO_OK;
  if (dst == nullptr || src == nullptr) return fail(MSCO_ERR_INVALID_ARG, "copy_device: NULL argument");
  MSCO_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return MSCO_OK;
}

extern "C" int msco_reshape_and_cache_bnsd(const void *key, const void *value, void *key_cache, void *value_cache,
                                           const int32_t *slot_mapping, int64_t num_tokens, int32_t num_heads,
                                           int64_t k_head_bytes, int64_t v_head_bytes, int32_t block_size,
                                           int64_t num_slots, int32_t *oob_count, void *stream) {
  if (num_tokens < 0 || num_heads < 0 || k_head_bytes < 0 || v_head_bytes < 0 || block_size < 0 || num_slots < 0)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_bnsd: negative size");
  if (num_tokens == 0 || num_heads == 0 || k_head_bytes == 0 || num_slots == 0) return MSCO_OK;
  if (block_size == 0) return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_bnsd: block_size must be positive");
  const bool has_v = (value != nullptr) || (value_cache != nullptr);
  if (has_v && (value == nullptr || value_cache == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_bnsd: value and value_cache must be given together");
  if (!has_v) v_head_bytes = 0;
  if (key == nullptr || key_cache == nullptr || slot_mapping == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_bnsd: key, key_cache and slot_mapping must not be NULL");
  if ((k_head_bytes + v_head_bytes) * num_heads > (int64_t)INT32_MAX)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_bnsd: row too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t blocks64 = (num_tokens + kRacWarps - 1) / kRacWarps;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const dim3 grid((unsigned)std::min<int64_t>(blocks64, (int64_t)sms * 16)), block(kRacThreads);
  const uintptr_t all = (uintptr_t)key | (uintptr_t)key_cache | (uintptr_t)value | (uintptr_t)value_cache;
  if (k_head_bytes % 16 == 0 && v_head_bytes % 16 == 0 && (all & 15) == 0) {
    rac_scatter_bnsd_kernel<uint4, 4><<<grid, block, 0, st>>>(
        (const uint4 *)key, (const uint4 *)value, (uint4 *)key_cache, (uint4 *)value_cache, slot_mapping, num_tokens,
        num_heads, (int)(k_head_bytes / 16), (int)(v_head_bytes / 16), block_size, num_slots, oob_count);
  } else if (k_head_bytes % 2 == 0 && v_head_bytes % 2 == 0 && (all & 1) == 0) {
    rac_scatter_bnsd_kernel<uint16_t, 4><<<grid, block, 0, st>>>(
        (const uint16_t *)key, (const uint16_t *)value, (uint16_t *)key_cache, (uint16_t *)value_cache, slot_mapping,
        num_tokens, num_heads, (int)(k_head_bytes / 2), (int)(v_head_bytes / 2), block_size, num_slots, oob_count);
  } else {
    rac_scatter_bnsd_kernel<uint8_t, 4><<<grid, block, 0, st>>>(
        (const uint8_t *)key, (const uint8_t *)value, (uint8_t *)key_cache, (uint8_t *)value_cache, slot_mapping,
        num_tokens, num_heads, (int)k_head_bytes, (int)v_head_bytes, block_size, num_slots, oob_count);
  }
  MSCO_CUDA_CHECK(cudaGetLastError());
  return MSCO_OK;
}

int msco::launch_rac_quant(const void *key, const void *value, int8_t *key_cache, int8_t *value_cache,
                           const int32_t *slot_mapping, int64_t num_tokens, int64_t k_row_elems, int64_t v_row_elems,
                           int32_t in_dtype, const float *k_descale, const int32_t *k_offset, const float *v_descale,
                           const int32_t *v_offset, int64_t num_slots, int32_t *oob_count, cudaStream_t st,
                           uint32_t *clear, int clear_words, bool *cleared) {
  *cleared = false;
  if (num_tokens < 0 || k_row_elems < 0 || v_row_elems < 0 || num_slots < 0)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_quant: negative size");
  if (in_dtype != MSCO_DTYPE_F16 && in_dtype != MSCO_DTYPE_BF16)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_quant: input rows must be float16 or bfloat16");
  if (num_tokens == 0 || k_row_elems == 0 || num_slots == 0) return MSCO_OK;
  const bool has_v = (value != nullptr) || (value_cache != nullptr);
  if (has_v && (value == nullptr || value_cache == nullptr || v_descale == nullptr))
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_quant: value, value_cache and v_descale go together");
  if (!has_v) v_row_elems = 0;
  if (key == nullptr || key_cache == nullptr || slot_mapping == nullptr || k_descale == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_quant: key, key_cache, slot_mapping, k_descale required");
  if (k_row_elems > (int64_t)INT32_MAX || v_row_elems > (int64_t)INT32_MAX)
    return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_quant: row too large");
  const int64_t blocks64 = (num_tokens * kQuantParts + kRacWarps - 1) / kRacWarps;
  if (blocks64 > 0x7fffffffLL) return fail(MSCO_ERR_INVALID_ARG, "reshape_and_cache_quant: too many tokens");
  const dim3 grid((unsigned)blocks64), block(kRacThreads);
  const bool vec = (k_row_elems % 8 == 0) && (v_row_elems % 8 == 0) && aligned16(key) && aligned16(k_descale) &&
                   ((uintptr_t)key_cache % 8 == 0) && (k_offset == nullptr || aligned16(k_offset)) &&
                   (!has_v || (aligned16(value) && aligned16(v_descale) && ((uintptr_t)value_cache % 8 == 0) &&
                               (v_offset == nullptr || aligned16(v_offset))));
  // common case: equal K / V rows of at most 1024 channels, same offsets presence for K and V
  const bool has_off = k_offset != nullptr;
  if (vec && k_row_elems <= 1024 && (!has_v || (v_row_elems == k_row_elems && (v_offset != nullptr) == has_off))) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    const int64_t rows = num_tokens * (has_v ? 2 : 1);
    const int64_t want = (rows + kRacWarps - 1) / kRacWarps;
    const dim3 gridf((unsigned)std::min<int64_t>(want, (int64_t)sms * kQuantFastBlocksPerSm));  // what is resident at once
#define MSCO_QF(T, OFF)                                                                                     \
  MSCO_CUDA_CHECK(launch_overlapped(rac_scatter_quant_fast_kernel<T, OFF>, gridf, block, st,                \
      (const T *)key, (const T *)value, key_cache, value_cache, slot_mapping, num_tokens, (int)k_row_elems, \
      k_descale, k_offset, v_descale, v_offset, num_slots, oob_count, has_v, clear, clear_words))
    if (in_dtype == MSCO_DTYPE_F16) { if (has_off) MSCO_QF(__half, true); else MSCO_QF(__half, false); }
    else { if (has_off) MSCO_QF(__nv_bfloat16, true); else MSCO_QF(__nv_bfloat16, false); }
#undef MSCO_QF
    MSCO_CUDA_CHECK(cudaGetLastError());
    *cleared = clear_words > 0;
    return MSCO_OK;
  }
#define MSCO_LAUNCH_Q(T, VEC)                                                                             \
  rac_scatter_quant_kernel<T, VEC><<<grid, block, 0, st>>>(                                               \
      (const T *)key, (const T *)value, key_cache, value_cache, slot_mapping, num_tokens, (int)k_row_elems, \
      (int)v_row_elems, k_descale, k_offset, v_descale, v_offset, num_slots, oob_count)
  if (in_dtype == MSCO_DTYPE_F16) {
    if (vec) MSCO_LAUNCH_Q(__half, true); else MSCO_LAUNCH_Q(__half, false);
  } else {
    if (vec) MSCO_LAUNCH_Q(__nv_bfloat16, true); else MSCO_LAUNCH_Q(__nv_bfloat16, false);
  }
#undef MSCO_LAUNCH_Q
  MSCO_CUDA_CHECK(cudaGetLastError());
  return MSCO_OK;
}
