// fa_update for B200: merge `sp` partial attention outputs of the same rows by their log-sum-exps,
//   out[r, :] = sum_s w[s, r] * local_out[s, r, :],   w[s, r] = exp(lse[s, r]) / sum_s' exp(lse[s', r])
// (the DECODE_UPDATE of the reference: ops/c_api/fa_update/fa_update_doc.md:5-27, golden
// tests/st/test_asd_faupdate.py:34-59).  float32 throughout.
//
// HBM-bound: sp * head_size * 4 bytes read and head_size * 4 written per row.  One thread owns one
// 16-byte column group of one row; all sp loads are issued before the first use.  The weights are
// computed with the row maximum subtracted (same value, no overflow); a row whose lse are all -inf
// (no partition saw a token) gives zeros.
#include <math_constants.h>

#include <algorithm>

#include "msco_common.cuh"

namespace msco {
namespace {

constexpr int kFaThreads = 256;
constexpr int kFaMaxSp = 64;

template <typename V> struct FaVec;
template <> struct FaVec<float4> {
  static __device__ __forceinline__ float4 load(const float4 *p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
  }
  static __device__ __forceinline__ float4 zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ void fma(float4 &a, float w, const float4 &v) {
    a.x = fmaf(w, v.x, a.x); a.y = fmaf(w, v.y, a.y); a.z = fmaf(w, v.z, a.z); a.w = fmaf(w, v.w, a.w);
  }
};
template <> struct FaVec<float> {
  static __device__ __forceinline__ float load(const float *p) { return __ldg(p); }
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ void fma(float &a, float w, const float &v) { a = fmaf(w, v, a); }
};

// SP > 0: compile-time partition count, everything in registers.  SP == 0: run-time count.
template <typename V, int SP>
__global__ void __launch_bounds__(kFaThreads)
fa_update_kernel(const float *__restrict__ lse, const V *__restrict__ local_out, V *__restrict__ out, int64_t rows,
                 int cols /* V per row */, int sp_rt) {
  const int sp = SP > 0 ? SP : sp_rt;
  const int64_t total = rows * cols;
  const int64_t stride = (int64_t)gridDim.x * kFaThreads;
  for (int64_t idx = (int64_t)blockIdx.x * kFaThreads + threadIdx.x; idx < total; idx += stride) {
    const int64_t r = idx / cols;
    if constexpr (SP > 0) {
      float l[SP > 0 ? SP : 1];
      V v[SP > 0 ? SP : 1];
#pragma unroll
      for (int s = 0; s < SP; ++s) {
        l[s] = __ldg(lse + (int64_t)s * rows + r);
        v[s] = FaVec<V>::load(local_out + (int64_t)s * total + idx);
      }
      float m = l[0];
#pragma unroll
      for (int s = 1; s < SP; ++s) m = fmaxf(m, l[s]);
      float sum = 0.f;
#pragma unroll
      for (int s = 0; s < SP; ++s) {
        l[s] = m == -CUDART_INF_F ? 0.f : expf(l[s] - m);
        sum += l[s];
      }
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      V acc = FaVec<V>::zero();
#pragma unroll
      for (int s = 0; s < SP; ++s) FaVec<V>::fma(acc, l[s] * inv, v[s]);
      out[idx] = acc;
    } else {
      float m = -CUDART_INF_F;
      for (int s = 0; s < sp; ++s) m = fmaxf(m, __ldg(lse + (int64_t)s * rows + r));
      float sum = 0.f;
      for (int s = 0; s < sp; ++s) sum += m == -CUDART_INF_F ? 0.f : expf(__ldg(lse + (int64_t)s * rows + r) - m);
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      V acc = FaVec<V>::zero();
      for (int s = 0; s < sp; ++s) {
        const float w = m == -CUDART_INF_F ? 0.f : expf(__ldg(lse + (int64_t)s * rows + r) - m) * inv;
        FaVec<V>::fma(acc, w, FaVec<V>::load(local_out + (int64_t)s * total + idx));
      }
      out[idx] = acc;
    }
  }
}

template <typename V>
cudaError_t launch_fa_update(const float *lse, const void *local_out, void *out, int64_t rows, int cols, int sp,
                             int sm_count, cudaStream_t st) {
  const int64_t total = rows * cols;
  const int64_t want = (total + kFaThreads - 1) / kFaThreads;
  const unsigned grid = (unsigned)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)sm_count * 16));
  const V *in = static_cast<const V *>(local_out);
  V *o = static_cast<V *>(out);
  switch (sp) {
#define MSCO_FA_CASE(N) \
  case N: fa_update_kernel<V, N><<<grid, kFaThreads, 0, st>>>(lse, in, o, rows, cols, sp); break;
    MSCO_FA_CASE(1) MSCO_FA_CASE(2) MSCO_FA_CASE(3) MSCO_FA_CASE(4)
    MSCO_FA_CASE(5) MSCO_FA_CASE(6) MSCO_FA_CASE(7) MSCO_FA_CASE(8)
#undef MSCO_FA_CASE
    default: fa_update_kernel<V, 0><<<grid, kFaThreads, 0, st>>>(lse, in, o, rows, cols, sp); break;
  }
  return cudaGetLastError();
}

}  // namespace
}  // namespace msco

using namespace msco;

extern "C" int msco_fa_update(const float *lse, const float *local_out, float *out, int64_t rows,
                              int32_t head_size, int32_t sp, void *stream) {
  if (rows < 0 || head_size < 0 || sp < 0) return fail(MSCO_ERR_INVALID_ARG, "fa_update: negative size");
  if (sp > kFaMaxSp) return fail(MSCO_ERR_INVALID_ARG, "fa_update: sp = %d exceeds %d", sp, kFaMaxSp);
  if (rows == 0 || head_size == 0 || sp == 0) return MSCO_OK;
  if (lse == nullptr || local_out == nullptr || out == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "fa_update: lse, local_out and out must not be NULL");
  if (rows > ((int64_t)1 << 40) / head_size) return fail(MSCO_ERR_INVALID_ARG, "fa_update: too many rows");
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      sm_count = n;
    else
      sm_count = 148;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = head_size % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(local_out) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  cudaError_t e = vec ? launch_fa_update<float4>(lse, local_out, out, rows, head_size / 4, sp, sm_count, st)
                      : launch_fa_update<float>(lse, local_out, out, rows, head_size, sp, sm_count, st);
  MSCO_CUDA_CHECK(e);
  return MSCO_OK;
}
