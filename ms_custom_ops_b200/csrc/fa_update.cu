// fa_update for B200: merge `sp` partial attention outputs of the same rows by their log-sum-exps,
//   out[r, :] = sum_s w[s, r] * local_out[s, r, :],   w[s, r] = exp(lse[s, r]) / sum_s' exp(lse[s', r])
// (the DECODE_UPDATE of the reference: ops/c_api/fa_update/fa_update_doc.md:3-24, golden
// tests/st/test_asd_faupdate.py:34-59).  The operator is float32 throughout; the strided entry point
// also takes fp16 / bf16 partial outputs (what paged attention writes) with any distance between
// the partitions, so that an all-gathered buffer is merged in place.
//
// HBM-bound: sp * head_size * e bytes read and head_size * e written per row.  One thread owns four
// consecutive columns of one row; all sp loads are issued before the first use.  The weights are
// computed with the row maximum subtracted (same value, no overflow); a row whose lse are all -inf
// (no partition saw a token) gives zeros.
#include <math_constants.h>

#include <algorithm>

#include "msco_common.cuh"

namespace msco {
namespace {

constexpr int kFaThreads = 256;
constexpr int kFaMaxSp = 64;

// four consecutive columns of a row, in registers as float4
template <typename T> struct Quad;
template <> struct Quad<float> {
  static __device__ __forceinline__ float4 load(const float *p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
  }
  static __device__ __forceinline__ void store(float *p, const float4 &v) { *reinterpret_cast<float4 *>(p) = v; }
};
template <> struct Quad<__half> {
  static __device__ __forceinline__ float4 load(const __half *p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__half *p, const float4 &v) {
    uint2 r;
    r.x = pack2<__half>(v.x, v.y);
    r.y = pack2<__half>(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = r;
  }
};
template <> struct Quad<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16 *p) {
    const uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float4 &v) {
    uint2 r;
    r.x = pack2<__nv_bfloat16>(v.x, v.y);
    r.y = pack2<__nv_bfloat16>(v.z, v.w);
    *reinterpret_cast<uint2 *>(p) = r;
  }
};

__device__ __forceinline__ void axpy4(float4 &a, float w, const float4 &v) {
  a.x = fmaf(w, v.x, a.x); a.y = fmaf(w, v.y, a.y); a.z = fmaf(w, v.z, a.z); a.w = fmaf(w, v.w, a.w);
}

// SP > 0: compile-time partition count, everything in registers.  SP == 0: run-time count.
// Partition s starts lse_stride floats / in_stride elements after partition s - 1.
template <typename T, int SP>
__global__ void __launch_bounds__(kFaThreads)
fa_update_kernel(const float *__restrict__ lse, int64_t lse_stride, const T *__restrict__ local_out,
                 int64_t in_stride, T *__restrict__ out, int64_t rows, int quads /* per row */, int sp_rt) {
  const int sp = SP > 0 ? SP : sp_rt;
  const int64_t total = rows * quads;
  const int64_t stride = (int64_t)gridDim.x * kFaThreads;
  for (int64_t idx = (int64_t)blockIdx.x * kFaThreads + threadIdx.x; idx < total; idx += stride) {
    const int64_t r = idx / quads;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if constexpr (SP > 0) {
      float l[SP > 0 ? SP : 1];
      float4 v[SP > 0 ? SP : 1];
#pragma unroll
      for (int s = 0; s < SP; ++s) {
        l[s] = __ldg(lse + s * lse_stride + r);
        v[s] = Quad<T>::load(local_out + s * in_stride + idx * 4);
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
#pragma unroll
      for (int s = 0; s < SP; ++s) axpy4(acc, l[s] * inv, v[s]);
    } else {
      float m = -CUDART_INF_F;
      for (int s = 0; s < sp; ++s) m = fmaxf(m, __ldg(lse + s * lse_stride + r));
      float sum = 0.f;
      for (int s = 0; s < sp; ++s) sum += m == -CUDART_INF_F ? 0.f : expf(__ldg(lse + s * lse_stride + r) - m);
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      for (int s = 0; s < sp; ++s) {
        const float w = m == -CUDART_INF_F ? 0.f : expf(__ldg(lse + s * lse_stride + r) - m) * inv;
        axpy4(acc, w, Quad<T>::load(local_out + s * in_stride + idx * 4));
      }
    }
    Quad<T>::store(out + idx * 4, acc);
  }
}

// float32 rows whose size or address rules out 16-byte accesses: one column per thread
__global__ void __launch_bounds__(kFaThreads)
fa_update_scalar_kernel(const float *__restrict__ lse, const float *__restrict__ local_out, float *__restrict__ out,
                        int64_t rows, int cols, int sp) {
  const int64_t total = rows * cols;
  const int64_t stride = (int64_t)gridDim.x * kFaThreads;
  for (int64_t idx = (int64_t)blockIdx.x * kFaThreads + threadIdx.x; idx < total; idx += stride) {
    const int64_t r = idx / cols;
    float m = -CUDART_INF_F;
    for (int s = 0; s < sp; ++s) m = fmaxf(m, __ldg(lse + s * rows + r));
    float sum = 0.f;
    for (int s = 0; s < sp; ++s) sum += m == -CUDART_INF_F ? 0.f : expf(__ldg(lse + s * rows + r) - m);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    float acc = 0.f;
    for (int s = 0; s < sp; ++s) {
      const float w = m == -CUDART_INF_F ? 0.f : expf(__ldg(lse + s * rows + r) - m) * inv;
      acc = fmaf(w, __ldg(local_out + s * total + idx), acc);
    }
    out[idx] = acc;
  }
}

int sm_count() {
  static int n_sm = 0;
  if (n_sm == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      n_sm = n;
    else
      n_sm = 148;
  }
  return n_sm;
}

unsigned grid_for(int64_t work_items) {
  const int64_t want = (work_items + kFaThreads - 1) / kFaThreads;
  return (unsigned)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)sm_count() * 16));
}

template <typename T>
cudaError_t launch_fa_update(const float *lse, int64_t lse_stride, const void *local_out, int64_t in_stride,
                             void *out, int64_t rows, int quads, int sp, cudaStream_t st) {
  const unsigned grid = grid_for(rows * quads);
  const T *in = static_cast<const T *>(local_out);
  T *o = static_cast<T *>(out);
  switch (sp) {
#define MSCO_FA_CASE(N)                                                                                           \
  case N:                                                                                                         \
    fa_update_kernel<T, N><<<grid, kFaThreads, 0, st>>>(lse, lse_stride, in, in_stride, o, rows, quads, sp);     \
    break;
    MSCO_FA_CASE(1) MSCO_FA_CASE(2) MSCO_FA_CASE(3) MSCO_FA_CASE(4)
    MSCO_FA_CASE(5) MSCO_FA_CASE(6) MSCO_FA_CASE(7) MSCO_FA_CASE(8)
#undef MSCO_FA_CASE
    default:
      fa_update_kernel<T, 0><<<grid, kFaThreads, 0, st>>>(lse, lse_stride, in, in_stride, o, rows, quads, sp);
      break;
  }
  return cudaGetLastError();
}

int check_sizes(const char *who, int64_t rows, int32_t head_size, int32_t sp) {
  if (rows < 0 || head_size < 0 || sp < 0) return fail(MSCO_ERR_INVALID_ARG, "%s: negative size", who);
  if (sp > kFaMaxSp) return fail(MSCO_ERR_INVALID_ARG, "%s: sp = %d exceeds %d", who, sp, kFaMaxSp);
  if (head_size > 0 && rows > ((int64_t)1 << 40) / head_size)
    return fail(MSCO_ERR_INVALID_ARG, "%s: too many rows", who);
  return MSCO_OK;
}

}  // namespace
}  // namespace msco

using namespace msco;

extern "C" int msco_fa_update(const float *lse, const float *local_out, float *out, int64_t rows,
                              int32_t head_size, int32_t sp, void *stream) {
  if (int rc = check_sizes("fa_update", rows, head_size, sp)) return rc;
  if (rows == 0 || head_size == 0 || sp == 0) return MSCO_OK;
  if (lse == nullptr || local_out == nullptr || out == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "fa_update: lse, local_out and out must not be NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = head_size % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(local_out) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (vec) {
    MSCO_CUDA_CHECK(launch_fa_update<float>(lse, rows, local_out, rows * head_size, out, rows, head_size / 4, sp, st));
  } else {
    fa_update_scalar_kernel<<<grid_for(rows * head_size), kFaThreads, 0, st>>>(lse, local_out, out, rows, head_size,
                                                                                sp);
    MSCO_CUDA_CHECK(cudaGetLastError());
  }
  return MSCO_OK;
}

extern "C" int msco_fa_update_strided(const float *lse, int64_t lse_stride, const void *local_out,
                                      int64_t local_out_stride, int32_t dtype, void *out, int64_t rows,
                                      int32_t head_size, int32_t sp, void *stream) {
  if (int rc = check_sizes("fa_update_strided", rows, head_size, sp)) return rc;
  if (dtype != MSCO_DTYPE_F32 && dtype != MSCO_DTYPE_F16 && dtype != MSCO_DTYPE_BF16)
    return fail(MSCO_ERR_INVALID_ARG, "fa_update_strided: local_out / out must be float32, float16 or bfloat16");
  if (rows == 0 || head_size == 0 || sp == 0) return MSCO_OK;
  if (lse == nullptr || local_out == nullptr || out == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "fa_update_strided: lse, local_out and out must not be NULL");
  const int es = dtype_size(dtype);
  const uintptr_t quad = (uintptr_t)(4 * es) - 1;  // 16-byte (float32) or 8-byte accesses
  if (head_size % 4 != 0 || lse_stride < rows || local_out_stride < rows * head_size ||
      ((reinterpret_cast<uintptr_t>(local_out) | reinterpret_cast<uintptr_t>(out) |
        (uintptr_t)(local_out_stride * es)) & quad) != 0)
    return fail(MSCO_ERR_INVALID_ARG,
                "fa_update_strided: head_size must be a multiple of 4, the strides at least one partition, and "
                "local_out, out and the partition stride aligned to four elements");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (dtype == MSCO_DTYPE_F32)
    e = launch_fa_update<float>(lse, lse_stride, local_out, local_out_stride, out, rows, head_size / 4, sp, st);
  else if (dtype == MSCO_DTYPE_F16)
    e = launch_fa_update<__half>(lse, lse_stride, local_out, local_out_stride, out, rows, head_size / 4, sp, st);
  else
    e = launch_fa_update<__nv_bfloat16>(lse, lse_stride, local_out, local_out_stride, out, rows, head_size / 4, sp, st);
  MSCO_CUDA_CHECK(e);
  return MSCO_OK;
}
