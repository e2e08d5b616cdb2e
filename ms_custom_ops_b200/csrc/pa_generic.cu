// Paged-attention decode: general-shape kernel and the split-KV reduce kernel.
//
// pa_generic_kernel covers every shape the operator accepts (any head_dim up
// to 256, any block size, additive NORM / ALIBI masks, int8 KV with offsets)
// with CUDA-core float32 arithmetic.  The TMA + tensor-core kernel in
// pa_tma.cu takes over for head_dim 128 without a mask; both follow the same
// plan (same work items, same split boundaries, same partial format).
//
// pa_reduce_kernel merges the per-split partials (running max m in the log2
// domain, running sum l, un-normalised output O) in split order:
//   M = max_s m_s,  out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s
// which is the log-sum-exp merge of the reference's fa_update golden
// (tests/st/test_asd_faupdate.py:34-59) written for un-normalised partials.
#include <math_constants.h>

#include "msco_common.cuh"
#include "pa_merge.cuh"
#include "pa_params.h"
#include "peer_gather.cuh"

namespace msco {
namespace {

constexpr int kGenThreads = 128;
constexpr int kGenWarps = kGenThreads / 32;
constexpr int kGenRows = 8;    // q rows per work item
constexpr int kGenMaxD = 256;  // head_dim limit
constexpr int kGenDL = kGenMaxD / 32;
constexpr float kNeg = -1.0e30f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float load_mask(const void *mask, int dtype, int64_t idx) {
  if (dtype == MSCO_DTYPE_F16) return __half2float(static_cast<const __half *>(mask)[idx]);
  if (dtype == MSCO_DTYPE_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(mask)[idx]);
  return static_cast<const float *>(mask)[idx];
}

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(kGenThreads) pa_generic_kernel(PaParams p, const __grid_constant__ PlanParam pp) {
  __shared__ float q_s[kGenRows][kGenMaxD];            // q (times k_descale for int8 KV)
  __shared__ float koff_s[kGenMaxD];                    // k_offset of this kv head (int8 KV)
  __shared__ float acc_s[kGenWarps][kGenRows][kGenMaxD];
  __shared__ float m_s[kGenWarps][kGenRows], l_s[kGenWarps][kGenRows];
  __shared__ WorkItem item_s;

  const PlanView pv = make_plan_view(p.plan_in_param ? pp.w : p.plan);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) item_s = decode_item(pv, blockIdx.x, p.num_kv_heads, p.group, kGenRows);
  __syncthreads();
  const WorkItem w = item_s;
  const int D = p.head_dim;
  const int hq0 = w.kvh * p.group + w.row0;  // first q head of this item
  constexpr bool kInt8 = sizeof(TKV) == 1;

  const TQ *q = static_cast<const TQ *>(p.q) + ((int64_t)w.b * p.num_q_heads + hq0) * D;
  for (int i = threadIdx.x; i < kGenRows * D; i += kGenThreads) {
    const int r = i / D, d = i - r * D;
    float v = (r < w.nrows) ? to_f32<TQ>(q[(int64_t)r * D + d]) : 0.f;
    if (kInt8) v *= __ldg(p.k_descale + w.kvh * D + d);
    q_s[r][d] = v;
  }
  if (kInt8) {
    for (int d = threadIdx.x; d < D; d += kGenThreads)
      koff_s[d] = p.k_offset ? (float)__ldg(p.k_offset + w.kvh * D + d) : 0.f;
  }
  __syncthreads();

  float m[kGenRows], l[kGenRows], acc[kGenRows][kGenDL];
#pragma unroll
  for (int r = 0; r < kGenRows; ++r) {
    m[r] = kNeg;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < kGenDL; ++i) acc[r][i] = 0.f;
  }

  const TKV *kc = static_cast<const TKV *>(p.key_cache);
  const TKV *vc = static_cast<const TKV *>(p.value_cache);
  const int64_t tok_stride = (int64_t)p.num_kv_heads * D;  // elements between tokens of a block
  const int32_t *trow = p.block_tables + (int64_t)w.b * p.max_blocks_per_seq;
  const float log2e = 1.4426950408889634f;

  // each warp takes 32 tokens at a time, round-robin over the item's range
  for (int base = w.tok0 + warp * 32; base < w.tok1; base += kGenWarps * 32) {
    const int tok = base + lane;
    bool valid = tok < w.tok1;
    int64_t row_off = 0;
    if (valid) {
      const int blk = __ldg(trow + tok / p.block_size);
      if (blk < 0 || blk >= p.num_blocks) {
        report_status(p.status, p.epoch, kStatusOob);
        valid = false;
      } else {
        row_off = p.cache_layout == 0
                      ? ((int64_t)blk * p.block_size + tok % p.block_size) * tok_stride + (int64_t)w.kvh * D
                      : (((int64_t)blk * p.num_kv_heads + w.kvh) * p.block_size + tok % p.block_size) * D;
      }
    }
    // scores of this lane's token against every q row
    float s[kGenRows];
#pragma unroll
    for (int r = 0; r < kGenRows; ++r) s[r] = 0.f;
    if (valid) {
      const TKV *krow = kc + row_off;
      for (int d = 0; d < D; ++d) {
        float kv = to_f32<TKV>(krow[d]);
        if (kInt8) kv += koff_s[d];
#pragma unroll
        for (int r = 0; r < kGenRows; ++r) s[r] = fmaf(q_s[r][d], kv, s[r]);
      }
    }
    float pr[kGenRows];
#pragma unroll
    for (int r = 0; r < kGenRows; ++r) {
      float x = kNeg;
      if (valid) {
        x = s[r] * p.scale;
        if (p.mask_type != 0 && r < w.nrows) {
          const int64_t mi = (int64_t)w.b * p.mask_batch_stride + (int64_t)(hq0 + r) * p.mask_head_stride + tok;
          x += load_mask(p.mask, p.mask_dtype, mi);
        }
        x *= log2e;
      }
      const float mnew = fmaxf(m[r], warp_max(x));
      const float alpha = exp2f(m[r] - mnew);
      const float pe = valid ? exp2f(x - mnew) : 0.f;
      l[r] = l[r] * alpha + warp_sum(pe);
      m[r] = mnew;
      pr[r] = pe;
#pragma unroll
      for (int i = 0; i < kGenDL; ++i) acc[r][i] *= alpha;
    }
    // O += P V over the 32 tokens of this group
    const int nvalid = min(32, w.tok1 - base);
    for (int j = 0; j < nvalid; ++j) {
      const int64_t voff = __shfl_sync(0xffffffffu, row_off, j);
      const bool vj = __shfl_sync(0xffffffffu, (int)valid, j) != 0;
      float pj[kGenRows];
#pragma unroll
      for (int r = 0; r < kGenRows; ++r) pj[r] = __shfl_sync(0xffffffffu, pr[r], j);
      if (!vj) continue;
      const TKV *vrow = vc + voff;
#pragma unroll
      for (int i = 0; i < kGenDL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) {
          const float vv = to_f32<TKV>(vrow[d]);
#pragma unroll
          for (int r = 0; r < kGenRows; ++r) acc[r][i] = fmaf(pj[r], vv, acc[r][i]);
        }
      }
    }
  }

  // merge the warps' running states
#pragma unroll
  for (int r = 0; r < kGenRows; ++r) {
    if (lane == 0) {
      m_s[warp][r] = m[r];
      l_s[warp][r] = l[r];
    }
#pragma unroll
    for (int i = 0; i < kGenDL; ++i) {
      const int d = lane + 32 * i;
      if (d < D) acc_s[warp][r][d] = acc[r][i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < w.nrows * D; i += kGenThreads) {
    const int r = i / D, d = i - r * D;
    float M = m_s[0][r];
#pragma unroll
    for (int ww = 1; ww < kGenWarps; ++ww) M = fmaxf(M, m_s[ww][r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int ww = 0; ww < kGenWarps; ++ww) {
      const float f = exp2f(m_s[ww][r] - M);
      L = fmaf(l_s[ww][r], f, L);
      O = fmaf(acc_s[ww][r][d], f, O);
    }
    const int hq = hq0 + r;
    if (w.nsplit == 1) {
      float o = O / L;
      if (kInt8) {
        const float vo = p.v_offset ? (float)__ldg(p.v_offset + w.kvh * D + d) : 0.f;
        o = (o + vo) * __ldg(p.v_descale + w.kvh * D + d);
      }
      static_cast<TQ *>(p.out)[((int64_t)w.b * p.num_q_heads + hq) * D + d] = from_f32<TQ>(o);
      if (d == 0 && p.lse != nullptr) p.lse[(int64_t)w.b * p.num_q_heads + hq] = (M + log2f(L)) * kLn2;
    } else {
      const int64_t prow = (int64_t)w.part * p.num_q_heads + hq;
      p.part_o[prow * D + d] = O;
      if (d == 0) {
        p.part_ml[prow * 2] = M;
        p.part_ml[prow * 2 + 1] = L;
      }
    }
  }
}

// One warp per (sequence, q head) output row.  The (m, l) pairs of up to 32 splits are loaded by
// the lanes in parallel (one split per lane, strided for more), the weights 2^(m_s - M) stay in
// registers, and the partial rows are accumulated in split order with several loads in flight.
template <typename TQ, int PF>
__device__ __forceinline__ void reduce_row(const PaParams &p, const PlanView &pv, int row, int lane) {
  const int b = row / p.num_q_heads, hq = row - b * p.num_q_heads;
  const int ns = __ldg(pv.b_nsplit + b);
  if (ns == 1) return;  // written directly by the attention kernel
  const int D = p.head_dim;
  TQ *out = static_cast<TQ *>(p.out) + (int64_t)row * D;
  if (ns == 0) {  // empty sequence: zeros, as the reference golden does; no token: lse = -inf
    for (int d = lane; d < D; d += 32) out[d] = from_f32<TQ>(0.f);
    if (lane == 0 && p.lse != nullptr) p.lse[row] = -CUDART_INF_F;
    return;
  }
  const int base = __ldg(pv.b_part_base + b);
  // same code as the TMA kernel's own epilogue: identical bits
  if (D == 128) { merge_row<TQ, 128, PF>(p, row, hq, ns, base, lane); return; }
  if (D == 64) { merge_row<TQ, 64, PF>(p, row, hq, ns, base, lane); return; }
  if (D == 256) { merge_row<TQ, 256>(p, row, hq, ns, base, lane); return; }  // (8 columns per lane: no batches, the registers of every launch would pay for them)
  const int64_t hq_stride = p.num_q_heads;
  // pass 1: M = max_s m_s (lanes stride over the splits)
  float M = kNeg;
  for (int s = lane; s < ns; s += 32)
    M = fmaxf(M, __ldg(p.part_ml + ((int64_t)(base + s) * hq_stride + hq) * 2));
  M = warp_max(M);
  const int kvh = hq / p.group;
  float L = 0.f;
  float o[kGenDL];
#pragma unroll
  for (int i = 0; i < kGenDL; ++i) o[i] = 0.f;
  for (int s = 0; s < ns; ++s) {  // fixed split order: bit-reproducible
    const int64_t prow = (int64_t)(base + s) * hq_stride + hq;
    const float f = exp2f(__ldg(p.part_ml + prow * 2) - M);
    L = fmaf(__ldg(p.part_ml + prow * 2 + 1), f, L);
#pragma unroll
    for (int i = 0; i < kGenDL; ++i) {
      const int d = lane + 32 * i;
      if (d < D) o[i] = fmaf(__ldg(p.part_o + prow * D + d), f, o[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < kGenDL; ++i) {
    const int d = lane + 32 * i;
    if (d < D) {
      float v = o[i] / L;
      if (p.v_descale != nullptr) {
        const float vo = p.v_offset ? (float)__ldg(p.v_offset + kvh * D + d) : 0.f;
        v = (v + vo) * __ldg(p.v_descale + kvh * D + d);
      }
      out[d] = from_f32<TQ>(v);
    }
  }
  if (lane == 0 && p.lse != nullptr) p.lse[row] = (M + log2f(L)) * kLn2;
}

// The kernel that finishes the output rows of a launch: merges the rows that were computed in
// several splits and -- for a rank of a kv-head-sharded step (g.world > 0) -- stores every finished
// row, merged here or written by the attention kernel, into slot `rank` of every rank's gathered
// buffer; the block that finishes last then publishes the step's flag and waits (bounded) for the
// peers, exactly as the stand-alone gather kernel does.
// PF: how many partial rows a lane requests at a time (see merge_row).  0 (56 registers, loads inside the
// loop) for grids of more than eight blocks per SM, where occupancy hides the latency better than
// prefetching does; otherwise 32 for launches with rows of more than 16 splits (long contexts; 190
// registers), and 16 when the grid fits the SMs in one wave at the 110 registers that costs.
template <typename TQ, int PW, int PF>
__global__ void __launch_bounds__(128)
pa_reduce_kernel(PaParams p, const __grid_constant__ PlanParamT<PW> pp, const __grid_constant__ GatherArgs g) {
  __shared__ bool is_last;
  // a kernel launched behind this one with programmatic stream serialisation may become resident
  // now; it waits for this grid before it reads the output
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // launched with programmatic stream serialisation: wait here until the attention grid before us
  // has completed and its partials are visible (a no-op for an ordinary launch)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const PlanView pv = make_plan_view(p.plan_in_param ? pp.w : p.plan);
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const bool live = row < pv.batch * p.num_q_heads;
  if (live) reduce_row<TQ, PF>(p, pv, row, lane);
  if (g.world == 0) return;
  const int64_t row_bytes = (int64_t)p.head_dim * (int64_t)sizeof(TQ);
  const char *src = static_cast<const char *>(p.out) + row * row_bytes;
  if (g.packets[0] != nullptr) {
    // packet form: every lane sends its 16 bytes of the row to the peers (and stores them into its own
    // gathered buffer), then waits for the same 16 bytes of every peer's row and copies them in.  No
    // fence, no flag, no last block: a lane depends on nothing but the packets it waits for.
    if (live) {
      __syncwarp();  // the row was written by the lanes of this warp (or by the grid before us)
      for (int64_t off = lane * 16; off < row_bytes; off += 32 * 16) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(src + off));
        *reinterpret_cast<uint4 *>(static_cast<char *>(g.gathered[g.rank]) + (int64_t)g.rank * g.slice_bytes +
                                   row * row_bytes + off) = v;
        packets_push16(g, row * row_bytes + off, v);
      }
      bool ok = true;
      for (int64_t off = lane * 16; off < row_bytes; off += 32 * 16) ok = packets_pull16(g, row * row_bytes + off) && ok;
      if (!ok) atomicExch(g.status, kStatusTimeout);  // a peer never sent: report, do not hang
    }
    return;
  }
  if (live) {
    __syncwarp();  // the row was written by the lanes of this warp (or by the grid before us)
    for (int64_t off = lane * 16; off < row_bytes; off += 32 * 16)
      gather_push16(g, row * row_bytes + off, __ldcg(reinterpret_cast<const uint4 *>(src + off)));
  }
  gather_finish(g, &is_last);
}

}  // namespace

int launch_pa_generic(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, cudaStream_t stream) {
  if (plan->total_items == 0) return MSCO_OK;
  const dim3 grid(plan->total_items), block(kGenThreads);
  const int qd = plan->desc.q_dtype, kd = plan->desc.kv_dtype;
  if (qd == MSCO_DTYPE_F16 && kd == MSCO_DTYPE_F16) pa_generic_kernel<__half, __half><<<grid, block, 0, stream>>>(p, pp);
  else if (qd == MSCO_DTYPE_BF16 && kd == MSCO_DTYPE_BF16) pa_generic_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, block, 0, stream>>>(p, pp);
  else if (qd == MSCO_DTYPE_F16 && kd == MSCO_DTYPE_I8) pa_generic_kernel<__half, int8_t><<<grid, block, 0, stream>>>(p, pp);
  else if (qd == MSCO_DTYPE_BF16 && kd == MSCO_DTYPE_I8) pa_generic_kernel<__nv_bfloat16, int8_t><<<grid, block, 0, stream>>>(p, pp);
  else return fail(MSCO_ERR_UNSUPPORTED, "paged_attention: unsupported dtype combination q=%d kv=%d", qd, kd);
  MSCO_CUDA_CHECK(cudaGetLastError());
  return MSCO_OK;
}

int launch_pa_reduce(const MscoPaPlan *plan, const PaParams &p, const PlanParam &pp, cudaStream_t stream,
                     const GatherArgs *gather) {
  static const GatherArgs no_gather = {};
  const GatherArgs &g = gather != nullptr ? *gather : no_gather;
  const int rows = plan->batch * plan->desc.num_q_heads;
  if (rows == 0) return MSCO_OK;
  if (g.world > 0) {
    const int64_t row_bytes = (int64_t)plan->desc.head_dim * 2;
    if (row_bytes % 16 != 0 || g.slice_bytes != rows * row_bytes)
      return fail(MSCO_ERR_INVALID_ARG, "decode_step_gather: the gather slice is %lld bytes, the output of this plan %lld",
                  (long long)g.slice_bytes, (long long)(rows * row_bytes));
    if (reinterpret_cast<uintptr_t>(p.out) & 15)
      return fail(MSCO_ERR_INVALID_ARG, "decode_step_gather: the output must be 16-byte aligned");
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((rows + 3) / 4);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const bool f16 = plan->desc.q_dtype == MSCO_DTYPE_F16;
  const int blocks = (rows + 3) / 4;
  const int pf = blocks > 8 * plan->num_sms ? 0 : (plan->max_splits > 16 ? 32 : (blocks <= 4 * plan->num_sms ? 16 : 0));
#define MSCO_RK(T, PW, PP)                                                                                 \
  do {                                                                                                    \
    if (pf == 32) MSCO_CUDA_CHECK(cudaLaunchKernelEx(&cfg, pa_reduce_kernel<T, PW, 32>, p, PP, g));       \
    else if (pf == 16) MSCO_CUDA_CHECK(cudaLaunchKernelEx(&cfg, pa_reduce_kernel<T, PW, 16>, p, PP, g));  \
    else MSCO_CUDA_CHECK(cudaLaunchKernelEx(&cfg, pa_reduce_kernel<T, PW, 0>, p, PP, g));                 \
  } while (0)
  if (p.plan_in_param && plan->plan_words <= (size_t)kPlanParamWordsSmall) {  // see PlanParamSmall
    const PlanParamSmall &ps = *reinterpret_cast<const PlanParamSmall *>(&pp);
    if (f16) MSCO_RK(__half, kPlanParamWordsSmall, ps); else MSCO_RK(__nv_bfloat16, kPlanParamWordsSmall, ps);
  } else {
    if (f16) MSCO_RK(__half, kPlanParamWords, pp); else MSCO_RK(__nv_bfloat16, kPlanParamWords, pp);
  }
#undef MSCO_RK
  return MSCO_OK;
}

}  // namespace msco
