// fa_update: operator glue for the B200 plugin.
//
// Mirrors the operator the reference registers in ops/c_api/fa_update:
//   fa_update_common.h:23-37       input order lse, local_out, fa_update_type, sp; local_out has rank 3
//   fa_update_pynative.cc:48-77    eager entry: rank and head_size checks, output (rows, head_size)
//   fa_update_graph.cc:23-42       the same checks at infer time; the output is Float32
//   fa_update_doc.md:7-24          lse (sp, rows) and local_out (sp, rows, head_size) are Float32,
//                                  fa_update_type 0 = DECODE_UPDATE is the only mode, sp in [1, 8]
// The device work is msco_fa_update (libmsco_b200.so).
#include "ms_custom_ops_c.h"
#include "ops/framework/module.h"
#include "ops/framework/tensor.h"

namespace ms_custom_ops {
namespace {

constexpr const char *kOpName = "FaUpdate";
constexpr int64_t kHeadSizeMin = 8, kHeadSizeMax = 512, kSpMax = 8;

struct MergeGeometry {
  int64_t sp = 0, rows = 0, head_size = 0;
};

MergeGeometry CheckInputs(const Tensor &lse, const Tensor &local_out, int64_t fa_update_type, int64_t sp) {
  MergeGeometry g;
  if (!lse.defined() || !local_out.defined())
    MS_VALUE_ERROR << "For " << kOpName << ", lse and local_out must be provided.";
  if (local_out.rank() != 3)
    MS_VALUE_ERROR << "For " << kOpName << ", local_out dim must be 3, but got : " << local_out.rank();
  g.head_size = local_out.dim(2);
  if (g.head_size < kHeadSizeMin || g.head_size > kHeadSizeMax || (g.head_size & 7) != 0)
    MS_VALUE_ERROR << "For " << kOpName << ", head_size must be in range [8, 512] and be the multiple of 8, "
                   << "but got : " << g.head_size;
  if (fa_update_type != 0)
    MS_VALUE_ERROR << "For " << kOpName << ", fa_update_type must be 0 (DECODE_UPDATE), but got " << fa_update_type
                   << ".";
  if (sp < 1 || sp > kSpMax)
    MS_VALUE_ERROR << "For " << kOpName << ", sp must be in range [1, 8], but got " << sp << ".";
  if (lse.dtype() != MSCO_DTYPE_F32 || local_out.dtype() != MSCO_DTYPE_F32)
    MS_TYPE_ERROR << "For " << kOpName << ", lse and local_out must be Float32, but got " << DTypeName(lse.dtype())
                  << " and " << DTypeName(local_out.dtype()) << ".";
  g.sp = local_out.dim(0);
  g.rows = local_out.dim(1);
  if (g.sp != sp)
    MS_VALUE_ERROR << "For " << kOpName << ", local_out holds " << g.sp << " partitions but sp is " << sp << ".";
  if (lse.rank() != 2 || lse.dim(0) != g.sp || lse.dim(1) != g.rows)
    MS_VALUE_ERROR << "For " << kOpName << ", lse must be (sp, rows) = (" << g.sp << ", " << g.rows << ").";
  return g;
}

int Infer(const Tensor &lse, const Tensor &local_out, int64_t fa_update_type, int64_t sp, int32_t *out_dtype,
          int32_t *out_ndim, int64_t *out_shape) {
  const MergeGeometry g = CheckInputs(lse, local_out, fa_update_type, sp);
  if (out_dtype != nullptr) *out_dtype = MSCO_DTYPE_F32;
  if (out_ndim != nullptr) *out_ndim = 2;
  if (out_shape != nullptr) {
    out_shape[0] = g.rows;
    out_shape[1] = g.head_size;
  }
  return MSCO_OK;
}

int Launch(const Tensor &lse, const Tensor &local_out, int64_t fa_update_type, int64_t sp, const Tensor &output,
           void *stream) {
  const MergeGeometry g = CheckInputs(lse, local_out, fa_update_type, sp);
  if (!output.defined()) MS_VALUE_ERROR << "For " << kOpName << ", output must be provided.";
  if (output.dtype() != MSCO_DTYPE_F32)
    MS_TYPE_ERROR << "For " << kOpName << ", output must be Float32, but got " << DTypeName(output.dtype()) << ".";
  if (output.rank() != 2 || output.dim(0) != g.rows || output.dim(1) != g.head_size)
    MS_VALUE_ERROR << "For " << kOpName << ", output must be (" << g.rows << ", " << g.head_size << ").";
  if (lse.on_host() || local_out.on_host() || output.on_host())
    MS_RUNTIME_ERROR << "For " << kOpName << ", lse, local_out and output must be device tensors.";
  CheckContiguous(lse, kOpName, "lse");
  CheckContiguous(local_out, kOpName, "local_out");
  CheckContiguous(output, kOpName, "output");
  return msco_fa_update(static_cast<const float *>(lse.data()), static_cast<const float *>(local_out.data()),
                        static_cast<float *>(output.data()), g.rows, static_cast<int32_t>(g.head_size),
                        static_cast<int32_t>(g.sp), stream);
}

}  // namespace
}  // namespace ms_custom_ops

MS_CUSTOM_OPS_REGISTER_OP(fa_update, "fa_update(lse, local_out, fa_update_type=0, sp=1)")

extern "C" int ms_custom_ops_fa_update_infer(const MsTensorDesc *lse, const MsTensorDesc *local_out,
                                             int64_t fa_update_type, int64_t sp, int32_t *out_dtype,
                                             int32_t *out_ndim, int64_t *out_shape) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return Infer(GetTensorOrEmpty(lse), GetTensorOrEmpty(local_out), fa_update_type, sp, out_dtype, out_ndim,
                 out_shape);
  });
}

extern "C" int ms_custom_ops_fa_update(const MsTensorDesc *lse, const MsTensorDesc *local_out,
                                       int64_t fa_update_type, int64_t sp, const MsTensorDesc *output,
                                       void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return Launch(GetTensorOrEmpty(lse), GetTensorOrEmpty(local_out), fa_update_type, sp, GetTensorOrEmpty(output),
                  stream);
  });
}
