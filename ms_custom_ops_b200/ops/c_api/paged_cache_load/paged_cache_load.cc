// paged_cache_load: operator glue for the B200 plugin.
//
// Mirrors the operator the reference registers in ops/c_api/paged_cache_load:
//   paged_cache_load_common.h:26-43     input order, ND = 0 / NZ = 1 cache formats
//   paged_cache_load_pynative.cc:48-117 eager entry: seq_lens must be int32; the output row count is
//                                       the sum of seq_lens, or its last element in cumulative mode;
//                                       key_out [sum, heads, head_size_k], value_out [sum, heads, head_size_v]
//   paged_cache_load_graph.cc:80-97    execution is skipped when an input has a zero dimension
//   paged_cache_load_doc.md:9-27        argument meaning; cumulative lengths and seq_starts are ND-only
// The device work is msco_paged_cache_load (libmsco_b200.so).  FRACTAL_NZ (kv_cache_cfg = 1) is an
// Ascend cube-unit layout and is not built for B200.
#include "ms_custom_ops_c.h"
#include "ops/framework/module.h"
#include "ops/framework/tensor.h"

namespace ms_custom_ops {
namespace {

constexpr const char *kOpName = "PagedCacheLoad";
constexpr int64_t kNdFormatType = 0, kNzFormatType = 1;

struct LoadGeometry {
  int64_t batch = 0, max_blocks = 0, block_size = 0, num_blocks = 0, heads = 0, dk = 0, dv = 0;
  bool skip = false;
};

LoadGeometry CheckInputs(const Tensor &key_cache, const Tensor &value_cache, const Tensor &block_tables,
                         const Tensor &seq_lens, const Tensor &seq_starts, int64_t kv_cache_cfg, bool cumsum,
                         bool has_seq_starts) {
  LoadGeometry g;
  if (!key_cache.defined() || !value_cache.defined() || !block_tables.defined() || !seq_lens.defined())
    MS_VALUE_ERROR << "For " << kOpName << ", key_cache, value_cache, block_tables and seq_lens must be provided.";
  if (kv_cache_cfg != kNdFormatType && kv_cache_cfg != kNzFormatType)
    MS_VALUE_ERROR << "For " << kOpName << ", kv_cache_cfg must be 0 (ND) or 1 (NZ), but got " << kv_cache_cfg << ".";
  if (kv_cache_cfg == kNzFormatType)
    MS_UNSUPPORTED << "For " << kOpName << ", kv_cache_cfg=1 (FRACTAL_NZ) is an Ascend-only cache layout; "
                   << "the B200 build supports kv_cache_cfg=0 (ND).";
  if (seq_lens.dtype() != MSCO_DTYPE_I32)
    MS_RUNTIME_ERROR << "For " << kOpName << ", the seq_lens dtype must be int32, but got : "
                     << DTypeName(seq_lens.dtype());
  if (has_seq_starts != seq_starts.defined())
    MS_VALUE_ERROR << "For " << kOpName << ", seq_starts must be given exactly when has_seq_starts is true.";
  for (const Tensor *t : {&key_cache, &value_cache, &block_tables, &seq_lens, &seq_starts})
    if (t->has_zero_dim()) {
      g.skip = true;
      return g;
    }
  auto allowed = [](int32_t dt) { return dt == MSCO_DTYPE_F16 || dt == MSCO_DTYPE_BF16 || dt == MSCO_DTYPE_I8; };
  if (!allowed(key_cache.dtype()) || !allowed(value_cache.dtype()))
    MS_TYPE_ERROR << "For " << kOpName << ", the caches must be Float16/BFloat16/Int8, but got "
                  << DTypeName(key_cache.dtype()) << " and " << DTypeName(value_cache.dtype()) << ".";
  if (key_cache.rank() != 4 || value_cache.rank() != 4)
    MS_VALUE_ERROR << "For " << kOpName << ", the ND caches must have rank 4 "
                   << "(num_blocks, block_size, num_heads, head_size).";
  if (value_cache.dim(0) != key_cache.dim(0) || value_cache.dim(1) != key_cache.dim(1) ||
      value_cache.dim(2) != key_cache.dim(2))
    MS_VALUE_ERROR << "For " << kOpName << ", key_cache and value_cache must agree in num_blocks, block_size and "
                   << "num_heads.";
  if (block_tables.dtype() != MSCO_DTYPE_I32)
    MS_TYPE_ERROR << "For " << kOpName << ", block_tables must be Int32, but got " << DTypeName(block_tables.dtype())
                  << ".";
  if (block_tables.rank() != 2)
    MS_VALUE_ERROR << "For " << kOpName << ", block_tables must have rank 2 (batch, block_indices), but got "
                   << block_tables.rank() << ".";
  if (seq_lens.rank() != 1)
    MS_VALUE_ERROR << "For " << kOpName << ", seq_lens must have rank 1, but got " << seq_lens.rank() << ".";
  g.batch = block_tables.dim(0);
  g.max_blocks = block_tables.dim(1);
  const int64_t want = cumsum ? g.batch + 1 : g.batch;
  if (seq_lens.numel() != want)
    MS_VALUE_ERROR << "For " << kOpName << ", seq_lens must have " << want << " elements ("
                   << (cumsum ? "batch + 1 running sums" : "one length per row of block_tables") << "), but got "
                   << seq_lens.numel() << ".";
  if (seq_starts.defined()) {
    if (seq_starts.dtype() != MSCO_DTYPE_I32)
      MS_TYPE_ERROR << "For " << kOpName << ", seq_starts must be Int32, but got " << DTypeName(seq_starts.dtype())
                    << ".";
    if (seq_starts.numel() != g.batch)
      MS_VALUE_ERROR << "For " << kOpName << ", seq_starts must have batch = " << g.batch << " elements, but got "
                     << seq_starts.numel() << ".";
  }
  g.num_blocks = key_cache.dim(0);
  g.block_size = key_cache.dim(1);
  g.heads = key_cache.dim(2);
  g.dk = key_cache.dim(3);
  g.dv = value_cache.dim(3);
  if (g.batch > INT32_MAX || g.max_blocks > INT32_MAX || g.block_size > INT32_MAX || g.num_blocks > INT32_MAX)
    MS_VALUE_ERROR << "For " << kOpName << ", a dimension exceeds the 32-bit range.";
  return g;
}

// Sum of the lengths when they are readable on the host, else -1 (a dynamic dimension).
int64_t SumContextLens(const Tensor &seq_lens, bool cumsum) {
  if (!seq_lens.on_host() || seq_lens.data() == nullptr || seq_lens.numel() == 0) return -1;
  const int32_t *p = static_cast<const int32_t *>(seq_lens.data());
  const int64_t n = seq_lens.numel();
  if (cumsum) return p[n - 1];
  int64_t s = 0;
  for (int64_t i = 0; i < n; ++i) s += p[i];
  return s;
}

int Infer(const Tensor &key_cache, const Tensor &value_cache, const Tensor &block_tables, const Tensor &seq_lens,
          const Tensor &seq_starts, int64_t kv_cache_cfg, bool cumsum, bool has_seq_starts, int32_t *k_dtype,
          int32_t *v_dtype, int32_t *ndim, int64_t *k_shape, int64_t *v_shape) {
  const LoadGeometry g =
      CheckInputs(key_cache, value_cache, block_tables, seq_lens, seq_starts, kv_cache_cfg, cumsum, has_seq_starts);
  const int64_t sum = g.skip ? 0 : SumContextLens(seq_lens, cumsum);
  if (k_dtype != nullptr) *k_dtype = key_cache.dtype();
  if (v_dtype != nullptr) *v_dtype = value_cache.dtype();
  if (ndim != nullptr) *ndim = 3;
  if (k_shape != nullptr) {
    k_shape[0] = sum;
    k_shape[1] = key_cache.rank() == 4 ? key_cache.dim(2) : 0;
    k_shape[2] = key_cache.rank() == 4 ? key_cache.dim(3) : 0;
  }
  if (v_shape != nullptr) {
    v_shape[0] = sum;
    v_shape[1] = value_cache.rank() == 4 ? value_cache.dim(2) : 0;
    v_shape[2] = value_cache.rank() == 4 ? value_cache.dim(3) : 0;
  }
  return MSCO_OK;
}

int Launch(const Tensor &key_cache, const Tensor &value_cache, const Tensor &block_tables, const Tensor &seq_lens,
           const Tensor &seq_starts, int64_t kv_cache_cfg, bool cumsum, bool has_seq_starts, const Tensor &key_out,
           const Tensor &value_out, void *workspace, size_t workspace_bytes, void *stream) {
  const LoadGeometry g =
      CheckInputs(key_cache, value_cache, block_tables, seq_lens, seq_starts, kv_cache_cfg, cumsum, has_seq_starts);
  if (g.skip) return MSCO_OK;
  if (!key_out.defined() || !value_out.defined())
    MS_VALUE_ERROR << "For " << kOpName << ", key_out and value_out must be provided.";
  if (seq_lens.on_host() || block_tables.on_host() || seq_starts.on_host())
    MS_RUNTIME_ERROR << "For " << kOpName << ", block_tables, seq_lens and seq_starts are read by the kernel and "
                     << "must be device tensors.";
  if (key_out.dtype() != key_cache.dtype() || value_out.dtype() != value_cache.dtype())
    MS_TYPE_ERROR << "For " << kOpName << ", key_out / value_out must have the dtypes of the caches.";
  if (key_out.rank() != 3 || value_out.rank() != 3 || key_out.dim(1) != g.heads || key_out.dim(2) != g.dk ||
      value_out.dim(1) != g.heads || value_out.dim(2) != g.dv || key_out.dim(0) != value_out.dim(0))
    MS_VALUE_ERROR << "For " << kOpName << ", key_out must be (sum_context_lens, " << g.heads << ", " << g.dk
                   << ") and value_out (sum_context_lens, " << g.heads << ", " << g.dv << ").";
  CheckContiguous(key_cache, kOpName, "key_cache");
  CheckContiguous(value_cache, kOpName, "value_cache");
  CheckContiguous(block_tables, kOpName, "block_tables");
  CheckContiguous(seq_lens, kOpName, "seq_lens");
  CheckContiguous(seq_starts, kOpName, "seq_starts");
  CheckContiguous(key_out, kOpName, "key_out");
  CheckContiguous(value_out, kOpName, "value_out");
  const int64_t ek = DTypeSize(key_cache.dtype()), ev = DTypeSize(value_cache.dtype());
  return msco_paged_cache_load(
      key_cache.data(), value_cache.data(), static_cast<const int32_t *>(block_tables.data()),
      static_cast<const int32_t *>(seq_lens.data()), static_cast<const int32_t *>(seq_starts.data()), key_out.data(),
      value_out.data(), static_cast<int32_t>(g.batch), static_cast<int32_t>(g.max_blocks),
      static_cast<int32_t>(g.block_size), static_cast<int32_t>(g.num_blocks), g.heads * g.dk * ek, g.heads * g.dv * ev,
      key_out.dim(0), cumsum ? 1 : 0, workspace, workspace_bytes, nullptr, stream);
}

}  // namespace
}  // namespace ms_custom_ops

MS_CUSTOM_OPS_REGISTER_OP(paged_cache_load,
                          "paged_cache_load(key_cache, value_cache, block_tables, seq_lens, seq_starts=None, "
                          "kv_cache_cfg=0, is_seq_lens_cumsum_type=False, has_seq_starts=False)")

extern "C" int ms_custom_ops_paged_cache_load_infer(const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                                    const MsTensorDesc *block_tables, const MsTensorDesc *seq_lens,
                                                    const MsTensorDesc *seq_starts, int64_t kv_cache_cfg,
                                                    int32_t is_seq_lens_cumsum_type, int32_t has_seq_starts,
                                                    int32_t *key_out_dtype, int32_t *value_out_dtype,
                                                    int32_t *out_ndim, int64_t *key_out_shape,
                                                    int64_t *value_out_shape) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return Infer(GetTensorOrEmpty(key_cache), GetTensorOrEmpty(value_cache), GetTensorOrEmpty(block_tables),
                 GetTensorOrEmpty(seq_lens), GetTensorOrEmpty(seq_starts), kv_cache_cfg, is_seq_lens_cumsum_type != 0,
                 has_seq_starts != 0, key_out_dtype, value_out_dtype, out_ndim, key_out_shape, value_out_shape);
  });
}

extern "C" size_t ms_custom_ops_paged_cache_load_workspace_size(const MsTensorDesc *block_tables) {
  if (block_tables == nullptr || block_tables->ndim != 2 || block_tables->shape[0] > INT32_MAX ||
      block_tables->shape[1] > INT32_MAX)
    return 0;
  return msco_paged_cache_load_workspace_bytes(static_cast<int32_t>(block_tables->shape[0]),
                                               static_cast<int32_t>(block_tables->shape[1]));
}

extern "C" int ms_custom_ops_paged_cache_load(const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                              const MsTensorDesc *block_tables, const MsTensorDesc *seq_lens,
                                              const MsTensorDesc *seq_starts, int64_t kv_cache_cfg,
                                              int32_t is_seq_lens_cumsum_type, int32_t has_seq_starts,
                                              const MsTensorDesc *key_out, const MsTensorDesc *value_out,
                                              void *workspace, size_t workspace_bytes, void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return Launch(GetTensorOrEmpty(key_cache), GetTensorOrEmpty(value_cache), GetTensorOrEmpty(block_tables),
                  GetTensorOrEmpty(seq_lens), GetTensorOrEmpty(seq_starts), kv_cache_cfg,
                  is_seq_lens_cumsum_type != 0, has_seq_starts != 0, GetTensorOrEmpty(key_out),
                  GetTensorOrEmpty(value_out), workspace, workspace_bytes, stream);
  });
}
