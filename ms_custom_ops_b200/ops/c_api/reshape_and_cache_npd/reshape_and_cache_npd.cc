// reshape_and_cache_npd: operator glue for the B200 plugin (cache write in either block layout).
//
// The reference registers this operator in ops/ascendc/ms_glue/reshape_and_cache_npd
// (reshape_and_cache_npd_op.yaml; argument meaning reshape_and_cache_npd.md:11-34; device code
// ops/ascendc/aclnn_src/reshape_and_cache_npd/op_kernel/reshape_and_cache_npd.cpp:145-179).  It writes the
// token rows into the paged caches in one of two block layouts,
//   "BSND"  (num_blocks, block_size, heads, head_dim)   -- what reshape_and_cache writes
//   "BNSD"  (num_blocks, heads, block_size, head_dim)   -- head-major: one head's rows of a block are contiguous
// and returns the current key / value in the "TH" layout (tokens, heads * head_dim) or re-blocked ("NPD",
// together with the cached history).  Built here: both cache layouts with the "TH" outputs (copies of
// key / value, tests/st/test_custom_reshape_and_cache_npd.py:573-577); the re-blocked "NPD" outputs are an
// input format of the Ascend attention kernels and raise an "unsupported" error.
#include <cstring>

#include "ms_custom_ops_c.h"
#include "ops/framework/module.h"
#include "ops/framework/tensor.h"

namespace ms_custom_ops {
namespace {

constexpr const char *kOpName = "ReshapeAndCacheNpd";

struct NpdGeometry {
  bool head_major = false, skip = false;
  int64_t num_tokens = 0, heads = 0, k_head = 0, v_head = 0, block_size = 0, num_slots = 0;
};

bool Is(const char *s, const char *a, const char *b) { return s != nullptr && (!strcmp(s, a) || !strcmp(s, b)); }

NpdGeometry Check(const Tensor &key, const Tensor &value, const Tensor &key_cache, const Tensor &value_cache,
                  const Tensor &slot_mapping, const Tensor &q_len, const Tensor &kv_len, const Tensor &block_tbl,
                  const char *cache_layout, const char *kv_layout) {
  NpdGeometry g;
  if (!Is(cache_layout, "BNSD", "NPD") && !Is(cache_layout, "BSND", "ND"))
    MS_VALUE_ERROR << "For " << kOpName << ", kv_cache_layout must be 'BNSD' or 'BSND', but got '"
                   << (cache_layout ? cache_layout : "") << "'.";
  if (!Is(kv_layout, "TH", "TH") && !Is(kv_layout, "NPD", "NPD"))
    MS_VALUE_ERROR << "For " << kOpName << ", key_value_layout must be 'TH' or 'NPD', but got '"
                   << (kv_layout ? kv_layout : "") << "'.";
  if (Is(kv_layout, "NPD", "NPD"))
    MS_UNSUPPORTED << "For " << kOpName << ", key_value_layout='NPD' (key / value re-blocked per page together with "
                   << "the cached history) is an input format of the Ascend attention kernels and is not built for "
                   << "B200; use key_value_layout='TH'.";
  g.head_major = Is(cache_layout, "BNSD", "NPD");
  for (const Tensor *t : {&key, &value, &key_cache, &value_cache, &slot_mapping})
    if (!t->defined()) MS_VALUE_ERROR << "For " << kOpName << ", key, value, key_cache, value_cache and slot_mapping are required.";
  for (const Tensor *t : {&key, &value, &key_cache, &value_cache, &slot_mapping})
    if (t->has_zero_dim()) {
      g.skip = true;
      return g;
    }
  if (key.rank() != 2 && key.rank() != 3)
    MS_VALUE_ERROR << "For " << kOpName << ", key's dim should be 2 or 3, but got " << key.rank() << ".";
  if (value.rank() != key.rank())
    MS_VALUE_ERROR << "For " << kOpName << ", value must have the same rank as key.";
  if (key_cache.rank() != 4 || value_cache.rank() != 4)
    MS_VALUE_ERROR << "For " << kOpName << ", the caches must have rank 4.";
  auto allowed = [](int32_t dt) { return dt == MSCO_DTYPE_F16 || dt == MSCO_DTYPE_BF16 || dt == MSCO_DTYPE_I8; };
  if (!allowed(key.dtype()))
    MS_TYPE_ERROR << "For " << kOpName << ", key must be Float16/BFloat16/Int8, but got " << DTypeName(key.dtype()) << ".";
  if (key.dtype() != key_cache.dtype() || value.dtype() != value_cache.dtype())
    MS_TYPE_ERROR << "For " << kOpName << ", key / key_cache and value / value_cache must have the same dtype.";
  if (slot_mapping.dtype() != MSCO_DTYPE_I32)
    MS_TYPE_ERROR << "For " << kOpName << ", slot_mapping must be Int32, but got " << DTypeName(slot_mapping.dtype()) << ".";
  for (const auto &nt : {std::make_pair(&q_len, "actual_seq_qlen"), std::make_pair(&kv_len, "actual_seq_kvlen"),
                         std::make_pair(&block_tbl, "block_tbl")})
    if (nt.first->defined() && nt.first->dtype() != MSCO_DTYPE_I32)
      MS_TYPE_ERROR << "For " << kOpName << ", " << nt.second << " must be Int32, but got "
                    << DTypeName(nt.first->dtype()) << ".";
  const int bs_dim = g.head_major ? 2 : 1, h_dim = g.head_major ? 1 : 2;
  g.heads = key_cache.dim(h_dim);
  g.block_size = key_cache.dim(bs_dim);
  g.k_head = key_cache.dim(3);
  g.v_head = value_cache.dim(3);
  g.num_slots = key_cache.dim(0) * g.block_size;
  g.num_tokens = slot_mapping.numel();
  if (value_cache.dim(0) != key_cache.dim(0) || value_cache.dim(bs_dim) != g.block_size || value_cache.dim(h_dim) != g.heads)
    MS_VALUE_ERROR << "For " << kOpName << ", key_cache and value_cache must agree in num_blocks, block_size and heads.";
  const int64_t key_tokens = key.rank() == 2 ? key.dim(0) : key.dim(0) * key.dim(1);
  if (key_tokens != g.num_tokens)
    MS_VALUE_ERROR << "For " << kOpName << ", key holds " << key_tokens << " tokens but slot_mapping has "
                   << g.num_tokens << " entries.";
  if (key.dim(key.rank() - 1) != g.heads * g.k_head || value.dim(value.rank() - 1) != g.heads * g.v_head ||
      value.numel() != g.num_tokens * g.heads * g.v_head)
    MS_VALUE_ERROR << "For " << kOpName << ", the hidden sizes of key / value must equal heads * head_dim of the caches.";
  for (const auto &nt : {std::make_pair(&key, "key"), std::make_pair(&value, "value"), std::make_pair(&key_cache, "key_cache"),
                         std::make_pair(&value_cache, "value_cache"), std::make_pair(&slot_mapping, "slot_mapping")})
    CheckContiguous(*nt.first, kOpName, nt.second);
  return g;
}

}  // namespace
}  // namespace ms_custom_ops

MS_CUSTOM_OPS_REGISTER_OP(reshape_and_cache_npd,
                          "reshape_and_cache_npd(key, value, key_cache, value_cache, slot_mapping, actual_seq_qlen, "
                          "actual_seq_kvlen, block_tbl, kv_cache_layout='BNSD', key_value_layout='NPD')")

extern "C" int ms_custom_ops_reshape_and_cache_npd_infer(
    const MsTensorDesc *key, const MsTensorDesc *value, const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
    const MsTensorDesc *slot_mapping, const MsTensorDesc *actual_seq_qlen, const MsTensorDesc *actual_seq_kvlen,
    const MsTensorDesc *block_tbl, const char *kv_cache_layout, const char *key_value_layout, int32_t *out_key_dtype,
    int32_t *out_value_dtype, int32_t *out_ndim, int64_t *out_key_shape, int64_t *out_value_shape) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    const Tensor k(key), v(value);
    (void)Check(k, v, Tensor(key_cache), Tensor(value_cache), Tensor(slot_mapping), GetTensorOrEmpty(actual_seq_qlen),
                GetTensorOrEmpty(actual_seq_kvlen), GetTensorOrEmpty(block_tbl), kv_cache_layout, key_value_layout);
    if (out_key_dtype) *out_key_dtype = k.dtype();
    if (out_value_dtype) *out_value_dtype = v.dtype();
    if (out_ndim) *out_ndim = static_cast<int32_t>(k.rank());
    for (size_t i = 0; i < k.rank(); ++i) {
      if (out_key_shape) out_key_shape[i] = k.dim(i);
      if (out_value_shape) out_value_shape[i] = v.dim(i);
    }
    return MSCO_OK;
  });
}

extern "C" int ms_custom_ops_reshape_and_cache_npd(
    const MsTensorDesc *key, const MsTensorDesc *value, const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
    const MsTensorDesc *slot_mapping, const MsTensorDesc *actual_seq_qlen, const MsTensorDesc *actual_seq_kvlen,
    const MsTensorDesc *block_tbl, const char *kv_cache_layout, const char *key_value_layout,
    const MsTensorDesc *out_key, const MsTensorDesc *out_value, void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    const Tensor k(key), v(value), kc(key_cache), vc(value_cache), sm(slot_mapping), ok(out_key), ov(out_value);
    const NpdGeometry g = Check(k, v, kc, vc, sm, GetTensorOrEmpty(actual_seq_qlen), GetTensorOrEmpty(actual_seq_kvlen),
                                GetTensorOrEmpty(block_tbl), kv_cache_layout, key_value_layout);
    if (g.skip) return static_cast<int>(MSCO_OK);
    for (const auto &io : {std::make_pair(&ok, &k), std::make_pair(&ov, &v)}) {
      if (!io.first->defined()) continue;
      if (io.first->dtype() != io.second->dtype() || io.first->shape() != io.second->shape() || io.first->data() == nullptr)
        MS_VALUE_ERROR << "For " << kOpName << ", out_key / out_value must be allocated with key's / value's shape and dtype.";
      CheckContiguous(*io.first, kOpName, "output");
    }
    const int64_t es = DTypeSize(k.dtype()), evs = DTypeSize(v.dtype());
    const int32_t *slots = static_cast<const int32_t *>(sm.data());
    int rc;
    if (g.head_major) {
      if (es != evs) MS_TYPE_ERROR << "For " << kOpName << ", key and value must have the same element size.";
      rc = msco_reshape_and_cache_bnsd(k.data(), v.data(), kc.data(), vc.data(), slots, g.num_tokens,
                                       static_cast<int32_t>(g.heads), g.k_head * es, g.v_head * evs,
                                       static_cast<int32_t>(g.block_size), g.num_slots, nullptr, stream);
    } else {
      rc = msco_reshape_and_cache(k.data(), v.data(), kc.data(), vc.data(), slots, g.num_tokens, g.heads * g.k_head * es,
                                  g.heads * g.v_head * evs, g.num_slots, nullptr, stream);
    }
    if (rc != MSCO_OK) return rc;
    // "TH" outputs: the current key / value, unchanged
    for (const auto &io : {std::make_pair(&ok, &k), std::make_pair(&ov, &v)}) {
      if (!io.first->defined() || io.first->data() == io.second->data()) continue;
      rc = msco_copy_device(io.first->data(), io.second->data(),
                            static_cast<size_t>(io.second->numel() * DTypeSize(io.second->dtype())), stream);
      if (rc != MSCO_OK) return rc;
    }
    return static_cast<int>(MSCO_OK);
  });
}
