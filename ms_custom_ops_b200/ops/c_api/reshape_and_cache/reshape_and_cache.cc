// reshape_and_cache: operator glue for the B200 plugin.
//
// Mirrors the operator the reference registers in
// ops/c_api/reshape_and_cache/reshape_and_cache.cc:
//   :31-34   CacheMode { ND = 0, NZ = 1 }
//   :36-44   input order key, value, key_cache, value_cache, slot_mapping, cache_mode, head_num
//   :90-119  execution is skipped when any input has a zero dimension
//   :181-201 eager entry: optional value / caches / slot_mapping, no output tensor
// The device work is msco_reshape_and_cache (libmsco_b200.so).  FRACTAL_NZ
// (cache_mode = 1) is an Ascend cube-unit layout and is not built for B200.
#include "ms_custom_ops_c.h"
#include "ops/framework/module.h"
#include "ops/framework/tensor.h"

namespace ms_custom_ops {
namespace {

enum class CacheMode : int64_t { ND = 0, NZ = 1 };
constexpr const char *kOpName = "ReshapeAndCache";

struct CacheGeometry {
  int64_t num_tokens = 0, num_slots = 0, k_row_elems = 0, v_row_elems = 0;
  bool has_value = false, skip = false;
};

// Shape / dtype rules shared by the plain and the quantising variant.
CacheGeometry CheckAndDescribe(const Tensor &key, const Tensor &value, const Tensor &key_cache,
                               const Tensor &value_cache, const Tensor &slot_mapping, int64_t cache_mode,
                               bool quantising) {
  CacheGeometry g;
  if (!key.defined()) MS_VALUE_ERROR << "For " << kOpName << ", key must be provided.";
  if (cache_mode != static_cast<int64_t>(CacheMode::ND) && cache_mode != static_cast<int64_t>(CacheMode::NZ))
    MS_VALUE_ERROR << "For " << kOpName << ", cache_mode must be 0 (ND) or 1 (NZ), but got " << cache_mode << ".";
  if (cache_mode == static_cast<int64_t>(CacheMode::NZ))
    MS_UNSUPPORTED << "For " << kOpName << ", cache_mode=1 (FRACTAL_NZ) is an Ascend-only cache layout; "
                   << "the B200 build supports cache_mode=0 (ND).";
  // zero-sized inputs: nothing to do (the reference short-circuits the same way)
  for (const Tensor *t : {&key, &value, &key_cache, &value_cache, &slot_mapping})
    if (t->has_zero_dim()) {
      g.skip = true;
      return g;
    }
  if (!key_cache.defined() || !slot_mapping.defined())
    MS_VALUE_ERROR << "For " << kOpName << ", key_cache and slot_mapping must be provided.";
  if (value.defined() != value_cache.defined())
    MS_VALUE_ERROR << "For " << kOpName << ", value and value_cache must be provided together.";
  g.has_value = value.defined();
  if (key.rank() != 2 && key.rank() != 3)
    MS_VALUE_ERROR << "For " << kOpName << ", key's dim should be 2 or 3, but got " << key.rank() << ".";
  if (g.has_value && value.rank() != key.rank())
    MS_VALUE_ERROR << "For " << kOpName << ", value must have the same rank as key, but got " << value.rank()
                   << " and " << key.rank() << ".";
  if (key_cache.rank() != 4 || (g.has_value && value_cache.rank() != 4))
    MS_VALUE_ERROR << "For " << kOpName << ", the ND caches must have rank 4 "
                   << "(num_blocks, block_size, kv_heads, head_dim).";
  if (slot_mapping.dtype() != MSCO_DTYPE_I32)
    MS_TYPE_ERROR << "For " << kOpName << ", slot_mapping must be Int32, but got " << DTypeName(slot_mapping.dtype())
                  << ".";
  auto allowed = [](int32_t dt) { return dt == MSCO_DTYPE_F16 || dt == MSCO_DTYPE_BF16 || dt == MSCO_DTYPE_I8; };
  if (quantising) {
    if (key.dtype() != MSCO_DTYPE_F16 && key.dtype() != MSCO_DTYPE_BF16)
      MS_TYPE_ERROR << "For " << kOpName << " (quant), key must be Float16/BFloat16, but got " << DTypeName(key.dtype())
                    << ".";
    if (key_cache.dtype() != MSCO_DTYPE_I8 || (g.has_value && value_cache.dtype() != MSCO_DTYPE_I8))
      MS_TYPE_ERROR << "For " << kOpName << " (quant), the caches must be Int8.";
    if (g.has_value && value.dtype() != key.dtype())
      MS_TYPE_ERROR << "For " << kOpName << " (quant), key and value must have the same dtype.";
  } else {
    // dtype_group (key, key_cache), (value, value_cache) of the registered definition
    if (!allowed(key.dtype()))
      MS_TYPE_ERROR << "For " << kOpName << ", key must be Float16/BFloat16/Int8, but got " << DTypeName(key.dtype())
                    << ".";
    if (key.dtype() != key_cache.dtype())
      MS_TYPE_ERROR << "For " << kOpName << ", key and key_cache must have the same dtype, but got "
                    << DTypeName(key.dtype()) << " and " << DTypeName(key_cache.dtype()) << ".";
    if (g.has_value && value.dtype() != value_cache.dtype())
      MS_TYPE_ERROR << "For " << kOpName << ", value and value_cache must have the same dtype, but got "
                    << DTypeName(value.dtype()) << " and " << DTypeName(value_cache.dtype()) << ".";
  }
  g.num_tokens = slot_mapping.numel();
  g.k_row_elems = key_cache.dim(2) * key_cache.dim(3);
  g.num_slots = key_cache.dim(0) * key_cache.dim(1);
  const int64_t key_tokens = key.rank() == 2 ? key.dim(0) : key.dim(0) * key.dim(1);
  if (key_tokens != g.num_tokens)
    MS_VALUE_ERROR << "For " << kOpName << ", key holds " << key_tokens << " tokens but slot_mapping has "
                   << g.num_tokens << " entries.";
  if (key.dim(key.rank() - 1) != g.k_row_elems)
    MS_VALUE_ERROR << "For " << kOpName << ", key's hidden size " << key.dim(key.rank() - 1)
                   << " must equal kv_heads * head_dim of key_cache (" << g.k_row_elems << ").";
  if (g.has_value) {
    g.v_row_elems = value_cache.dim(2) * value_cache.dim(3);
    if (value.numel() != g.num_tokens * g.v_row_elems)
      MS_VALUE_ERROR << "For " << kOpName << ", value's shape does not match slot_mapping and value_cache.";
    if (value_cache.dim(0) != key_cache.dim(0) || value_cache.dim(1) != key_cache.dim(1))
      MS_VALUE_ERROR << "For " << kOpName << ", key_cache and value_cache must have the same num_blocks and block_size.";
  }
  CheckContiguous(key, kOpName, "key");
  CheckContiguous(value, kOpName, "value");
  CheckContiguous(key_cache, kOpName, "key_cache");
  CheckContiguous(value_cache, kOpName, "value_cache");
  CheckContiguous(slot_mapping, kOpName, "slot_mapping");
  return g;
}

int ReshapeAndCache(const Tensor &key, const Tensor &value, const Tensor &key_cache, const Tensor &value_cache,
                    const Tensor &slot_mapping, int64_t cache_mode, int64_t head_num, void *stream) {
  (void)head_num;  // only meaningful for the NZ layout
  const CacheGeometry g = CheckAndDescribe(key, value, key_cache, value_cache, slot_mapping, cache_mode, false);
  if (g.skip) return MSCO_OK;
  const int64_t es = DTypeSize(key.dtype());
  return msco_reshape_and_cache(key.data(), value.data(), key_cache.data(), value_cache.data(),
                                static_cast<const int32_t *>(slot_mapping.data()), g.num_tokens,
                                g.k_row_elems * es, g.v_row_elems * es, g.num_slots, nullptr, stream);
}

int ReshapeAndCacheQuant(const Tensor &key, const Tensor &value, const Tensor &key_cache, const Tensor &value_cache,
                         const Tensor &slot_mapping, const Tensor &k_descale, const Tensor &v_descale,
                         const Tensor &k_offset, const Tensor &v_offset, void *stream) {
  const CacheGeometry g = CheckAndDescribe(key, value, key_cache, value_cache, slot_mapping, 0, true);
  if (g.skip) return MSCO_OK;
  auto check_vec = [&](const Tensor &t, const char *name, int32_t dt, int64_t n, bool required) {
    if (!t.defined()) {
      if (required) MS_VALUE_ERROR << "For " << kOpName << " (quant), " << name << " must be provided.";
      return;
    }
    if (t.dtype() != dt)
      MS_TYPE_ERROR << "For " << kOpName << " (quant), " << name << " must be " << DTypeName(dt) << ", but got "
                    << DTypeName(t.dtype()) << ".";
    if (t.numel() != n)
      MS_VALUE_ERROR << "For " << kOpName << " (quant), " << name << " must have kv_heads * head_dim = " << n
                     << " elements, but got " << t.numel() << ".";
    CheckContiguous(t, kOpName, name);
  };
  check_vec(k_descale, "k_descale", MSCO_DTYPE_F32, g.k_row_elems, true);
  check_vec(k_offset, "k_offset", MSCO_DTYPE_I32, g.k_row_elems, false);
  if (g.has_value) {
    check_vec(v_descale, "v_descale", MSCO_DTYPE_F32, g.v_row_elems, true);
    check_vec(v_offset, "v_offset", MSCO_DTYPE_I32, g.v_row_elems, false);
  }
  return msco_reshape_and_cache_quant(
      key.data(), value.data(), static_cast<int8_t *>(key_cache.data()), static_cast<int8_t *>(value_cache.data()),
      static_cast<const int32_t *>(slot_mapping.data()), g.num_tokens, g.k_row_elems, g.v_row_elems, key.dtype(),
      static_cast<const float *>(k_descale.data()), static_cast<const int32_t *>(k_offset.data()),
      static_cast<const float *>(v_descale.data()), static_cast<const int32_t *>(v_offset.data()), g.num_slots,
      nullptr, stream);
}

}  // namespace
}  // namespace ms_custom_ops

MS_CUSTOM_OPS_REGISTER_OP(reshape_and_cache,
                          "reshape_and_cache(key, value=None, key_cache=None, value_cache=None, slot_mapping=None, "
                          "cache_mode=0, head_num=0)")
MS_CUSTOM_OPS_REGISTER_OP(reshape_and_cache_quant,
                          "reshape_and_cache_quant(key, value, key_cache, value_cache, slot_mapping, k_descale, "
                          "v_descale, k_offset=None, v_offset=None)")

extern "C" int ms_custom_ops_reshape_and_cache(const MsTensorDesc *key, const MsTensorDesc *value,
                                               const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                               const MsTensorDesc *slot_mapping, int64_t cache_mode,
                                               int64_t head_num, void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return ReshapeAndCache(Tensor(key), GetTensorOrEmpty(value), GetTensorOrEmpty(key_cache),
                           GetTensorOrEmpty(value_cache), GetTensorOrEmpty(slot_mapping), cache_mode, head_num, stream);
  });
}

// Placeholder output of the registered operator: key's shape and dtype
// (CustomReshapeAndCacheOpFuncImpl, reshape_and_cache.cc:66-75 of the reference), after the checks.
extern "C" int ms_custom_ops_reshape_and_cache_infer(const MsTensorDesc *key, const MsTensorDesc *value,
                                                     const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                                     const MsTensorDesc *slot_mapping, int64_t cache_mode,
                                                     int64_t head_num, int32_t *out_dtype, int32_t *out_ndim,
                                                     int64_t *out_shape) {
  using namespace ms_custom_ops;
  (void)head_num;
  return GuardedCall(kOpName, [&] {
    const Tensor k(key);
    (void)CheckAndDescribe(k, GetTensorOrEmpty(value), GetTensorOrEmpty(key_cache), GetTensorOrEmpty(value_cache),
                           GetTensorOrEmpty(slot_mapping), cache_mode, false);
    if (out_dtype) *out_dtype = k.dtype();
    if (out_ndim) *out_ndim = static_cast<int32_t>(k.rank());
    if (out_shape)
      for (size_t i = 0; i < k.rank(); ++i) out_shape[i] = k.dim(i);
    return MSCO_OK;
  });
}

extern "C" int ms_custom_ops_reshape_and_cache_quant(const MsTensorDesc *key, const MsTensorDesc *value,
                                                     const MsTensorDesc *key_cache, const MsTensorDesc *value_cache,
                                                     const MsTensorDesc *slot_mapping, const MsTensorDesc *k_descale,
                                                     const MsTensorDesc *v_descale, const MsTensorDesc *k_offset,
                                                     const MsTensorDesc *v_offset, void *stream) {
  using namespace ms_custom_ops;
  return GuardedCall(kOpName, [&] {
    return ReshapeAndCacheQuant(Tensor(key), GetTensorOrEmpty(value), GetTensorOrEmpty(key_cache),
                                GetTensorOrEmpty(value_cache), GetTensorOrEmpty(slot_mapping),
                                GetTensorOrEmpty(k_descale), GetTensorOrEmpty(v_descale), GetTensorOrEmpty(k_offset),
                                GetTensorOrEmpty(v_offset), stream);
  });
}
