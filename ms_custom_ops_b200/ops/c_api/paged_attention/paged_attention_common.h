// Argument positions and attribute values of paged_attention.
//
// Values are those of the registered operator (reference:
// ops/c_api/paged_attention/paged_attention_common.h:24-110); callers pass the
// same integers they pass to the reference plugin.
#ifndef MS_CUSTOM_OPS_B200_PAGED_ATTENTION_COMMON_H_
#define MS_CUSTOM_OPS_B200_PAGED_ATTENTION_COMMON_H_

#include <cstdint>

namespace ms_custom_ops {

// position of each registered argument (tensors 0..14, attributes 15..28)
enum PagedAttentionArg : int32_t {
  kPaArgQuery = 0, kPaArgKeyCache, kPaArgValueCache, kPaArgBlockTables, kPaArgContextLens, kPaArgAttnMask,
  kPaArgBatchRunStatus, kPaArgKDescale, kPaArgKOffset, kPaArgVDescale, kPaArgVOffset, kPaArgRazorOffset,
  kPaArgPScale, kPaArgLogN, kPaArgQSeqLens, kPaArgQHeadNum, kPaArgQkScale, kPaArgKvHeadNum, kPaArgMaskType,
  kPaArgBatchRunStatusEnable, kPaArgQuantType, kPaArgOutDataType, kPaArgHasQuantOffset, kPaArgCompressType,
  kPaArgCalcType, kPaArgScaleType, kPaArgInputLayout, kPaArgMlaVDim, kPaArgInputFormat, kPaArgCount
};

enum PaMaskType : int64_t { kMaskUndefined = 0, kMaskNorm = 1, kMaskAlibi = 2, kMaskSpec = 3, kMaskFree = 4 };
enum PaQuantType : int64_t { kQuantUnquant = 0, kQuantDequantFusion = 1, kQuantQkvOffline = 2, kQuantQkvOnline = 3 };
enum PaCompressType : int64_t { kCompressNone = 0, kCompressKvHead = 1, kCompressKvHeadRope = 2, kCompressMax = 3 };
enum PaCalcType : int64_t { kCalcDefault = 0, kCalcSpec = 1 };
enum PaOutDataType : int64_t { kOutUndefined = -1, kOutFloat16 = 1, kOutBFloat16 = 27 };
enum PaInputLayout : int64_t { kLayoutBSND = 0, kLayoutBNSD = 1 };
enum PaScaleType : int64_t { kScaleTor = 0, kScaleLogN = 1, kScaleMax = 2 };
enum PaInputFormat : int64_t { kFormatND = 0, kFormatNZ = 1 };

constexpr size_t kPaQueryRank = 3;
constexpr size_t kPaCacheRank = 4;
constexpr size_t kPaBlockTableRank = 2;
constexpr size_t kPaContextLenRank = 1;

}  // namespace ms_custom_ops
#endif  // MS_CUSTOM_OPS_B200_PAGED_ATTENTION_COMMON_H_
