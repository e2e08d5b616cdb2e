// Sequence-length change detection shared by the attention operators
// (role of ops/c_api/utils/attention_utils.h:26-50 in the reference).
#ifndef MS_CUSTOM_OPS_B200_ATTENTION_UTILS_H_
#define MS_CUSTOM_OPS_B200_ATTENTION_UTILS_H_

#include <cstdint>
#include <vector>

namespace ms_custom_ops {
// Stores `fresh` into `*kept` when they differ; returns whether they did.
inline bool CheckAndUpdate(const std::vector<int32_t> &fresh, std::vector<int32_t> *kept) {
  if (*kept == fresh) return false;
  *kept = fresh;
  return true;
}
}  // namespace ms_custom_ops
#endif  // MS_CUSTOM_OPS_B200_ATTENTION_UTILS_H_
