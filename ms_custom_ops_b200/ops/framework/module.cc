#include "ops/framework/module.h"

#include <exception>

#include "ms_custom_ops_c.h"
#include "ops/framework/plan_cache.h"
#include "ops/framework/tensor.h"

namespace ms_custom_ops {
namespace {
thread_local std::string g_last_error;
thread_local int g_last_kind = MS_ERR_KIND_NONE;
}  // namespace

void SetLastError(int kind, const std::string &msg) {
  g_last_kind = kind;
  g_last_error = msg;
}

int GuardedCall(const char *op_name, const std::function<int()> &fn) {
  try {
    const int rc = fn();
    if (rc != MSCO_OK) {
      // failure reported by the kernel library: keep its message
      SetLastError(rc == MSCO_ERR_UNSUPPORTED ? MS_ERR_KIND_UNSUPPORTED
                   : rc == MSCO_ERR_INVALID_ARG ? MS_ERR_KIND_VALUE : MS_ERR_KIND_RUNTIME,
                   std::string("For ") + op_name + ": " + msco_last_error());
    } else {
      g_last_kind = MS_ERR_KIND_NONE;
    }
    return rc;
  } catch (const OpError &e) {
    SetLastError(e.kind(), e.what());
    return e.code();
  } catch (const std::exception &e) {
    SetLastError(MS_ERR_KIND_RUNTIME, std::string("For ") + op_name + ": " + e.what());
    return MSCO_ERR_INTERNAL;
  }
}
}  // namespace ms_custom_ops

extern "C" const char *ms_custom_ops_last_error(void) { return ms_custom_ops::g_last_error.c_str(); }
extern "C" int ms_custom_ops_last_error_kind(void) { return ms_custom_ops::g_last_kind; }

extern "C" int ms_custom_ops_num_ops(void) {
  return static_cast<int>(ms_custom_ops::ModuleRegistry::Instance().ops().size());
}
extern "C" const char *ms_custom_ops_op_name(int index) {
  const auto &ops = ms_custom_ops::ModuleRegistry::Instance().ops();
  return (index >= 0 && index < static_cast<int>(ops.size())) ? ops[index].name.c_str() : nullptr;
}
extern "C" const char *ms_custom_ops_op_signature(int index) {
  const auto &ops = ms_custom_ops::ModuleRegistry::Instance().ops();
  return (index >= 0 && index < static_cast<int>(ops.size())) ? ops[index].signature.c_str() : nullptr;
}

extern "C" void ms_custom_ops_plan_cache_stats(int64_t *hits, int64_t *misses, int64_t *entries) {
  ms_custom_ops::PlanCache::Instance().Stats(hits, misses, entries);
}
extern "C" void ms_custom_ops_plan_cache_clear(void) { ms_custom_ops::PlanCache::Instance().Clear(); }
extern "C" void ms_custom_ops_plan_cache_miss_stats(int64_t *recycled, int64_t *created) {
  ms_custom_ops::PlanCache::Instance().MissStats(recycled, created);
}
extern "C" void ms_custom_ops_plan_arena_stats(int64_t *stats) { msco_plan_arena_stats(stats); }
