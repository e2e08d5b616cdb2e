// Hash-keyed cache of paged-attention launch plans.
//
// Role of the reference's InternalTilingCache
// (ops/framework/ms_kernels_internal/internal_tiling_cache.h:110-226,
//  internal_tiling_cache.cc:220-426): tiling (here: the split plan) is a pure
// function of the operator attributes, the tensor shapes / dtypes and the host
// values of context_lens, so it is computed once per distinct key and reused.
// Entries are reference counted; only unreferenced entries are evicted, least
// recently used first.
//
// In a decode loop every length grows every step, so every step is a miss.  A
// miss therefore does not build a new plan when it can avoid it: once a few
// plans of the same descriptor exist, the least recently used unreferenced one
// is re-planned in place (msco_paged_attention_replan) and re-keyed.  Its plan
// words stay in the same block of the kernel library's pinned arena, its tensor
// maps stay valid, and the step path touches no allocator -- the role of the
// reference's TilingMemMgr (ops/framework/ms_kernels_internal/tiling_mem_mgr.cc:82-137,
// 224-238), which serves tiling buffers from memory set aside at start-up.
#ifndef MS_CUSTOM_OPS_B200_FRAMEWORK_PLAN_CACHE_H_
#define MS_CUSTOM_OPS_B200_FRAMEWORK_PLAN_CACHE_H_

#include <cstdint>
#include <deque>
#include <list>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "msco_b200.h"

namespace ms_custom_ops {

// 64-bit mix over a byte string (splitmix-style avalanche per 8-byte word).
uint64_t HashBytes(const void *data, size_t len, uint64_t seed);

struct PlanKey {
  uint64_t h1 = 0, h2 = 0;  // two independent 64-bit hashes: 128-bit key
  bool operator==(const PlanKey &o) const { return h1 == o.h1 && h2 == o.h2; }
};
struct PlanKeyHash {
  size_t operator()(const PlanKey &k) const { return static_cast<size_t>(k.h1 ^ (k.h2 * 0x9e3779b97f4a7c15ull)); }
};

// `q_seq_lens` (NULL for a decode batch): query tokens per sequence of a multi-token call.
PlanKey MakePlanKey(const MscoPaDesc &desc, const std::vector<int32_t> &context_lens,
                    const std::vector<int32_t> *q_seq_lens = nullptr);
// Hash of the descriptor alone (what a re-plan must leave unchanged); decode and multi-token plans differ.
uint64_t MakeDescHash(const MscoPaDesc &desc, bool multi_token = false);

class PlanCache;

// RAII reference to a cached plan.
class PlanRef {
 public:
  PlanRef() = default;
  PlanRef(PlanCache *cache, void *entry, MscoPaPlan *plan) : cache_(cache), entry_(entry), plan_(plan) {}
  PlanRef(PlanRef &&o) noexcept { *this = std::move(o); }
  PlanRef &operator=(PlanRef &&o) noexcept;
  PlanRef(const PlanRef &) = delete;
  PlanRef &operator=(const PlanRef &) = delete;
  ~PlanRef();
  MscoPaPlan *get() const { return plan_; }
  explicit operator bool() const { return plan_ != nullptr; }

 private:
  PlanCache *cache_ = nullptr;
  void *entry_ = nullptr;
  MscoPaPlan *plan_ = nullptr;
};

class PlanCache {
 public:
  static PlanCache &Instance();
  // Returns the cached plan for (desc, lens), building it on a miss.  Throws OpError on failure.
  PlanRef GetOrCreate(const MscoPaDesc &desc, const std::vector<int32_t> &context_lens,
                      const std::vector<int32_t> *q_seq_lens = nullptr);
  void Stats(int64_t *hits, int64_t *misses, int64_t *entries);
  // misses served by re-planning an existing plan in place / by building a new plan
  void MissStats(int64_t *recycled, int64_t *created);
  void set_per_desc_keep(size_t n) { per_desc_keep_ = n; }
  void Clear();
  void set_capacity(size_t n) { capacity_ = n; }

 private:
  friend class PlanRef;
  struct Entry {
    PlanKey key;
    uint64_t desc_hash = 0;
    MscoPaPlan *plan = nullptr;
    int refs = 0;
    std::list<Entry *>::iterator lru_it;
  };
  PlanCache();
  ~PlanCache();
  void Release(void *entry);
  void EvictLocked();
  void RetireLocked(MscoPaPlan *plan);

  std::mutex mu_;
  std::unordered_map<PlanKey, std::unique_ptr<Entry>, PlanKeyHash> map_;
  std::list<Entry *> lru_;            // front = most recently used
  std::deque<MscoPaPlan *> retired_;  // evicted plans awaiting destruction
  std::unordered_map<uint64_t, int> per_desc_;  // entries per descriptor hash
  size_t capacity_ = 256;
  size_t per_desc_keep_ = 4;  // plans of one descriptor kept before misses start recycling them
  int64_t hits_ = 0, misses_ = 0, recycled_ = 0, created_ = 0;
};

}  // namespace ms_custom_ops
#endif  // MS_CUSTOM_OPS_B200_FRAMEWORK_PLAN_CACHE_H_
