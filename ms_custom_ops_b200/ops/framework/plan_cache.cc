#include "ops/framework/plan_cache.h"

#include <cstdlib>
#include <cstring>

#include "ops/framework/tensor.h"

namespace ms_custom_ops {

uint64_t HashBytes(const void *data, size_t len, uint64_t seed) {
  const unsigned char *p = static_cast<const unsigned char *>(data);
  uint64_t h = seed ^ (len * 0x9e3779b97f4a7c15ull);
  auto mix = [](uint64_t x) {
    x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
    x ^= x >> 27; x *= 0x94d049bb133111ebull;
    x ^= x >> 31;
    return x;
  };
  while (len >= 8) {
    uint64_t w;
    memcpy(&w, p, 8);
    h = mix(h ^ w) + 0x9e3779b97f4a7c15ull;
    p += 8;
    len -= 8;
  }
  if (len) {
    uint64_t w = 0;
    memcpy(&w, p, len);
    h = mix(h ^ w) + 0x9e3779b97f4a7c15ull;
  }
  return mix(h);
}

namespace {
// field by field: the struct has padding bytes that must not enter a key
struct DescFields {
  int64_t f[17];
  uint32_t scale_bits;
};
DescFields FieldsOf(const MscoPaDesc &desc) {
  DescFields d = {{desc.q_dtype, desc.kv_dtype, desc.num_q_heads, desc.num_kv_heads, desc.head_dim,
                   desc.block_size, desc.num_blocks, desc.max_blocks_per_seq, desc.quant_type,
                   desc.has_quant_offset, desc.mask_type, desc.mask_dtype, desc.mask_batch_stride,
                   desc.mask_head_stride, desc.kernel, desc.cache_layout, 0},
                  0};
  memcpy(&d.scale_bits, &desc.qk_scale, 4);
  return d;
}
}  // namespace

uint64_t MakeDescHash(const MscoPaDesc &desc, bool multi_token) {
  const DescFields d = FieldsOf(desc);
  return HashBytes(d.f, sizeof(d.f), (0x452821e638d01377ull ^ d.scale_bits) + (multi_token ? 1 : 0));
}

PlanKey MakePlanKey(const MscoPaDesc &desc, const std::vector<int32_t> &lens, const std::vector<int32_t> *q_lens) {
  DescFields d = FieldsOf(desc);
  d.f[16] = static_cast<int64_t>(lens.size()) * 2 + (q_lens != nullptr ? 1 : 0);
  PlanKey k;
  k.h1 = HashBytes(d.f, sizeof(d.f), 0x243f6a8885a308d3ull ^ d.scale_bits);
  k.h2 = HashBytes(d.f, sizeof(d.f), 0x13198a2e03707344ull + d.scale_bits);
  k.h1 = HashBytes(lens.data(), lens.size() * sizeof(int32_t), k.h1);
  k.h2 = HashBytes(lens.data(), lens.size() * sizeof(int32_t), k.h2);
  if (q_lens != nullptr) {
    k.h1 = HashBytes(q_lens->data(), q_lens->size() * sizeof(int32_t), k.h1);
    k.h2 = HashBytes(q_lens->data(), q_lens->size() * sizeof(int32_t), k.h2);
  }
  return k;
}

PlanRef &PlanRef::operator=(PlanRef &&o) noexcept {
  if (this != &o) {
    if (cache_ && entry_) cache_->Release(entry_);
    cache_ = o.cache_; entry_ = o.entry_; plan_ = o.plan_;
    o.cache_ = nullptr; o.entry_ = nullptr; o.plan_ = nullptr;
  }
  return *this;
}
PlanRef::~PlanRef() {
  if (cache_ && entry_) cache_->Release(entry_);
}

PlanCache &PlanCache::Instance() {
  static PlanCache *inst = new PlanCache();  // intentionally leaked: no CUDA calls at process exit
  return *inst;
}

PlanCache::PlanCache() {
  if (const char *e = getenv("MSCO_PLAN_CACHE_CAPACITY")) {
    const long v = strtol(e, nullptr, 10);
    if (v > 0) capacity_ = static_cast<size_t>(v);
  }
}
PlanCache::~PlanCache() = default;

PlanRef PlanCache::GetOrCreate(const MscoPaDesc &desc, const std::vector<int32_t> &lens,
                               const std::vector<int32_t> *q_lens) {
  const PlanKey key = MakePlanKey(desc, lens, q_lens);
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(key);
    if (it != map_.end()) {
      Entry *e = it->second.get();
      ++hits_;
      ++e->refs;
      lru_.erase(e->lru_it);
      lru_.push_front(e);
      e->lru_it = lru_.begin();
      return PlanRef(this, e, e->plan);
    }
    ++misses_;
  }
  auto throw_plan_error = [](int rc) {
    ErrorBuilder b(rc == MSCO_ERR_UNSUPPORTED ? MS_ERR_KIND_UNSUPPORTED
                   : rc == MSCO_ERR_INVALID_ARG ? MS_ERR_KIND_VALUE : MS_ERR_KIND_RUNTIME, rc);
    b << "For PagedAttention, planning failed: " << msco_last_error();
    b.Throw();
  };
  const uint64_t desc_hash = MakeDescHash(desc, q_lens != nullptr);
  // Recycle: take the least recently used unreferenced plan of the same descriptor out of the cache
  // and re-plan it in place for the new lengths (no allocation in the steady state).
  std::unique_ptr<Entry> reuse;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto cnt = per_desc_.find(desc_hash);
    if (cnt != per_desc_.end() && static_cast<size_t>(cnt->second) >= per_desc_keep_) {
      for (auto it = lru_.end(); it != lru_.begin();) {
        --it;
        Entry *e = *it;
        if (e->refs == 0 && e->desc_hash == desc_hash) {
          auto mit = map_.find(e->key);
          reuse = std::move(mit->second);
          map_.erase(mit);
          lru_.erase(it);
          --cnt->second;
          break;
        }
      }
    }
  }
  // plan outside the lock: pure host work
  MscoPaPlan *plan = nullptr;
  if (reuse) {
    plan = reuse->plan;
    const int rc = q_lens != nullptr
                       ? msco_paged_attention_replan_tokens(plan, lens.data(), q_lens->data(), static_cast<int32_t>(lens.size()))
                       : msco_paged_attention_replan(plan, lens.data(), static_cast<int32_t>(lens.size()));
    if (rc != MSCO_OK) {
      msco_paged_attention_plan_destroy(plan);  // its contents are undefined now
      throw_plan_error(rc);
    }
  } else {
    const int rc = q_lens != nullptr
                       ? msco_paged_attention_plan_tokens(&desc, lens.data(), q_lens->data(),
                                                          static_cast<int32_t>(lens.size()), &plan)
                       : msco_paged_attention_plan(&desc, lens.data(), static_cast<int32_t>(lens.size()), &plan);
    if (rc != MSCO_OK) throw_plan_error(rc);
  }
  std::lock_guard<std::mutex> g(mu_);
  auto it = map_.find(key);
  if (it != map_.end()) {  // another thread planned the same key meanwhile
    RetireLocked(plan);
    Entry *e = it->second.get();
    ++e->refs;
    return PlanRef(this, e, e->plan);
  }
  if (reuse) ++recycled_; else ++created_;
  std::unique_ptr<Entry> e = reuse ? std::move(reuse) : std::make_unique<Entry>();
  e->key = key;
  e->desc_hash = desc_hash;
  e->plan = plan;
  e->refs = 1;
  lru_.push_front(e.get());
  e->lru_it = lru_.begin();
  Entry *raw = e.get();
  map_.emplace(key, std::move(e));
  ++per_desc_[desc_hash];
  EvictLocked();
  return PlanRef(this, raw, plan);
}

void PlanCache::MissStats(int64_t *recycled, int64_t *created) {
  std::lock_guard<std::mutex> g(mu_);
  if (recycled) *recycled = recycled_;
  if (created) *created = created_;
}

void PlanCache::Release(void *entry) {
  std::lock_guard<std::mutex> g(mu_);
  Entry *e = static_cast<Entry *>(entry);
  if (e->refs > 0) --e->refs;
}

void PlanCache::RetireLocked(MscoPaPlan *plan) {
  // keep the last few evicted plans alive: an asynchronous copy from a plan's pinned buffer may
  // still be queued on a stream
  retired_.push_back(plan);
  while (retired_.size() > 32) {
    msco_paged_attention_plan_destroy(retired_.front());
    retired_.pop_front();
  }
}

void PlanCache::EvictLocked() {
  auto it = lru_.end();
  while (map_.size() > capacity_ && it != lru_.begin()) {
    --it;
    Entry *e = *it;
    if (e->refs == 0) {
      RetireLocked(e->plan);
      const PlanKey key = e->key;
      --per_desc_[e->desc_hash];
      it = lru_.erase(it);
      map_.erase(key);
    }
  }
}

void PlanCache::Stats(int64_t *hits, int64_t *misses, int64_t *entries) {
  std::lock_guard<std::mutex> g(mu_);
  if (hits) *hits = hits_;
  if (misses) *misses = misses_;
  if (entries) *entries = static_cast<int64_t>(map_.size());
}

void PlanCache::Clear() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto it = lru_.begin(); it != lru_.end();) {
    Entry *e = *it;
    if (e->refs == 0) {
      RetireLocked(e->plan);
      const PlanKey key = e->key;
      --per_desc_[e->desc_hash];
      it = lru_.erase(it);
      map_.erase(key);
    } else {
      ++it;
    }
  }
  hits_ = misses_ = recycled_ = created_ = 0;
}

}  // namespace ms_custom_ops
