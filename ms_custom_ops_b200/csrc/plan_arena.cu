// Pooled pinned host memory for paged-attention plans (see plan_arena.h).
#include "plan_arena.h"

#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>
#include <vector>

namespace msco {

namespace {
constexpr size_t kMinBlock = 1024;          // smallest block: 256 plan words
constexpr size_t kSlabBytes = 2u << 20;     // one slab: 2 MiB of page-locked memory
constexpr int kClasses = 12;                // 1 KiB << 0 .. 11 (= 2 MiB)

int class_of(size_t bytes) {
  int k = 0;
  size_t cap = kMinBlock;
  while (cap < bytes) { cap <<= 1; ++k; }
  return k;
}
}  // namespace

struct PlanArena::Impl {
  std::mutex mu;
  std::vector<void *> free_list[kClasses];
  char *slab = nullptr;   // slab being carved
  size_t slab_used = 0;
  std::vector<void *> oversize_pinned;  // oversize blocks that came from cudaHostAlloc
  bool pinned = true;     // turns false the first time cudaHostAlloc fails (no device): malloc from then on
  PlanArenaStats st = {0, 0, 0, 0, 0, 1};

  void *raw_alloc(size_t bytes) {
    void *p = nullptr;
    if (pinned) {
      if (cudaHostAlloc(&p, bytes, cudaHostAllocDefault) == cudaSuccess) return p;
      (void)cudaGetLastError();
      pinned = false;
      st.pinned = 0;
    }
    return malloc(bytes);
  }
};

PlanArena &PlanArena::Instance() {
  static PlanArena *inst = new PlanArena();  // never destroyed: no CUDA calls at process exit
  return *inst;
}

PlanArena::Impl *PlanArena::impl() {
  static std::once_flag once;
  std::call_once(once, [this] { impl_ = new Impl(); });
  return impl_;
}

void *PlanArena::Alloc(size_t bytes, size_t *capacity) {
  Impl *m = impl();
  std::lock_guard<std::mutex> g(m->mu);
  if (bytes > kSlabBytes) {  // far beyond any plan of this library's operators: an allocation of its own
    void *p = m->raw_alloc(bytes);
    if (p == nullptr) return nullptr;
    if (m->pinned) m->oversize_pinned.push_back(p);
    ++m->st.oversize_allocs;
    ++m->st.blocks_in_use;
    ++m->st.block_allocs;
    *capacity = bytes;
    return p;
  }
  const int k = class_of(bytes);
  const size_t cap = kMinBlock << k;
  void *p = nullptr;
  if (!m->free_list[k].empty()) {
    p = m->free_list[k].back();
    m->free_list[k].pop_back();
  } else {
    if (m->slab == nullptr || m->slab_used + cap > kSlabBytes) {
      // the rest of the old slab goes to the free lists, largest blocks first
      while (m->slab != nullptr && m->slab_used + kMinBlock <= kSlabBytes) {
        int kk = kClasses - 1;
        while ((kMinBlock << kk) > kSlabBytes - m->slab_used || (m->slab_used & ((kMinBlock << kk) - 1))) --kk;
        m->free_list[kk].push_back(m->slab + m->slab_used);
        m->slab_used += kMinBlock << kk;
      }
      char *s = static_cast<char *>(m->raw_alloc(kSlabBytes));
      if (s == nullptr) return nullptr;
      m->slab = s;
      m->slab_used = 0;
      ++m->st.slabs;
      m->st.slab_bytes += (int64_t)kSlabBytes;
    }
    p = m->slab + m->slab_used;
    m->slab_used += cap;
  }
  ++m->st.blocks_in_use;
  ++m->st.block_allocs;
  *capacity = cap;
  return p;
}

void PlanArena::Free(void *block, size_t capacity) {
  if (block == nullptr) return;
  Impl *m = impl();
  std::lock_guard<std::mutex> g(m->mu);
  --m->st.blocks_in_use;
  if (capacity > kSlabBytes) {
    bool was_pinned = false;
    for (size_t i = 0; i < m->oversize_pinned.size(); ++i)
      if (m->oversize_pinned[i] == block) {
        m->oversize_pinned.erase(m->oversize_pinned.begin() + (long)i);
        was_pinned = true;
        break;
      }
    if (was_pinned) cudaFreeHost(block); else free(block);
    return;
  }
  m->free_list[class_of(capacity)].push_back(block);
}

void PlanArena::Stats(PlanArenaStats *out) {
  Impl *m = impl();
  std::lock_guard<std::mutex> g(m->mu);
  *out = m->st;
}

}  // namespace msco
