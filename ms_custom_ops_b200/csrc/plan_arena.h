// Pooled pinned host memory for paged-attention plans.
//
// Role of the reference's TilingMemMgr
// (ops/framework/ms_kernels_internal/tiling_mem_mgr.cc:82-137, 224-238; tiling_mem_mgr.h:27-29): tiling
// buffers come from memory the plugin allocated up front, so the step path never calls the allocator.
// Here the plan words of every MscoPaPlan are a block of this arena: page-locked slabs obtained with
// cudaHostAlloc (plain malloc when no CUDA device is present), carved into power-of-two blocks with a
// free list per size.  In the steady state -- a decode loop re-plans every step because every length
// grows -- blocks are recycled and no slab is ever added; the counters below let a test assert that.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace msco {

struct PlanArenaStats {
  int64_t slabs;           // slabs obtained so far (cudaHostAlloc / malloc calls of the arena)
  int64_t slab_bytes;      // their total size
  int64_t blocks_in_use;   // blocks handed out and not yet returned
  int64_t block_allocs;    // alloc() calls served
  int64_t oversize_allocs; // requests larger than a slab, served by an allocation of their own
  int64_t pinned;          // 1 when the slabs are page-locked
};

class PlanArena {
 public:
  static PlanArena &Instance();
  // A block of at least `bytes` (a power of two >= 1 KiB); *capacity receives its size.  NULL when
  // the host is out of memory.
  void *Alloc(size_t bytes, size_t *capacity);
  void Free(void *block, size_t capacity);
  void Stats(PlanArenaStats *out);

 private:
  PlanArena() = default;
  struct Impl;
  Impl *impl();
  Impl *impl_ = nullptr;
};

}  // namespace msco
