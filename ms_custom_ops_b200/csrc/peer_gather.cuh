// Device-side pieces of the all-gather over NVLink peer memory, shared by the stand-alone gather kernel
// (peer_gather.cu) and by the kernel that finishes the attention output rows of a sharded decode step
// (pa_reduce_kernel in pa_generic.cu), which pushes each row to the peers as soon as it is final.
//
// Protocol: a rank stores its slice into slot `rank` of every rank's gathered buffer with plain peer
// stores, the block that finishes last publishes the step counter in every rank's flag array with a
// system-scope release, and then waits -- with an iteration limit -- for the counters of all peers.
// No TMA, no multicast; the kernels of different ranks run on different GPUs.
#pragma once

#include "msco_common.cuh"

namespace msco {

constexpr uint32_t kPeerWaitLimit = 1u << 22;  // polls of ~0.1 us: gives up after about half a second

struct GatherArgs {
  void *gathered[MSCO_MAX_PEERS];   // rank r's gathered buffer as mapped into this process
  uint32_t *flags[MSCO_MAX_PEERS];  // rank r's flag array (uint32[world]) as mapped into this process
  int64_t slice_bytes;
  int world, rank;                  // world == 0: no gather (the finishing kernel of an unsharded step)
  uint32_t wait_limit;
  uint32_t step;
  unsigned int *ticket;             // local word: blocks of the grid that have pushed their part
  int32_t *status;                  // local word: kStatusTimeout when a peer never arrived
  void *packets[MSCO_MAX_PEERS];    // rank r's packet buffer (2 x world x slice_bytes), or all NULL
};

// Checks a gather descriptor and copies it into kernel arguments; `what` names the caller in the error text.
int fill_gather_args(const MscoGatherDesc *desc, uint32_t step, const char *what, GatherArgs *out);

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// 16 bytes at byte offset `off` of the local slice into slot `rank` of every rank's gathered buffer
__device__ __forceinline__ void gather_push16(const GatherArgs &a, int64_t off, const uint4 &v) {
  for (int r = 0; r < a.world; ++r)
    *reinterpret_cast<uint4 *>(static_cast<char *>(a.gathered[r]) + (int64_t)a.rank * a.slice_bytes + off) = v;
}

// ---- packet form of the exchange (GatherArgs::packets set) ----
// 16 data bytes travel as four 8-byte packets {data word, step}, written with two 16-byte stores.  A
// packet is valid when its step word equals the step waited for: data and validity arrive together, so the
// sender needs no fence and publishes no flag.  (Stores of 8 aligned bytes are not torn; the two packets
// of a 16-byte store may arrive apart, which is harmless.)
__device__ __forceinline__ void packets_push16(const GatherArgs &a, int64_t off, const uint4 &v) {
  const uint4 p0 = make_uint4(v.x, a.step, v.y, a.step), p1 = make_uint4(v.z, a.step, v.w, a.step);
  for (int r = 0; r < a.world; ++r) {
    if (r == a.rank) continue;
    uint4 *dst = reinterpret_cast<uint4 *>(static_cast<char *>(a.packets[r]) + ((int64_t)a.rank * a.slice_bytes + off) * 2);
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(p0.x), "r"(p0.y), "r"(p0.z), "r"(p0.w) : "memory");
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + 1), "r"(p1.x), "r"(p1.y), "r"(p1.z), "r"(p1.w) : "memory");
  }
}
// Waits (bounded) for the 16 data bytes at byte offset `off` of every peer's slice in this rank's packet
// buffer and copies them into this rank's plain gathered buffer.  Returns false when a peer never sent.
__device__ __forceinline__ bool packets_pull16(const GatherArgs &a, int64_t off) {
  bool all = true;
  for (int r = 0; r < a.world; ++r) {
    if (r == a.rank) continue;
    const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const char *>(a.packets[a.rank]) +
                                                       ((int64_t)r * a.slice_bytes + off) * 2);
    uint4 p0, p1;
    bool ok = false;
    for (uint32_t it = 0; it < a.wait_limit; ++it) {
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(p0.x), "=r"(p0.y), "=r"(p0.z), "=r"(p0.w) : "l"(src) : "memory");
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(p1.x), "=r"(p1.y), "=r"(p1.z), "=r"(p1.w) : "l"(src + 1) : "memory");
      if (p0.y == a.step && p0.w == a.step && p1.y == a.step && p1.w == a.step) { ok = true; break; }
      __nanosleep(40);
    }
    if (ok)
      *reinterpret_cast<uint4 *>(static_cast<char *>(a.gathered[a.rank]) + (int64_t)r * a.slice_bytes + off) =
          make_uint4(p0.x, p0.z, p1.x, p1.z);
    all = all && ok;
  }
  return all;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by every thread of every block after the block's pushes: the block that arrives last
// publishes the flags and waits for the peers.  `is_last` is a shared-memory flag of the caller.
// System-scope fences are what this exchange costs (each waits for the acknowledgement of the peer
// stores in flight, a round trip over NVLink), so there is exactly one per block on the way in -- by one
// thread, after the block barrier, which makes it cover the whole block's stores -- and the flag itself
// is a release store; the spin reads relaxed and fences once when the flag has arrived.  (One fence per
// thread plus an acquiring load per poll cost 20 us per exchange on two GPUs, twice a library all-gather.)
__device__ __forceinline__ void gather_finish(const GatherArgs &a, bool *is_last) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // the block's pushes (ordered before the barrier) precede its ticket
    const unsigned int t = atomicAdd(a.ticket, 1u);
    *is_last = (t == gridDim.x - 1);
    if (*is_last) {
      *a.ticket = 0u;        // ready for the next launch on this stream
      __threadfence_system();  // the tickets of the other blocks (and with them their pushes) precede the flags
    }
  }
  __syncthreads();
  if (!*is_last) return;
  if ((int)threadIdx.x < a.world) {
    const int r = threadIdx.x;
    st_release_sys(a.flags[r] + a.rank, a.step);  // "rank's slice of step `step` is in your buffer"
    const uint32_t *mine = a.flags[a.rank] + r;   // peer r's announcement in my own flag array
    bool ok = false;
    for (uint32_t it = 0; it < a.wait_limit; ++it) {
      if ((int32_t)(ld_relaxed_sys(mine) - a.step) >= 0) { ok = true; break; }
      __nanosleep(40);
    }
    __threadfence_system();  // acquire side: the peer's slice (written before its flag) is visible from here on
    if (!ok) atomicExch(a.status, kStatusTimeout);  // a peer never arrived: report, do not hang
  }
}

}  // namespace msco
