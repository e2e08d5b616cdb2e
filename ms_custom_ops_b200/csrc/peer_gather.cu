// All-gather of the per-rank attention outputs over NVLink peer memory.
//
// With the KV cache partitioned by kv head the only exchange of a decode step
// is the all-gather of each rank's [batch, q_heads / N, head_dim] output: a few
// hundred KB in total, i.e. a latency-bound collective.  Instead of a library
// collective, one small kernel pushes the local slice with plain 16-byte
// stores into the gathered buffer of every peer (mapped through CUDA IPC; no
// TMA, no multicast), publishes a per-step flag in every peer's flag array
// with a system-scope release, and then waits -- with an iteration limit -- for
// the flags of all peers, so that when the kernel has completed the gathered
// buffer of this rank holds every rank's slice.
//
// The kernels of the different ranks run on different GPUs (one process per
// GPU); nothing here waits on another launch of the same GPU.
#include <cuda.h>

#include <cstring>

#include "msco_common.cuh"
#include "peer_gather.cuh"

namespace msco {
namespace {

constexpr int kPushThreads = 512;
constexpr int kPushMaxBlocks = 16;

__global__ void __launch_bounds__(kPushThreads)
peer_gather_kernel(const __grid_constant__ GatherArgs a, const uint4 *__restrict__ local) {
  __shared__ bool is_last;
  const int64_t n16 = a.slice_bytes / 16;
  // launched with programmatic stream serialisation: the kernels of this library that produce
  // `local` let their dependents start early; wait here until they have completed and their
  // writes are visible (a no-op behind anything else)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // 1. push the local slice into slot `rank` of every rank's gathered buffer (own copy included)
  for (int64_t i = (int64_t)blockIdx.x * kPushThreads + threadIdx.x; i < n16; i += (int64_t)gridDim.x * kPushThreads)
    gather_push16(a, i * 16, __ldcg(local + i));
  // 2. the block that finishes last publishes the flags and waits for the peers
  gather_finish(a, &is_last);
}

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);

}  // namespace
}  // namespace msco

using namespace msco;

extern "C" int msco_ipc_export(const void *dev_ptr, unsigned char *handle, int64_t *offset) {
  if (dev_ptr == nullptr || handle == nullptr || offset == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "ipc_export: NULL argument");
  static GetAddressRangeFn get_range = nullptr;
  if (get_range == nullptr) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    MSCO_CUDA_CHECK(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || fn == nullptr)
      return fail(MSCO_ERR_CUDA, "ipc_export: cuMemGetAddressRange is not available");
    get_range = reinterpret_cast<GetAddressRangeFn>(fn);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = get_range(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr));
  if (r != CUDA_SUCCESS) return fail(MSCO_ERR_CUDA, "ipc_export: cuMemGetAddressRange failed (%d)", (int)r);
  cudaIpcMemHandle_t h;
  MSCO_CUDA_CHECK(cudaIpcGetMemHandle(&h, reinterpret_cast<void *>(base)));
  static_assert(sizeof(h) == MSCO_IPC_HANDLE_BYTES, "unexpected IPC handle size");
  memcpy(handle, &h, sizeof(h));
  *offset = (int64_t)(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
  return MSCO_OK;
}

extern "C" int msco_ipc_import(const unsigned char *handle, int64_t offset, void **dev_ptr) {
  if (handle == nullptr || dev_ptr == nullptr) return fail(MSCO_ERR_INVALID_ARG, "ipc_import: NULL argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *base = nullptr;
  MSCO_CUDA_CHECK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *dev_ptr = static_cast<char *>(base) + offset;
  return MSCO_OK;
}

extern "C" int msco_ipc_release(void *dev_ptr, int64_t offset) {
  if (dev_ptr == nullptr) return MSCO_OK;
  MSCO_CUDA_CHECK(cudaIpcCloseMemHandle(static_cast<char *>(dev_ptr) - offset));
  return MSCO_OK;
}

int msco::fill_gather_args(const MscoGatherDesc *desc, uint32_t step, const char *what, GatherArgs *out) {
  if (desc == nullptr) return fail(MSCO_ERR_INVALID_ARG, "%s: NULL gather descriptor", what);
  if (desc->world < 1 || desc->world > MSCO_MAX_PEERS || desc->rank < 0 || desc->rank >= desc->world)
    return fail(MSCO_ERR_INVALID_ARG, "%s: bad rank %d of %d", what, desc->rank, desc->world);
  if (desc->slice_bytes <= 0 || desc->slice_bytes % 16 != 0)
    return fail(MSCO_ERR_INVALID_ARG, "%s: slices must be multiples of 16 bytes", what);
  if (desc->ticket == nullptr || desc->status == nullptr)
    return fail(MSCO_ERR_INVALID_ARG, "%s: ticket / status words are required", what);
  GatherArgs &a = *out;
  memset(&a, 0, sizeof(a));
  for (int r = 0; r < desc->world; ++r) {
    if (desc->gathered[r] == nullptr || desc->flags[r] == nullptr)
      return fail(MSCO_ERR_INVALID_ARG, "%s: rank %d's buffers are not mapped", what, r);
    if (reinterpret_cast<uintptr_t>(desc->gathered[r]) & 15)
      return fail(MSCO_ERR_INVALID_ARG, "%s: rank %d's gathered buffer is not 16-byte aligned", what, r);
    a.gathered[r] = desc->gathered[r];
    a.flags[r] = desc->flags[r];
  }
  // the packet buffers: all of them or none
  int with_packets = 0;
  for (int r = 0; r < desc->world; ++r) with_packets += desc->packets[r] != nullptr ? 1 : 0;
  if (with_packets != 0 && with_packets != desc->world)
    return fail(MSCO_ERR_INVALID_ARG, "%s: packet buffers must be given for every rank or for none", what);
  for (int r = 0; r < desc->world; ++r) {
    if (reinterpret_cast<uintptr_t>(desc->packets[r]) & 15)
      return fail(MSCO_ERR_INVALID_ARG, "%s: rank %d's packet buffer is not 16-byte aligned", what, r);
    a.packets[r] = desc->packets[r];
  }
  if (with_packets != 0 && step == 0)
    return fail(MSCO_ERR_INVALID_ARG, "%s: steps count from 1 (0 marks an empty packet)", what);
  a.slice_bytes = desc->slice_bytes;
  a.world = desc->world;
  a.rank = desc->rank;
  a.wait_limit = desc->wait_polls != 0 ? desc->wait_polls : kPeerWaitLimit;
  a.step = step;
  a.ticket = desc->ticket;
  a.status = desc->status;
  return MSCO_OK;
}

extern "C" int msco_peer_allgather(const MscoGatherDesc *desc, const void *local_out, uint32_t step,
                                   void *stream) {
  if (desc == nullptr || local_out == nullptr) return fail(MSCO_ERR_INVALID_ARG, "peer_allgather: NULL argument");
  if (reinterpret_cast<uintptr_t>(local_out) & 15)
    return fail(MSCO_ERR_INVALID_ARG, "peer_allgather: the local slice must be 16-byte aligned");
  GatherArgs a;
  const int rc = fill_gather_args(desc, step, "peer_allgather", &a);
  if (rc != MSCO_OK) return rc;
  const int64_t n16 = desc->slice_bytes / 16;
  int blocks = (int)((n16 + kPushThreads - 1) / kPushThreads);
  blocks = blocks < 1 ? 1 : (blocks > kPushMaxBlocks ? kPushMaxBlocks : blocks);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(kPushThreads);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MSCO_CUDA_CHECK(cudaLaunchKernelEx(&cfg, peer_gather_kernel, a, static_cast<const uint4 *>(local_out)));
  return MSCO_OK;
}
