// Dispatch permutation for callers that must not allocate device memory.
//
// Who needs this: code that runs where a cudaMalloc is not an option -- a host runtime that has
// already handed all of the GPU's memory to its own pool (the reference engine's pooled staging
// buffers work that way, and a plain cudaMalloc beside such a pool can fail or fragment it), a
// serving loop that cannot afford the device-wide synchronisation an allocation implies, or a
// plugin that is only given the buffers it is called with.  Such callers cannot create an
// AteniaMoeLayer, whose workspace is allocated with cudaMalloc, but they can still ask for the
// canonical dispatch order of a batch: this entry point needs only the caller's input and output
// buffers.  Its per-block histograms live in a fixed array compiled into the library.
//
// The array is `static __device__`: every GPU that loads the library carries its own 256 KiB copy
// until the process exits.  In host code the array's name is only a stand-in, not a device address,
// so the address each device uses is looked up once per device with cudaGetSymbolAddress (with that
// device current) and that pointer is what the kernels receive.
#include <mutex>

#include "common.cuh"

namespace atenia {
namespace {

constexpr int kNoAllocMaxEntries = ATENIA_NOALLOC_MAX_ENTRIES;  // tokens * top_k
constexpr int kNoAllocMaxExperts = ATENIA_NOALLOC_MAX_EXPERTS;
constexpr int kNoAllocBlocks = kNoAllocMaxEntries / kDispatchChunk;
constexpr int kNoAllocWords = 2 * kNoAllocBlocks * kNoAllocMaxExperts;  // counts + bases: 65536 words

static __device__ __align__(256) int32_t g_dispatch_scratch[kNoAllocWords];

std::mutex g_setup_mu;
int32_t* g_scratch_addr[kMaxDevices] = {};  // kMaxDevices: common.cuh

// Device address of the scratch array on the current device; looked up on the first call per device
// and kept for the life of the process.  A cudaDeviceReset (or any other teardown of the device's
// primary context) invalidates the kept address: a process that resets a device must not call this
// entry point on that device afterwards.
int scratch_for_current_device(int32_t** out) {
  int dev = -1;
  ATENIA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ATENIA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    ATENIA_CUDA_TRY(cudaGetSymbolAddress(&p, g_dispatch_scratch));
    if (!p) return ATENIA_ERR_DRIVER;
    g_scratch_addr[dev] = static_cast<int32_t*>(p);
  }
  *out = g_scratch_addr[dev];
  return ATENIA_OK;
}

}  // namespace
}  // namespace atenia

extern "C" int atenia_moe_dispatch_noalloc(const int32_t* topk_idx, int T, int k, int E, int32_t* perm,
                                           int32_t* inv_perm, int32_t* expert_offsets, void* stream) {
  using namespace atenia;
  if (!topk_idx || !perm || !inv_perm || !expert_offsets) return ATENIA_ERR_NULL;
  if (T < 0 || k < 1 || E < 1) return ATENIA_ERR_SHAPE;
  if (E > kNoAllocMaxExperts || (int64_t)T * k > kNoAllocMaxEntries) return ATENIA_ERR_SCRATCH_LIMIT;
  int32_t* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  const int n = T * k;
  const int nblk = (n + kDispatchChunk - 1) / kDispatchChunk;
  DispatchArgs a{};
  a.topk_idx = topk_idx;
  a.n = n;
  a.E = E;
  // Nothing in the array has to start at zero: the histogram kernel writes all E counters of every
  // block it runs, the scan reads exactly those blocks and writes their bases, and the placement
  // reads exactly those bases.  Whatever an earlier call left behind is never read.
  a.block_counts = scratch;
  a.block_base = scratch + (size_t)nblk * E;
  a.expert_offsets = expert_offsets;
  a.perm = perm;
  a.inv_perm = inv_perm;
  a.extra_offsets = nullptr;
  a.T = T;
  a.err = nullptr;
  return launch_dispatch(a, static_cast<cudaStream_t>(stream));
}
