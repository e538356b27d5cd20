// Expert parallelism: experts sharded contiguously by id over the ranks of one node, rows exchanged
// with NCCL point-to-point groups (an all-to-all with per-peer sizes) over NVLink.
//
// Per forward, on every rank:
//   1. route the rank's own tokens over all E experts and sort its (token, slot) rows by expert
//      (done by the caller); rows bound for one rank are then contiguous
//   2. all-gather the per-expert row counts, read them on the host (the one host sync of the path)
//   3. exchange rows: send each peer its slice, receive the peers' slices into recv_x, laid out
//      [source rank][local expert][rows]
//   4. run the local experts over recv_x with one GEMM group per (source rank, local expert)
//   5. exchange the results back into y_perm, which has the caller's dispatch order again
// The reference has no multi-GPU path; the result is defined by the single-GPU path: rows are the
// same rows, experts the same experts, and the combine order is unchanged.
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <thread>
#include <vector>

#include "ep_plan.cuh"
#include "layer.cuh"

namespace atenia {

struct EpComm {
  ncclComm_t comm = nullptr;  // null once aborted: every layer sharing it then reports ATENIA_ERR_STATE
};

namespace {

void ep_comm_delete(EpComm* p) {
  if (p->comm) ncclCommDestroy(p->comm);
  delete p;
}

__global__ void counts_kernel(const int32_t* __restrict__ off, int E, int32_t* __restrict__ counts) {
  int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < E) counts[e] = off[e + 1] - off[e];
}

// group g = p * e_local + j covers the rows source rank p sent for local expert j
__global__ void group_offsets_kernel(const int32_t* __restrict__ counts_all, int world, int E, int e_begin,
                                     int e_local, int32_t* __restrict__ group_offsets) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int run = 0;
  for (int p = 0; p < world; ++p)
    for (int j = 0; j < e_local; ++j) {
      group_offsets[p * e_local + j] = run;
      run += counts_all[p * E + e_begin + j];
    }
  group_offsets[world * e_local] = run;
}

// ---- direct exchange: rows stored into peer memory ---------------------------------------------
__global__ void ep_plan_kernel(const int32_t* __restrict__ counts_all, int world, int E, int rank,
                               int32_t* __restrict__ dst_base, int32_t* __restrict__ src_base,
                               int32_t* __restrict__ sub_offsets, int32_t* __restrict__ gemm_offsets) {
  // one thread per plan entry (E <= 128): the entries are independent prefix sums over the count matrix
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < E) ep_direct_plan_entry(counts_all, world, E, rank, i, dst_base, src_base, sub_offsets, gemm_offsets);
}

// One warp moves one row: 16-byte vectors, four loads in flight per lane before the stores.
__device__ __forceinline__ void warp_copy_row_bf16(uint4* __restrict__ drow, const uint4* __restrict__ srow, int nvec,
                                                   int lane) {
  for (int v = lane; v < nvec; v += 128) {
    uint4 t[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (v + 32 * j < nvec) t[j] = srow[v + 32 * j];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (v + 32 * j < nvec) drow[v + 32 * j] = t[j];
  }
}

constexpr int kEpRowWarps = 8;  // warps (rows in flight) per block of the two row-moving kernels

// ---- flag synchronisation -------------------------------------------------------------------------
// Every rank owns a sync buffer that all ranks map: words [phase][source rank] hold the epoch (forward
// number) up to which that source has finished the phase -- 0: its expert counts are stored here,
// 1: its rows are stored in this rank's receive buffer, 2: its results are stored in this rank's y_perm --
// followed by the count matrix [world][E].  A rank publishes with a system-scope fence and a release
// store into every peer's buffer; a rank consumes by polling its OWN buffer (local memory) with acquire
// loads.  Every poll is bounded in time and in iterations: a peer that never arrives costs
// ATENIA_ERR_DEVICE_TIMEOUT and a sticky "gave up" word that makes the later waits of this layer return
// at once; the kernels then run on stale but in-range counts (every index is range-checked).
constexpr int kEpMaxWorld = 16;
constexpr int kEpSyncFlagWords = 4 * kEpMaxWorld;  // epochs [3][kEpMaxWorld] + spare; the counts follow
constexpr size_t kEpSyncBytes = (size_t)2 << 20;   // a whole allocation granule: nothing else shares the mapping

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// true once *flag has reached `epoch`; false after limit_ns (or the matching number of polls)
__device__ bool wait_epoch(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t max_polls = limit_ns / 64 + 1024;
  for (uint64_t polls = 0; polls < max_polls; ++polls) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    __nanosleep(polls < 256 ? 32 : 256);
    if ((polls & 255) == 255 && globaltimer_ns() - t0 > limit_ns) return false;
  }
  return false;
}

// lanes 0 .. world-1 of the calling block wait for their source's epoch of `phase`
__device__ void wait_phase(const uint32_t* my_sync, uint32_t* state, int phase, int world, uint64_t limit_ns,
                           DeviceError* err) {
  if ((int)threadIdx.x >= world) return;
  if (state[3] != 0) {  // an earlier wait of this layer gave up: the exchange is out of step for good
    report_error(err, ATENIA_ERR_STATE, 3110 + phase);
    return;
  }
  if (!wait_epoch(my_sync + phase * kEpMaxWorld + threadIdx.x, state[0], limit_ns)) {
    state[3] = 1;
    report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 3100 + phase);
  }
}

// End of a row-moving kernel: when the last block of the grid has finished, tell every rank that this
// rank's stores of `phase` are done.  Every thread fences its own peer stores; the block counter is
// the usual release (fence, then add) / acquire (add, then fence) pair.
__device__ void grid_done_publish(uint32_t* const* peer_sync, uint32_t* state, int phase, int world, int rank) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&state[phase], 1u);
    if (prev == gridDim.x - 1) {
      state[phase] = 0;  // the next launch of this kernel follows in stream order
      __threadfence_system();
      const uint32_t epoch = state[0];
      for (int p = 0; p < world; ++p) st_release_sys(peer_sync[p] + phase * kEpMaxWorld + rank, epoch);
    }
  }
}

// Start of a forward: next epoch; this rank's row counts per expert into every rank's count matrix.
__global__ void ep_counts_publish_kernel(const int32_t* __restrict__ off, int E, int world, int rank,
                                         uint32_t* const* __restrict__ peer_sync, uint32_t* state) {
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) {
    epoch_s = state[0] + 1;
    state[0] = epoch_s;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int p = i / E, e = i - p * E;
    reinterpret_cast<int32_t*>(peer_sync[p] + kEpSyncFlagWords)[rank * E + e] = off[e + 1] - off[e];
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < world) st_release_sys(peer_sync[threadIdx.x] + rank, epoch_s);
}

// Row placement once every rank's counts of this forward have arrived (one block; E <= 128 threads work).
__global__ void ep_plan_flags_kernel(const uint32_t* my_sync, uint32_t* state, int world, int E, int rank,
                                     uint64_t limit_ns, int32_t* __restrict__ dst_base, int32_t* __restrict__ src_base,
                                     int32_t* __restrict__ sub_offsets, int32_t* __restrict__ gemm_offsets,
                                     DeviceError* err) {
  wait_phase(my_sync, state, 0, world, limit_ns, err);
  __syncthreads();
  const int32_t* counts_all = reinterpret_cast<const int32_t*>(my_sync + kEpSyncFlagWords);
  const int i = threadIdx.x;
  if (i < E) ep_direct_plan_entry(counts_all, world, E, rank, i, dst_base, src_base, sub_offsets, gemm_offsets);
}

__global__ void ep_wait_kernel(const uint32_t* my_sync, uint32_t* state, int phase, int world, uint64_t limit_ns,
                               DeviceError* err) {
  wait_phase(my_sync, state, phase, world, limit_ns, err);
}

// Warp w of the grid moves dispatch rows w, w + W, ... (token perm[i] / k, expert topk_idx[perm[i]])
// of this rank into the receive buffer of the expert's owner: gather and send in one pass.  A row
// index outside the owner's buffer is recorded and skipped.
__global__ void __launch_bounds__(kEpRowWarps * 32) ep_scatter_kernel(
    const void* __restrict__ x, int x_is_f32, const int32_t* __restrict__ perm, const int32_t* __restrict__ topk_idx,
    const int32_t* __restrict__ expert_offsets, const int32_t* __restrict__ dst_base,
    __nv_bfloat16* const* __restrict__ peer_recv_x, int n_rows, int k, int d, int E, int e_local, int recv_cap,
    DeviceError* err, uint32_t* const* __restrict__ peer_sync, uint32_t* state, int world, int rank) {
  const int lane = threadIdx.x & 31;
  const int nvec = d / 8;
  // entries with an invalid expert id were given no row: perm beyond the placed count is stale
  const int placed = expert_offsets[E] < n_rows ? expert_offsets[E] : n_rows;
  for (int i = blockIdx.x * kEpRowWarps + (threadIdx.x >> 5); i < placed; i += gridDim.x * kEpRowWarps) {
    const int flat = perm[i];
    if (flat < 0 || flat >= n_rows) continue;
    const int e = topk_idx[flat];
    if (e < 0 || e >= E) continue;
    const int row = dst_base[e] + (i - expert_offsets[e]);
    if (row < 0 || row >= recv_cap) {
      if (lane == 0) report_error(err, ATENIA_ERR_CAPACITY, 3000);
      continue;
    }
    const int tok = flat / k;
    uint4* drow = reinterpret_cast<uint4*>(peer_recv_x[e / e_local] + (size_t)row * d);
    if (x_is_f32) {
      const float4* srow = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)tok * d);
      for (int v = lane; v < nvec; v += 32) {
        const float4 a = srow[2 * v], b = srow[2 * v + 1];
        drow[v] = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                             pack_bf16x2(b.z, b.w));
      }
    } else {
      warp_copy_row_bf16(drow, reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + (size_t)tok * d),
                         nvec, lane);
    }
  }
  if (peer_sync) grid_done_publish(peer_sync, state, 1, world, rank);
}

// Row i of this rank's expert outputs belongs to sub-group g = (local expert j, source rank p) and
// goes back to row src_base[g] + (i - sub_offsets[g]) of rank p's y_perm.  One warp per row.
__global__ void __launch_bounds__(kEpRowWarps * 32) ep_return_kernel(
    const __nv_bfloat16* __restrict__ recv_y, const int32_t* __restrict__ group_offsets,
    const int32_t* __restrict__ src_base, __nv_bfloat16* const* __restrict__ peer_y_perm, int n_groups, int world,
    int d, int rows_cap, DeviceError* err, uint32_t* const* __restrict__ peer_sync, uint32_t* state, int rank) {
  const int total = group_offsets[n_groups];
  const int lane = threadIdx.x & 31;
  const int nvec = d / 8;
  for (int i = blockIdx.x * kEpRowWarps + (threadIdx.x >> 5); i < total; i += gridDim.x * kEpRowWarps) {
    int lo = 0, hi = n_groups;  // group_offsets[lo] <= i < group_offsets[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (group_offsets[mid] <= i) lo = mid;
      else hi = mid;
    }
    const int row = src_base[lo] + (i - group_offsets[lo]);
    if (row < 0 || row >= rows_cap) {
      if (lane == 0) report_error(err, ATENIA_ERR_CAPACITY, 3001);
      continue;
    }
    warp_copy_row_bf16(reinterpret_cast<uint4*>(peer_y_perm[lo % world] + (size_t)row * d),
                       reinterpret_cast<const uint4*>(recv_y + (size_t)i * d), nvec, lane);
  }
  if (peer_sync) grid_done_publish(peer_sync, state, 2, world, rank);
}

#define NCCL_TRY(expr)                                 \
  do {                                                 \
    ncclResult_t r__ = (expr);                         \
    if (r__ != ncclSuccess) return ATENIA_ERR_NCCL;    \
  } while (0)

// Wait for `s` with a deadline instead of blocking: a peer that died or never joined must not hang
// this rank for ever.  Polls the stream and the communicator's asynchronous error state; on an
// error or when the deadline (ATENIA_MOE_EP_TIMEOUT_S, default 60 s) passes the communicator is
// aborted, which also ends NCCL kernels still waiting on the device, and ATENIA_ERR_NCCL is returned.
int bounded_stream_wait(AteniaMoeLayer* L, cudaStream_t s) {
  if (!L->ep || !L->ep->comm) return ATENIA_ERR_STATE;
  static const double limit_s = [] {
    const char* e = std::getenv("ATENIA_MOE_EP_TIMEOUT_S");
    double v = e ? std::atof(e) : 60.0;
    return v > 0.0 ? v : 60.0;
  }();
  ncclComm_t comm = L->ep->comm;
  const auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    cudaError_t q = cudaStreamQuery(s);
    if (q == cudaSuccess) return ATENIA_OK;
    if (q != cudaErrorNotReady) return (int)q;
    (void)cudaGetLastError();  // "not ready" is recorded as the last error: clear it, or the next
                               // launch check of this thread would report it
    ncclResult_t async = ncclSuccess;
    const bool bad = ncclCommGetAsyncError(comm, &async) != ncclSuccess || (async != ncclSuccess && async != ncclInProgress);
    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (bad || waited > limit_s) {
      ncclCommAbort(comm);
      L->ep->comm = nullptr;
      return ATENIA_ERR_NCCL;
    }
    if (waited > 0.002) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

int exchange(ncclComm_t comm, int rank, int world, const __nv_bfloat16* send, const std::vector<int64_t>& s_off,
             const std::vector<int64_t>& s_cnt, __nv_bfloat16* recv, const std::vector<int64_t>& r_off,
             const std::vector<int64_t>& r_cnt, int d, cudaStream_t s) {
  if (s_cnt[rank] > 0)
    ATENIA_CUDA_TRY(cudaMemcpyAsync(recv + r_off[rank] * d, send + s_off[rank] * d,
                                    (size_t)s_cnt[rank] * d * sizeof(__nv_bfloat16), cudaMemcpyDeviceToDevice, s));
  NCCL_TRY(ncclGroupStart());
  for (int p = 0; p < world; ++p) {
    if (p == rank) continue;
    if (s_cnt[p] > 0) NCCL_TRY(ncclSend(send + s_off[p] * d, (size_t)s_cnt[p] * d, ncclBfloat16, p, comm, s));
    if (r_cnt[p] > 0) NCCL_TRY(ncclRecv(recv + r_off[p] * d, (size_t)r_cnt[p] * d, ncclBfloat16, p, comm, s));
  }
  NCCL_TRY(ncclGroupEnd());
  return ATENIA_OK;
}

}  // namespace

int ep_forward_exchange(AteniaMoeLayer* L, int T, cudaStream_t s) {
  (void)T;
  const AteniaMoeConfig& c = L->cfg;
  const int G = c.ep_world, E = c.num_experts, El = L->e_local, rank = c.ep_rank, d = c.d_model;
  ncclComm_t comm = L->ep->comm;
  counts_kernel<<<1, 128, 0, s>>>(L->expert_offsets, E, L->d_counts_all + (size_t)rank * E);
  count_launch();
  NCCL_TRY(ncclAllGather(L->d_counts_all + (size_t)rank * E, L->d_counts_all, (size_t)E, ncclInt32, comm, s));
  ATENIA_CUDA_TRY(cudaMemcpyAsync(L->h_counts_all, L->d_counts_all, (size_t)G * E * sizeof(int32_t),
                                  cudaMemcpyDeviceToHost, s));
  group_offsets_kernel<<<1, 32, 0, s>>>(L->d_counts_all, G, E, L->e_begin, El, L->d_group_offsets);
  count_launch();
  {
    int wrc = bounded_stream_wait(L, s);
    if (wrc) return wrc;
  }
  std::vector<int64_t> s_off(G), s_cnt(G), r_off(G), r_cnt(G);
  int64_t ro = 0;
  int prc = atenia_moe_ep_plan(L->h_counts_all, G, E, rank, s_off.data(), s_cnt.data(), r_off.data(),
                               r_cnt.data(), nullptr, &ro);
  if (prc) return prc;
  if (ro > L->recv_cap) return ATENIA_ERR_CAPACITY;
  int rc = exchange(comm, rank, G, L->x_perm, s_off, s_cnt, L->recv_x, r_off, r_cnt, d, s);
  if (rc) return rc;
  if (L->timing) cudaEventRecord(L->ph[2], s);
  L->last_recv_rows = (int)ro;
  rc = run_expert_gemms(L, L->tm_recv_x, L->tm_recv_h, L->recv_x, L->recv_h, L->recv_y, L->d_group_offsets,
                        L->n_groups, (int)ro, s);
  if (rc) return rc;
  if (L->timing) cudaEventRecord(L->ph[3], s);
  rc = exchange(comm, rank, G, L->recv_y, r_off, r_cnt, L->y_perm, s_off, s_cnt, d, s);
  if (L->timing) cudaEventRecord(L->ph[4], s);
  return rc;
}

// Replicated tokens (decode): every rank holds the same batch and has routed and sorted it
// identically.  A rank runs the grouped GEMMs over the groups of its own experts only, which sit at
// the same rows of the dispatch-ordered buffers on every rank; rows of experts owned elsewhere stay
// zero.  Summing y_perm over the ranks then assembles all rows on all ranks.  Exactly one rank
// contributes a non-zero value to any element, so the sum is exact in whatever order NCCL adds, and
// the combine that follows sees the bytes of the single-GPU run.  No host read: the whole forward is
// launches on `s` and can be captured into a CUDA graph.
int ep_forward_replicated(AteniaMoeLayer* L, int n_rows, cudaStream_t s) {
  if (n_rows <= 0) return ATENIA_OK;
  const int d = L->cfg.d_model;
  ATENIA_CUDA_TRY(cudaMemsetAsync(L->y_perm, 0, (size_t)n_rows * d * sizeof(__nv_bfloat16), s));
  if (L->timing) cudaEventRecord(L->ph[2], s);
  int rc = run_expert_gemms(L, L->tm_x_perm, L->tm_recv_h, L->x_perm, L->recv_h, L->y_perm,
                            L->expert_offsets + L->e_begin, L->e_local, n_rows, s);
  if (rc) return rc;
  if (L->timing) cudaEventRecord(L->ph[3], s);
  NCCL_TRY(ncclAllReduce(L->y_perm, L->y_perm, (size_t)n_rows * d, ncclBfloat16, ncclSum, L->ep->comm, s));
  if (L->timing) cudaEventRecord(L->ph[4], s);
  return ATENIA_OK;
}

// Direct exchange, in two halves (ep_direct_send, ep_direct_finish).  Every step is a launch on `s`: the counts travel by all-gather, every rank derives
// all row positions from them on the device (ep_plan.cuh; the receive buffer is expert-major, so the
// GEMM has one group per local expert), rows are stored into the owners' receive buffers by
// ep_scatter_kernel (which also replaces the local gather), a one-word all-reduce orders
// those stores before the grouped GEMMs of every rank, ep_return_kernel stores the results into the
// sources' y_perm and a second all-reduce orders them before the combine.  The collectives are the
// only cross-GPU synchronisation (no flags, no spinning kernels), a kernel's peer stores are complete
// when the kernel is, and nothing is read on the host.
int ep_direct_send(AteniaMoeLayer* L, const void* x, int x_is_f32, int T, cudaStream_t s) {
  const AteniaMoeConfig& c = L->cfg;
  const int G = c.ep_world, E = c.num_experts, El = L->e_local, rank = c.ep_rank, d = c.d_model;
  const int n = T * c.experts_per_token;
  ncclComm_t comm = L->ep->comm;
  const bool flags = L->ep_flags;
  if (flags) {
    ep_counts_publish_kernel<<<1, 128, 0, s>>>(L->expert_offsets, E, G, rank, L->d_peer_sync, L->d_ep_state);
    count_launch();
    ep_plan_flags_kernel<<<1, 128, 0, s>>>(L->d_sync, L->d_ep_state, G, E, rank, L->ep_flag_limit_ns, L->d_dst_base,
                                           L->d_src_base, L->d_group_offsets, L->d_gemm_offsets, L->d_err);
    count_launch();
  } else {
    counts_kernel<<<1, 128, 0, s>>>(L->expert_offsets, E, L->d_counts_all + (size_t)rank * E);
    count_launch();
    NCCL_TRY(ncclAllGather(L->d_counts_all + (size_t)rank * E, L->d_counts_all, (size_t)E, ncclInt32, comm, s));
    ep_plan_kernel<<<1, 128, 0, s>>>(L->d_counts_all, G, E, rank, L->d_dst_base, L->d_src_base, L->d_group_offsets,
                                    L->d_gemm_offsets);
    count_launch();
  }
  if (n > 0 || flags) {  // (with flags the kernel also publishes "my rows are out", rows or no rows)
    const int blocks = n > 0 ? (n + kEpRowWarps - 1) / kEpRowWarps : 1;
    const int cap = L->num_sms * 16;
    ep_scatter_kernel<<<blocks < cap ? blocks : cap, kEpRowWarps * 32, 0, s>>>(
        x, x_is_f32, L->perm, L->topk_idx, L->expert_offsets, L->d_dst_base, L->d_peer_recv_x, n,
        c.experts_per_token, d, E, El, L->recv_cap, L->d_err, flags ? L->d_peer_sync : nullptr, L->d_ep_state, G,
        rank);
    count_launch();
  }
  return (int)cudaGetLastError();
}

// Second half: call after any local work that does not need the routed results (the shared expert),
// so that it runs while the peers' rows are still arriving.
int ep_direct_finish(AteniaMoeLayer* L, cudaStream_t s) {
  const AteniaMoeConfig& c = L->cfg;
  const int G = c.ep_world, El = L->e_local, d = c.d_model;
  ncclComm_t comm = L->ep->comm;
  const bool flags = L->ep_flags;
  if (flags) {
    ep_wait_kernel<<<1, 32, 0, s>>>(L->d_sync, L->d_ep_state, 1, G, L->ep_flag_limit_ns, L->d_err);
    count_launch();
  } else {
    NCCL_TRY(ncclAllReduce(L->d_bar, L->d_bar, 1, ncclInt32, ncclSum, comm, s));
  }
  if (L->timing) cudaEventRecord(L->ph[2], s);
  // the number of rows received is known on the device only: size by the buffer.
  // one GEMM group per local expert: its rows from all sources are contiguous
  int rc = run_expert_gemms(L, L->tm_recv_x, L->tm_recv_h, L->recv_x, L->recv_h, L->recv_y, L->d_gemm_offsets, El,
                            L->recv_cap, s);
  if (rc) return rc;
  if (L->timing) cudaEventRecord(L->ph[3], s);
  ep_return_kernel<<<L->num_sms * 16, kEpRowWarps * 32, 0, s>>>(L->recv_y, L->d_group_offsets, L->d_src_base, L->d_peer_y_perm,
                                                  L->n_groups, G, d, L->rows_cap, L->d_err,
                                                  flags ? L->d_peer_sync : nullptr, L->d_ep_state, c.ep_rank);
  count_launch();
  ATENIA_CUDA_TRY(cudaGetLastError());
  if (flags) {
    ep_wait_kernel<<<1, 32, 0, s>>>(L->d_sync, L->d_ep_state, 2, G, L->ep_flag_limit_ns, L->d_err);
    count_launch();
  } else {
    NCCL_TRY(ncclAllReduce(L->d_bar, L->d_bar, 1, ncclInt32, ncclSum, comm, s));
  }
  if (L->timing) cudaEventRecord(L->ph[4], s);
  return ATENIA_OK;
}

bool ep_ready(const AteniaMoeLayer* L) { return L->ep && L->ep->comm; }

int ep_bounded_wait(AteniaMoeLayer* L, cudaStream_t s) { return bounded_stream_wait(L, s); }

void ep_destroy(AteniaMoeLayer* L) {
  for (void* p : L->ipc_opened) cudaIpcCloseMemHandle(p);
  L->ipc_opened.clear();
  L->ep_direct = false;
  L->ep.reset();
}

}  // namespace atenia

extern "C" {

// Exchange plan of one rank, from the all-gathered count matrix.  Pure host arithmetic.
int atenia_moe_ep_plan(const int32_t* counts_all, int world, int num_experts, int rank, int64_t* send_off,
                       int64_t* send_cnt, int64_t* recv_off, int64_t* recv_cnt, int64_t* group_offsets,
                       int64_t* total_recv) {
  if (!counts_all || !send_off || !send_cnt || !recv_off || !recv_cnt) return ATENIA_ERR_NULL;
  if (world < 1 || num_experts < 1 || num_experts % world || rank < 0 || rank >= world) return ATENIA_ERR_SHAPE;
  const int El = num_experts / world, e_begin = rank * El;
  int64_t so = 0, ro = 0;
  for (int p = 0; p < world; ++p) {
    int64_t sc = 0, rc = 0;
    for (int j = 0; j < El; ++j) {
      sc += counts_all[(size_t)rank * num_experts + p * El + j];
      const int32_t c = counts_all[(size_t)p * num_experts + e_begin + j];
      if (group_offsets) group_offsets[p * El + j] = ro + rc;
      rc += c;
    }
    send_off[p] = so;
    send_cnt[p] = sc;
    recv_off[p] = ro;
    recv_cnt[p] = rc;
    so += sc;
    ro += rc;
  }
  if (group_offsets) group_offsets[world * El] = ro;
  if (total_recv) *total_recv = ro;
  return ATENIA_OK;
}

int atenia_moe_ep_unique_id_bytes(void) { return (int)sizeof(ncclUniqueId); }

int atenia_moe_ep_get_unique_id(void* id_out) {
  if (!id_out) return ATENIA_ERR_NULL;
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return ATENIA_ERR_NCCL;
  memcpy(id_out, &id, sizeof(id));
  return ATENIA_OK;
}

int atenia_moe_ep_init(AteniaMoeLayer* L, const void* unique_id) {
  if (!L || !unique_id) return ATENIA_ERR_NULL;
  if (L->cfg.ep_world <= 1) return ATENIA_ERR_STATE;
  if (atenia::ep_ready(L)) return ATENIA_OK;
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  ncclComm_t comm = nullptr;
  if (ncclCommInitRank(&comm, L->cfg.ep_world, id, L->cfg.ep_rank) != ncclSuccess) return ATENIA_ERR_NCCL;
  atenia::EpComm* holder = new atenia::EpComm();
  holder->comm = comm;
  L->ep = std::shared_ptr<atenia::EpComm>(holder, atenia::ep_comm_delete);
  return ATENIA_OK;
}

int atenia_moe_ep_attach(AteniaMoeLayer* L, AteniaMoeLayer* owner) {
  if (!L || !owner) return ATENIA_ERR_NULL;
  if (L->cfg.ep_world <= 1 || !atenia::ep_ready(owner)) return ATENIA_ERR_STATE;
  if (L->cfg.ep_world != owner->cfg.ep_world || L->cfg.ep_rank != owner->cfg.ep_rank || L->device != owner->device)
    return ATENIA_ERR_SHAPE;
  L->ep = owner->ep;
  return ATENIA_OK;
}

namespace {
struct IpcBlob {
  cudaIpcMemHandle_t recv_x, y_perm, sync;
  int32_t recv_cap, rows_cap, d_model, pad;  // buffer sizes: every rank must have been created alike
};
}  // namespace

int atenia_moe_ep_ipc_bytes(void) { return (int)sizeof(IpcBlob); }

int atenia_moe_ep_ipc_export(AteniaMoeLayer* L, void* blob) {
  if (!L || !blob) return ATENIA_ERR_NULL;
  if (L->cfg.ep_world <= 1 || !L->recv_x || !L->y_perm) return ATENIA_ERR_STATE;
  IpcBlob b;
  ATENIA_CUDA_TRY(cudaIpcGetMemHandle(&b.recv_x, L->recv_x));
  ATENIA_CUDA_TRY(cudaIpcGetMemHandle(&b.y_perm, L->y_perm));
  if (!L->d_sync) {
    if ((size_t)atenia::kEpSyncFlagWords * 4 + (size_t)L->cfg.ep_world * L->cfg.num_experts * 4 > atenia::kEpSyncBytes ||
        L->cfg.ep_world > atenia::kEpMaxWorld)
      return ATENIA_ERR_UNSUPPORTED;
    ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_sync), atenia::kEpSyncBytes));
    ATENIA_CUDA_TRY(cudaMemset(L->d_sync, 0, atenia::kEpSyncBytes));
    ATENIA_CUDA_TRY(cudaDeviceSynchronize());  // zero before any peer can store into it
  }
  ATENIA_CUDA_TRY(cudaIpcGetMemHandle(&b.sync, L->d_sync));
  b.recv_cap = L->recv_cap;
  b.rows_cap = L->rows_cap;
  b.d_model = L->cfg.d_model;
  b.pad = 0;
  memcpy(blob, &b, sizeof(b));
  return ATENIA_OK;
}

int atenia_moe_ep_ipc_import(AteniaMoeLayer* L, const void* blobs) {
  if (!L || !blobs) return ATENIA_ERR_NULL;
  const int G = L->cfg.ep_world, rank = L->cfg.ep_rank;
  if (G <= 1 || !atenia::ep_ready(L) || L->ep_replicated || L->ep_direct) return ATENIA_ERR_STATE;
  if (!L->d_sync) return ATENIA_ERR_STATE;  // (allocated by this layer's export)
  std::vector<__nv_bfloat16*> px(G), py(G);
  std::vector<uint32_t*> ps(G);
  // the sender bounds its stores by its own buffer sizes: they must be the sizes of every peer
  for (int p = 0; p < G; ++p) {
    IpcBlob b;
    memcpy(&b, static_cast<const unsigned char*>(blobs) + (size_t)p * sizeof(IpcBlob), sizeof(b));
    if (b.recv_cap != L->recv_cap || b.rows_cap != L->rows_cap || b.d_model != L->cfg.d_model) return ATENIA_ERR_SHAPE;
  }
  for (int p = 0; p < G; ++p) {
    if (p == rank) {
      px[p] = L->recv_x;
      py[p] = L->y_perm;
      ps[p] = L->d_sync;
      continue;
    }
    IpcBlob b;
    memcpy(&b, static_cast<const unsigned char*>(blobs) + (size_t)p * sizeof(IpcBlob), sizeof(b));
    void* a = nullptr;
    void* y = nullptr;
    void* z = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&a, b.recv_x, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess) {
      L->ipc_opened.push_back(a);
      e = cudaIpcOpenMemHandle(&y, b.y_perm, cudaIpcMemLazyEnablePeerAccess);
    }
    if (e == cudaSuccess) {
      L->ipc_opened.push_back(y);
      e = cudaIpcOpenMemHandle(&z, b.sync, cudaIpcMemLazyEnablePeerAccess);
    }
    if (e != cudaSuccess) {
      for (void* q : L->ipc_opened) cudaIpcCloseMemHandle(q);
      L->ipc_opened.clear();
      return (int)e;
    }
    L->ipc_opened.push_back(z);
    px[p] = static_cast<__nv_bfloat16*>(a);
    py[p] = static_cast<__nv_bfloat16*>(y);
    ps[p] = static_cast<uint32_t*>(z);
  }
  const size_t pb = (size_t)G * sizeof(void*);
  if (!L->d_peer_recv_x) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_peer_recv_x), pb));
  if (!L->d_peer_y_perm) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_peer_y_perm), pb));
  if (!L->d_dst_base) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_dst_base), (size_t)L->cfg.num_experts * 4));
  if (!L->d_src_base) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_src_base), (size_t)L->n_groups * 4));
  if (!L->d_gemm_offsets)
    ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_gemm_offsets), (size_t)(L->e_local + 1) * 4));
  if (!L->d_bar) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_bar), 4));
  if (!L->d_peer_sync) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_peer_sync), pb));
  if (!L->d_ep_state) ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->d_ep_state), 16));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_peer_sync, ps.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemset(L->d_ep_state, 0, 16));
  {
    // ATENIA_MOE_EP_FLAGS=1: counts and completion epochs through the peers' sync buffers instead of one
    // all-gather and two one-word all-reduces per forward; ATENIA_MOE_EP_FLAG_TIMEOUT_MS bounds a wait
    const char* f = std::getenv("ATENIA_MOE_EP_FLAGS");
    L->ep_flags = f && std::atoi(f) != 0;
    const char* t = std::getenv("ATENIA_MOE_EP_FLAG_TIMEOUT_MS");
    const long ms = t ? std::atol(t) : 20000;
    L->ep_flag_limit_ns = (uint64_t)(ms < 1 ? 1 : ms) * 1000000ull;
  }
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_peer_recv_x, px.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_peer_y_perm, py.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemset(L->d_bar, 0, 4));
  L->ep_direct = true;
  return ATENIA_OK;
}

// Host form of the row placement the direct exchange computes on the device (ep_plan.cuh), exported so
// that it can be tested without GPUs.  Arrays: dst_base[E], src_base[E], sub_offsets[E + 1] (a rank
// has E / world * world = E sub-groups), gemm_offsets[E / world + 1].
int atenia_moe_ep_plan_direct(const int32_t* counts_all, int world, int num_experts, int rank, int32_t* dst_base,
                              int32_t* src_base, int32_t* sub_offsets, int32_t* gemm_offsets) {
  if (!counts_all || !dst_base || !src_base || !sub_offsets || !gemm_offsets) return ATENIA_ERR_NULL;
  if (world < 1 || num_experts < 1 || num_experts % world || rank < 0 || rank >= world) return ATENIA_ERR_SHAPE;
  atenia::ep_direct_plan(counts_all, world, num_experts, rank, dst_base, src_base, sub_offsets, gemm_offsets);
  return ATENIA_OK;
}

int atenia_moe_ep_set_token_layout(AteniaMoeLayer* L, int layout) {
  if (!L) return ATENIA_ERR_NULL;
  if (layout != ATENIA_EP_TOKENS_SHARDED && layout != ATENIA_EP_TOKENS_REPLICATED) return ATENIA_ERR_SHAPE;
  if (L->cfg.ep_world <= 1 || L->ep_direct) return ATENIA_ERR_STATE;
  L->ep_replicated = layout == ATENIA_EP_TOKENS_REPLICATED;
  return ATENIA_OK;
}

}  // extern "C"
