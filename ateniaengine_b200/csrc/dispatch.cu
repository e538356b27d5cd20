// Dispatch: the canonical permutation of (token, slot) entries by expert, and the row gather.
//
// The reference never builds a permutation: it loops over tokens in order and, inside a token, over
// the selected experts in ascending order (src/moe/graph_op.rs:346-348, src/moe/sparse.rs:173-175).
// The only order it defines is therefore "tokens ascending, experts ascending inside a token", and
// the permutation emitted here is the stable counting sort of the flat entry list i = t*k + s by
// expert id: expert_offsets[e] = number of entries with a smaller expert, and the rows of one
// expert keep ascending i.  Three launches: per-block histogram, scan, stable placement.
#include "common.cuh"

namespace atenia {
namespace {

constexpr int kMaxE = 128;

__global__ void __launch_bounds__(kDispatchChunk) count_kernel(DispatchArgs a) {
  __shared__ int hist[kMaxE];
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  int i = blockIdx.x * kDispatchChunk + threadIdx.x;
  if (i < a.n) {
    int e = a.topk_idx[i];
    if (e < 0 || e >= a.E) {
      report_error(a.err, ATENIA_ERR_ROUTING, 2000);
    } else {
      atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) a.block_counts[(size_t)blockIdx.x * a.E + e] = hist[e];
}

// One block.  Warp w scans experts w, w + nwarps, ... over the blocks; then thread 0 scans experts.
__global__ void __launch_bounds__(1024) scan_kernel(DispatchArgs a, int nblk) {
  __shared__ int totals[kMaxE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int e = warp; e < a.E; e += nwarps) {
    int running = 0;
    for (int b0 = 0; b0 < nblk; b0 += 32) {
      int b = b0 + lane;
      int c = b < nblk ? a.block_counts[(size_t)b * a.E + e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (b < nblk) a.block_base[(size_t)b * a.E + e] = running + incl - c;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) totals[e] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < a.E; ++e) {
      a.expert_offsets[e] = run;
      run += totals[e];
    }
    a.expert_offsets[a.E] = run;
    if (a.extra_offsets) {
      a.extra_offsets[0] = 0;
      a.extra_offsets[1] = a.T;
    }
  }
}

__global__ void __launch_bounds__(kDispatchChunk) place_kernel(DispatchArgs a) {
  constexpr int kW = kDispatchChunk / 32;
  __shared__ int warp_cnt[kW][kMaxE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int j = threadIdx.x; j < kW * kMaxE; j += blockDim.x) (&warp_cnt[0][0])[j] = 0;
  __syncthreads();
  const int i = blockIdx.x * kDispatchChunk + threadIdx.x;
  int e = -1;
  if (i < a.n) {
    e = a.topk_idx[i];
    if (e < 0 || e >= a.E) e = -1;
  }
  // lanes holding the same expert, in lane order = entry order
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) warp_cnt[warp][e] = __popc(peers);
  __syncthreads();
  if (e >= 0) {
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
    const int pos = a.expert_offsets[e] + a.block_base[(size_t)blockIdx.x * a.E + e] + before + rank_in_warp;
    a.perm[pos] = i;
    a.inv_perm[i] = pos;
  } else if (i < a.n) {
    a.inv_perm[i] = -1;  // an entry with an invalid expert id has no row: the combine skips it
  }
}

// One block per destination row; 16-byte vectors.  `placed` points at expert_offsets[E], the number
// of rows the placement actually wrote: entries with an invalid expert id get no row, so perm beyond
// that count holds whatever an earlier call left there and must not be followed.
__global__ void __launch_bounds__(256) gather_rows_kernel(const void* __restrict__ x, int x_is_f32,
                                                           const int32_t* __restrict__ perm,
                                                           const int32_t* __restrict__ placed, int n_rows, int k,
                                                           int d, __nv_bfloat16* __restrict__ x_perm,
                                                           __nv_bfloat16* __restrict__ x_bf16, int T) {
  const int r = blockIdx.x;
  const bool copy_row = r >= n_rows;  // blocks past n_rows convert x itself (f32 input, shared expert)
  int src_t, dst_r;
  __nv_bfloat16* dst;
  if (!copy_row) {
    if (r >= *placed) return;
    src_t = perm[r] / k;
    if (src_t < 0 || src_t >= T) return;
    dst_r = r;
    dst = x_perm;
  } else {
    src_t = r - n_rows;
    if (src_t >= T) return;
    dst_r = src_t;
    dst = x_bf16;
  }
  uint4* drow = reinterpret_cast<uint4*>(dst + (size_t)dst_r * d);
  const int nvec = d / 8;
  if (x_is_f32) {
    const float4* srow = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)src_t * d);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float4 a = srow[2 * v], b = srow[2 * v + 1];
      drow[v] = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                           pack_bf16x2(b.z, b.w));
    }
  } else {
    const uint4* srow = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + (size_t)src_t * d);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) drow[v] = srow[v];
  }
}

}  // namespace

int launch_dispatch(const DispatchArgs& a, cudaStream_t s) {
  if (a.E > kMaxE) return ATENIA_ERR_UNSUPPORTED;
  const int nblk = (a.n + kDispatchChunk - 1) / kDispatchChunk;
  if (nblk > 0) {
    count_kernel<<<nblk, kDispatchChunk, 0, s>>>(a);
    count_launch();
  }
  scan_kernel<<<1, 1024, 0, s>>>(a, nblk);
  count_launch();
  if (nblk > 0) {
    place_kernel<<<nblk, kDispatchChunk, 0, s>>>(a);
    count_launch();
  }
  return (int)cudaGetLastError();
}

int launch_gather_rows(const void* x, int x_is_f32, const int32_t* perm, const int32_t* placed, int n_rows, int k,
                       int d, __nv_bfloat16* x_perm, __nv_bfloat16* x_bf16, int T, cudaStream_t s) {
  const int extra = x_bf16 ? T : 0;
  if (n_rows + extra <= 0) return ATENIA_OK;
  gather_rows_kernel<<<n_rows + extra, 256, 0, s>>>(x, x_is_f32, perm, placed, n_rows, k, d, x_perm, x_bf16, T);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace atenia
