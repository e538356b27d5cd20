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
  // counts are kept expert-major, [E][gridDim.x]: the scan then reads consecutive blocks of one expert
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) a.block_counts[(size_t)e * gridDim.x + blockIdx.x] = hist[e];
}

// One block.  Warp w scans experts w, w + nwarps, ... over the blocks (32 blocks per step, the loads of
// up to eight steps issued before the first is consumed); then thread 0 scans experts.
__global__ void __launch_bounds__(1024) scan_kernel(DispatchArgs a, int nblk) {
  __shared__ int totals[kMaxE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  constexpr int kBatch = 8;
  for (int e = warp; e < a.E; e += nwarps) {
    const int32_t* cnt = a.block_counts + (size_t)e * nblk;
    int32_t* base = a.block_base + (size_t)e * nblk;
    int running = 0;
    for (int b0 = 0; b0 < nblk; b0 += 32 * kBatch) {
      int c[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int b = b0 + 32 * j + lane;
        c[j] = b < nblk ? cnt[b] : 0;
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int b = b0 + 32 * j + lane;
        int incl = c[j];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int v = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += v;
        }
        if (b < nblk) base[b] = running + incl - c[j];
        running += __shfl_sync(0xffffffffu, incl, 31);
      }
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
    const int pos = a.expert_offsets[e] + a.block_base[(size_t)e * gridDim.x + blockIdx.x] + before + rank_in_warp;
    a.perm[pos] = i;
    a.inv_perm[i] = pos;
  } else if (i < a.n) {
    a.inv_perm[i] = -1;  // an entry with an invalid expert id has no row: the combine skips it
  }
}

// Small batches (at most 1024 entries, i.e. decode): histogram, scan and stable placement in ONE block,
// one thread per entry -- the same permutation as the three launches above without their launch gaps.
constexpr int kSmallDispatchMax = 1024;

__global__ void __launch_bounds__(kSmallDispatchMax) dispatch_small_kernel(DispatchArgs a) {
  __shared__ int warp_cnt[kSmallDispatchMax / 32][kMaxE];  // entries of expert e in warp w, then their base
  __shared__ int offsets[kMaxE + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int j = threadIdx.x; j < nwarps * kMaxE; j += blockDim.x) (&warp_cnt[0][0])[j] = 0;
  __syncthreads();
  const int i = threadIdx.x;
  int e = -1;
  if (i < a.n) {
    e = a.topk_idx[i];
    if (e < 0 || e >= a.E) {
      report_error(a.err, ATENIA_ERR_ROUTING, 2001);
      e = -1;
    }
  }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) warp_cnt[warp][e] = __popc(peers);
  __syncthreads();
  // thread e: exclusive scan of its expert's counts over the warps (entry order), total into offsets
  if (threadIdx.x < a.E) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) {
      const int c = warp_cnt[w][threadIdx.x];
      warp_cnt[w][threadIdx.x] = run;
      run += c;
    }
    offsets[threadIdx.x + 1] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    offsets[0] = 0;
    for (int x = 0; x < a.E; ++x) offsets[x + 1] += offsets[x];
    if (a.extra_offsets) {
      a.extra_offsets[0] = 0;
      a.extra_offsets[1] = a.T;
    }
  }
  __syncthreads();
  for (int x = threadIdx.x; x <= a.E; x += blockDim.x) a.expert_offsets[x] = offsets[x];
  if (e >= 0) {
    const int pos = offsets[e] + warp_cnt[warp][e] + rank_in_warp;
    a.perm[pos] = i;
    a.inv_perm[i] = pos;
  } else if (i < a.n) {
    a.inv_perm[i] = -1;
  }
}

// Medium batches (at most 8192 entries): the same in ONE block that walks the entries in chunks of 1024 --
// a histogram pass (shared-memory atomics; the order of additions does not matter for counts), the scan,
// then per chunk the stable placement of dispatch_small_kernel on top of the counts of the chunks before.
constexpr int kMediumDispatchMax = 8192;

__global__ void __launch_bounds__(kSmallDispatchMax) dispatch_medium_kernel(DispatchArgs a) {
  __shared__ int warp_cnt[kSmallDispatchMax / 32][kMaxE];  // current chunk: entries of expert e in warp w, then their base
  __shared__ int offsets[kMaxE + 1];
  __shared__ int hist[kMaxE];     // pass 1: entries per expert; pass 2: entries of the current chunk per expert
  __shared__ int running[kMaxE];  // entries per expert placed by earlier chunks
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kSmallDispatchMax / 32;
  if (threadIdx.x < kMaxE) {
    hist[threadIdx.x] = 0;
    running[threadIdx.x] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.n; i += blockDim.x) {
    const int e = a.topk_idx[i];
    if (e >= 0 && e < a.E) atomicAdd(&hist[e], 1);
    else report_error(a.err, ATENIA_ERR_ROUTING, 2002);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    offsets[0] = 0;
    for (int x = 0; x < a.E; ++x) offsets[x + 1] = offsets[x] + hist[x];
    if (a.extra_offsets) {
      a.extra_offsets[0] = 0;
      a.extra_offsets[1] = a.T;
    }
  }
  __syncthreads();
  for (int x = threadIdx.x; x <= a.E; x += blockDim.x) a.expert_offsets[x] = offsets[x];
  for (int c0 = 0; c0 < a.n; c0 += kSmallDispatchMax) {
    for (int j = threadIdx.x; j < kWarps * kMaxE; j += blockDim.x) (&warp_cnt[0][0])[j] = 0;
    __syncthreads();
    const int i = c0 + threadIdx.x;
    int e = -1;
    if (i < a.n) {
      e = a.topk_idx[i];
      if (e < 0 || e >= a.E) e = -1;  // (reported by the histogram pass)
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_cnt[warp][e] = __popc(peers);
    __syncthreads();
    if (threadIdx.x < a.E) {
      int run = 0;
      for (int w = 0; w < kWarps; ++w) {
        const int c = warp_cnt[w][threadIdx.x];
        warp_cnt[w][threadIdx.x] = run;
        run += c;
      }
      hist[threadIdx.x] = run;
    }
    __syncthreads();
    if (e >= 0) {
      const int pos = offsets[e] + running[e] + warp_cnt[warp][e] + rank_in_warp;
      a.perm[pos] = i;
      a.inv_perm[i] = pos;
    } else if (i < a.n) {
      a.inv_perm[i] = -1;
    }
    __syncthreads();
    if (threadIdx.x < a.E) running[threadIdx.x] += hist[threadIdx.x];
    // (the zeroing at the top of the next chunk is followed by a barrier before running[] is read again)
  }
}

// Row gather: x_perm[r, :] = bf16(x[perm[r] / k, :]).  One warp per destination row, eight rows per
// block in flight and a grid that loops; every lane keeps four 16-byte vectors in flight.  `placed`
// points at expert_offsets[E], the number of rows the placement actually wrote: entries with an
// invalid expert id get no row, so perm beyond that count holds whatever an earlier call left there
// and must not be followed.  Rows n_rows .. n_rows + T - 1 of the index space convert x itself
// (f32 input with a shared expert: x_bf16 = bf16(x)).
constexpr int kGatherWarps = 8;

__global__ void __launch_bounds__(kGatherWarps * 32) gather_rows_kernel(const void* __restrict__ x, int x_is_f32,
                                                                         const int32_t* __restrict__ perm,
                                                                         const int32_t* __restrict__ placed,
                                                                         int n_rows, int k, int d,
                                                                         __nv_bfloat16* __restrict__ x_perm,
                                                                         __nv_bfloat16* __restrict__ x_bf16, int T,
                                                                         int total_rows) {
  const int lane = threadIdx.x & 31;
  const int nvec = d / 8;
  const int n_placed = n_rows > 0 ? *placed : 0;
  for (int r = blockIdx.x * kGatherWarps + (threadIdx.x >> 5); r < total_rows; r += gridDim.x * kGatherWarps) {
    int src_t, dst_r;
    __nv_bfloat16* dst;
    if (r < n_rows) {
      if (r >= n_placed) continue;
      src_t = perm[r] / k;
      if (src_t < 0 || src_t >= T) continue;
      dst_r = r;
      dst = x_perm;
    } else {
      src_t = r - n_rows;
      dst_r = src_t;
      dst = x_bf16;
    }
    uint4* drow = reinterpret_cast<uint4*>(dst + (size_t)dst_r * d);
    if (x_is_f32) {
      const float4* srow = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)src_t * d);
      for (int v = lane; v < nvec; v += 64) {
        float4 a0 = srow[2 * v], b0 = srow[2 * v + 1], a1, b1;
        const bool two = v + 32 < nvec;
        if (two) {
          a1 = srow[2 * (v + 32)];
          b1 = srow[2 * (v + 32) + 1];
        }
        drow[v] = make_uint4(pack_bf16x2(a0.x, a0.y), pack_bf16x2(a0.z, a0.w), pack_bf16x2(b0.x, b0.y),
                             pack_bf16x2(b0.z, b0.w));
        if (two)
          drow[v + 32] = make_uint4(pack_bf16x2(a1.x, a1.y), pack_bf16x2(a1.z, a1.w), pack_bf16x2(b1.x, b1.y),
                                    pack_bf16x2(b1.z, b1.w));
      }
    } else {
      const uint4* srow = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + (size_t)src_t * d);
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
  }
}

}  // namespace

int launch_dispatch(const DispatchArgs& a, cudaStream_t s) {
  if (a.E > kMaxE) return ATENIA_ERR_UNSUPPORTED;
  if (a.n > 0 && a.n <= kSmallDispatchMax) {
    const int threads = ((a.n + 31) / 32 * 32) < a.E ? ((a.E + 31) / 32 * 32) : ((a.n + 31) / 32 * 32);
    dispatch_small_kernel<<<1, threads, 0, s>>>(a);
    count_launch();
    return (int)cudaGetLastError();
  }
  if (a.n > kSmallDispatchMax && a.n <= kMediumDispatchMax) {
    dispatch_medium_kernel<<<1, kSmallDispatchMax, 0, s>>>(a);
    count_launch();
    return (int)cudaGetLastError();
  }
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
  const int total = n_rows + extra;
  if (total <= 0) return ATENIA_OK;
  // enough blocks to keep every SM's memory pipeline full; the kernel loops over the rest
  const int want = (total + kGatherWarps - 1) / kGatherWarps;
  const int cap = 148 * 8;
  gather_rows_kernel<<<want < cap ? want : cap, kGatherWarps * 32, 0, s>>>(x, x_is_f32, perm, placed, n_rows, k, d, x_perm,
                                                                          x_bf16, T, total);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace atenia
