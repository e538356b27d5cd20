// Router on the f64 tensor cores: logits[t, e] = sum_c W[e, c] * x[t, c] as an m8n8k4 DMMA product,
// then the same softmax + top-k as router.cu.
//
// The reference accumulates the router matvec in f64 (src/moe/dense.rs:97-115, :333) and rounds the
// sum to f32.  router.cu does that with scalar f64 multiply-adds and is bound by the FP64 pipe of
// the CUDA cores; for 64 experts it is a fifth of a DeepSeek-shaped forward.  Here the same f64
// products go through mma.sync.m8n8k4.f64 (there is no tcgen05 form for f64): inputs are the exact
// f64 values of the bf16 / f32 operands, accumulation is f64, only the order of the additions
// differs from the serial loop (last bits of a 53-bit sum, far below the rounding to f32).
//
// Operands are streamed from global memory straight into the fragments: nothing is staged in shared
// memory and the main loop has no barrier.  (An earlier form that staged x and the router matrix as f64
// in shared memory, 32 tokens per CTA, was bound by its two block-wide barriers per 32-k chunk; measured
// on B200 it was never faster -- DeepSeek-V2-Lite shape, whole forward: 512 tokens 0.310 vs 0.302 ms,
// 2048 tokens 0.437 vs 0.426 ms, 8192 tokens 1.103 vs 1.100 ms -- and was removed.)
#include <cstdlib>
#include <type_traits>

#include "route_warp.cuh"

namespace atenia {
namespace {

constexpr int kDW = 8;  // warps per CTA (16 in the form for small batches)

// D[8x8] += A[8x4] * B[4x8].  Lane l holds A[l / 4][l % 4], B[l % 4][l / 4] and D[l / 4][2 (l % 4) + {0, 1}].
__device__ __forceinline__ void dmma884(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

template <int I>
using Int = std::integral_constant<int, I>;

// N consecutive 32-bit words (N = 4 or 8) from a 16-byte aligned address
template <int N, bool LDG>
__device__ __forceinline__ void ld_words(uint32_t (&w)[N], const void* p) {
#pragma unroll
  for (int i = 0; i < N / 4; ++i) {
    const uint4 v = LDG ? __ldg(static_cast<const uint4*>(p) + i) : static_cast<const uint4*>(p)[i];
    w[4 * i] = v.x;
    w[4 * i + 1] = v.y;
    w[4 * i + 2] = v.z;
    w[4 * i + 3] = v.w;
  }
}
template <int N>
__device__ __forceinline__ void zero_words(uint32_t (&w)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) w[i] = 0u;
}
// element j (a constant after unrolling) of a lane's eight consecutive x values held as raw words
template <bool XF, int N>
__device__ __forceinline__ double x_elem(const uint32_t (&w)[N], int j) {
  if (XF) return (double)__uint_as_float(w[j]);
  return (double)((j & 1) ? bf16hi(w[j >> 1]) : bf16lo(w[j >> 1]));
}

// The WARPS warps of a CTA are arranged NW_N x NW_K (NW_N = (E_T / 8) / NTW across the 8-expert tiles,
// the rest across k): a warp owns NTW 8-expert tiles and the k-range [kslice KW, (kslice+1) KW)
// of the dot products of the CTA's 8 MT tokens.  The summation index of an m8n8k4 product is free to be
// permuted as long as A and B agree, so lane (r, c) = (lane / 4, lane % 4) loads EIGHT consecutive k of
// token row r (16 bytes of bf16) and of expert row r of each of its tiles (32 bytes of f32) at
// k = base + 8 c, and step j of eight uses element j of every lane's values: the four lanes of a row
// cover 32 consecutive k, global loads are whole sectors (the warps of one k-slice read the same token
// values: the first brings them into L1).  The raw words of the next 32 k are in flight, in a second set
// of registers, while the current ones are converted and multiplied.
//
// A value is converted to f64 each time a warp uses it: a warp that owns NTW tiles and MT token tiles
// converts MT + NTW values per MT * NTW products, and the conversion unit is as scarce as the f64 tensor
// pipe.  With one tile per warp (NTW = 1, MT = 2: 1.5 conversions per product) the conversions set the
// pace; two tiles per warp (1.0) leave the tensor pipe as the busier unit.  Measured on B200, routing
// phase (router + dispatch + gather) of a DeepSeek-V2-Lite-shaped layer, 8192 tokens: 0.195 ms with one
// tile per warp, 0.171 ms with two; four tiles per warp (0.75 conversions per product) measured 0.163 ms
// alone but need 42 KB of shared memory for the partial sums, which no longer fits on an SM beside a CTA
// of the expert GEMMs (the shared expert runs there at the same time).  m16n8k4 products instead of
// m8n8k4 changed nothing.
//
// Partial sums of the k-slices are added through shared memory in slice order (fixed), then the bias, the
// rounding to f32 and the routing of each token by one warp (route_one_warp).
template <int E_T, int MT, int NTW, bool XF, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) router_dmma_direct_kernel(RouterArgs a, int kw) {
  constexpr int NT = E_T / 8;
  constexpr int NW_N = NT / NTW;
  constexpr int NW_K = WARPS / NW_N;
  static_assert(NW_N >= 1 && NW_N * NTW == NT && NW_N * NW_K == WARPS, "warp arrangement");
  constexpr int kTok = 8 * MT;
  constexpr int XW = XF ? 8 : 4;  // 32-bit words of a lane's eight x values
  __shared__ double part_s[WARPS][MT][NTW][32][2];
  __shared__ double gpart_s[NW_K][kTok];
  __shared__ float lg_s[kTok][E_T];
  __shared__ double exps_s[WARPS][E_T];
  __shared__ int32_t idx_s[kTok][kMaxK];
  __shared__ float w_s[kTok][kMaxK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ngrp = warp % NW_N, kslice = warp / NW_N;
  const int r = lane >> 2, c = lane & 3;
  const int t0 = blockIdx.x * kTok;
  const int d = a.d, E = a.E;
  const int k_begin = kslice * kw < d ? kslice * kw : d, k_end = (k_begin + kw < d) ? k_begin + kw : d;
  const bool do_gate = a.gate_vec != nullptr && ngrp == 0;  // one warp per k-slice takes the gate dot product

  double acc[MT][NTW][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < NTW; ++j) acc[mt][j][0] = acc[mt][j][1] = 0.0;
  double gacc[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) gacc[mt] = 0.0;

  // raw words of two steps
  uint32_t xq[2][MT][XW];
  uint32_t wq[2][NTW][8];
  uint32_t gq[2][8];
  auto fetch = [&](auto BUF, int kb) {
    constexpr int b = decltype(BUF)::value;
    const int k = kb + c * 8;
    const bool k_ok = k < k_end;  // d and kw are multiples of 8: a lane's values are all in or all out
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int tg = t0 + mt * 8 + r;
      zero_words(xq[b][mt]);
      if (k_ok && tg < a.T) {
        if (XF) ld_words<XW, false>(xq[b][mt], static_cast<const float*>(a.x) + (size_t)tg * d + k);
        else ld_words<XW, false>(xq[b][mt], static_cast<const __nv_bfloat16*>(a.x) + (size_t)tg * d + k);
      }
    }
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int e = (ngrp * NTW + j) * 8 + r;
      zero_words(wq[b][j]);
      if (k_ok && e < E) ld_words<8, true>(wq[b][j], a.w_router + (size_t)e * d + k);
    }
    zero_words(gq[b]);
    if (do_gate && k_ok) ld_words<8, true>(gq[b], a.gate_vec + k);
  };
  auto multiply = [&](auto BUF) {
    constexpr int b = decltype(BUF)::value;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      double xv[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) xv[mt] = x_elem<XF>(xq[b][mt], j);
      if (do_gate) {
        const double g = (double)__uint_as_float(gq[b][j]);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) gacc[mt] = fma(g, xv[mt], gacc[mt]);
      }
#pragma unroll
      for (int jt = 0; jt < NTW; ++jt) {
        const double wv = (double)__uint_as_float(wq[b][jt][j]);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) dmma884(acc[mt][jt], xv[mt], wv);
      }
    }
  };
  if (k_begin < k_end) fetch(Int<0>{}, k_begin);
  for (int kb = k_begin; kb < k_end; kb += 64) {
    const bool more = kb + 32 < k_end;
    if (more) fetch(Int<1>{}, kb + 32);
    multiply(Int<0>{});
    if (more) {
      if (kb + 64 < k_end) fetch(Int<0>{}, kb + 64);
      multiply(Int<1>{});
    }
  }
  // partial sums of this warp's k-range: C[row r][columns 2c, 2c + 1] of every tile it owns
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int jt = 0; jt < NTW; ++jt) {
      part_s[warp][mt][jt][lane][0] = acc[mt][jt][0];
      part_s[warp][mt][jt][lane][1] = acc[mt][jt][1];
    }
  if (do_gate) {
    // the four lanes of a row hold the four k-quarters of the gate dot product: fold them (fixed tree)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      double v = gacc[mt];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      if (c == 0) gpart_s[kslice][mt * 8 + r] = v;
    }
  }
  __syncthreads();
  // logits: the k-slices' partial sums in slice order, then the bias, then the rounding to f32
  for (int i = threadIdx.x; i < kTok * E_T; i += blockDim.x) {
    const int t = i / E_T, e = i - t * E_T;
    if (e >= E) continue;
    const int mt = t >> 3, rr = t & 7, nt = e >> 3, col = e & 7;
    const int og = nt / NTW, jt = nt - og * NTW;
    const int src_lane = rr * 4 + (col >> 1), which = col & 1;
    double v = 0.0;
#pragma unroll
    for (int ks = 0; ks < NW_K; ++ks) v += part_s[ks * NW_N + og][mt][jt][src_lane][which];
    if (a.bias) v += (double)a.bias[e];
    const float f = (float)v;
    lg_s[t][e] = f;
    const int tg = t0 + t;
    if (a.logits && tg < a.T) a.logits[(size_t)tg * E + e] = f;
  }
  if (a.gate_vec && a.gate_scale && threadIdx.x < kTok) {
    const int t = threadIdx.x, tg = t0 + t;
    double v = 0.0;
    for (int ks = 0; ks < NW_K; ++ks) v += gpart_s[ks][t];
    if (tg < a.T) a.gate_scale[tg] = (float)(1.0 / (1.0 + exp(-v)));
  }
  __syncthreads();
  for (int t = warp; t < kTok; t += WARPS) {
    const int tg = t0 + t;
    if (tg >= a.T) continue;
    int rc = route_one_warp<(E_T + 31) / 32>(lg_s[t], E, a.k, a.renormalize, lane, idx_s[t], w_s[t], exps_s[warp]);
    if (rc) {
      if (lane == 0) report_error(a.err, rc, 1005);
      if (lane < a.k) {  // keep downstream kernels in bounds
        idx_s[t][lane] = lane;
        w_s[t][lane] = 0.f;
      }
    }
    __syncwarp();
    if (lane < a.k) {
      a.topk_idx[(size_t)tg * a.k + lane] = idx_s[t][lane];
      a.topk_w[(size_t)tg * a.k + lane] = w_s[t][lane];
    }
  }
}

template <int E_T, int MT, int NTW, int WARPS>
int launch_form(const RouterArgs& a, cudaStream_t s) {
  constexpr int NW_K = WARPS / ((E_T / 8) / NTW);
  constexpr int kTok = 8 * MT;
  // k-range of a k-slice: d over the slices, rounded up to whole 32-k steps
  const int kw = ((a.d + NW_K - 1) / NW_K + 31) / 32 * 32;
  const int grid = (a.T + kTok - 1) / kTok;
  if (a.x_is_f32) router_dmma_direct_kernel<E_T, MT, NTW, true, WARPS><<<grid, WARPS * 32, 0, s>>>(a, kw);
  else router_dmma_direct_kernel<E_T, MT, NTW, false, WARPS><<<grid, WARPS * 32, 0, s>>>(a, kw);
  return (int)cudaGetLastError();
}

// Two forms.  A batch whose 8-token CTAs fit the SMs in one round is bound by the latency of its
// dependent load -> multiply steps, not by a pipe: 16 warps per CTA cut the k-range, and with it the
// number of steps, of every warp in half (DeepSeek-V2-Lite shape, 1024 tokens: router 41 -> 22 us).
// Larger batches take 16 tokens and 8 warps per CTA, 2 to 3 CTAs per SM.
constexpr int kSmallBatchCtas = 148;

template <int E_T>
int launch_direct(const RouterArgs& a, cudaStream_t s) {
  constexpr int NT = E_T / 8;
  constexpr int NTW = NT < 2 ? NT : 2;
  if ((a.T + 7) / 8 <= kSmallBatchCtas) return launch_form<E_T, 1, NTW, 2 * kDW>(a, s);
  return launch_form<E_T, 2, NTW, kDW>(a, s);
}

}  // namespace

int launch_router_dmma(const RouterArgs& a, cudaStream_t s) {
  if (a.T <= 0) return ATENIA_OK;
  if (a.k > kMaxK || a.E > 128 || a.d % 16 != 0) return ATENIA_ERR_UNSUPPORTED;
  int rc;
  if (a.E <= 8) rc = launch_direct<8>(a, s);
  else if (a.E <= 16) rc = launch_direct<16>(a, s);
  else if (a.E <= 32) rc = launch_direct<32>(a, s);
  else if (a.E <= 64) rc = launch_direct<64>(a, s);
  else rc = launch_direct<128>(a, s);
  count_launch();
  return rc;
}

}  // namespace atenia
