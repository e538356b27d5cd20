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

#include "route_warp.cuh"

namespace atenia {
namespace {

constexpr int kDW = 8;  // warps per CTA

// D[8x8] += A[8x4] * B[4x8].  Lane l holds A[l / 4][l % 4], B[l % 4][l / 4] and D[l / 4][2 (l % 4) + {0, 1}].
__device__ __forceinline__ void dmma884(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

// The eight warps of a CTA are arranged NW_N x NW_K (NW_N = min(8, E_T / 8) across the 8-expert tiles,
// the rest across k): a warp owns NTW 8-expert tiles and the k-range [kslice KW, (kslice+1) KW)
// of the dot products of the CTA's 8 MT tokens.  The summation index of an m8n8k4 product is free to be
// permuted as long as A and B agree, so lane (r, c) = (lane / 4, lane % 4) loads EIGHT consecutive k of
// token row r (16 bytes of bf16) and of expert row r of each of its tiles (32 bytes of f32) at
// k = base + 8 c, and step j of eight uses element j of every lane's vectors: the four lanes of a row
// cover 32 consecutive k, global loads are whole sectors (the warps of one k-slice read the same token
// vectors: the first brings them into L1).  The vectors of the next 32 k are in flight while the current
// ones are multiplied.  Partial sums of the k-slices are added through shared memory in slice order
// (fixed), then the bias, the rounding to f32 and the routing of each token by one warp (route_one_warp).
template <int E_T, int MT>
__global__ void __launch_bounds__(kDW * 32) router_dmma_direct_kernel(RouterArgs a, int kw) {
  constexpr int NT = E_T / 8;
  constexpr int NW_N = NT < kDW ? NT : kDW;
  constexpr int NW_K = kDW / NW_N;
  constexpr int NTW = NT / NW_N;
  constexpr int kTok = 8 * MT;
  __shared__ double part_s[kDW][MT][NTW][32][2];
  __shared__ double gpart_s[NW_K][kTok];
  __shared__ float lg_s[kTok][E_T];
  __shared__ double exps_s[kDW][E_T];
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

  // raw vectors of one step: x as bf16 uses xq[mt][0] only, as f32 both; W always two float4
  uint4 xq[MT][2];
  float4 wq[NTW][2];
  float4 gq[2];
  auto fetch = [&](int kb) {
    const int k = kb + c * 8;
    const bool k_ok = k < k_end;  // d and kw are multiples of 8: a vector is all in or all out
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int tg = t0 + mt * 8 + r;
      xq[mt][0] = make_uint4(0, 0, 0, 0);
      xq[mt][1] = make_uint4(0, 0, 0, 0);
      if (k_ok && tg < a.T) {
        if (a.x_is_f32) {
          const uint4* p = reinterpret_cast<const uint4*>(static_cast<const float*>(a.x) + (size_t)tg * d + k);
          xq[mt][0] = p[0];
          xq[mt][1] = p[1];
        } else {
          xq[mt][0] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.x) + (size_t)tg * d + k);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NTW; ++j) {
      const int e = (ngrp * NTW + j) * 8 + r;
      wq[j][0] = wq[j][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k_ok && e < E) {
        const float4* p = reinterpret_cast<const float4*>(a.w_router + (size_t)e * d + k);
        wq[j][0] = __ldg(p);
        wq[j][1] = __ldg(p + 1);
      }
    }
    gq[0] = gq[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (do_gate && k_ok) {
      const float4* p = reinterpret_cast<const float4*>(a.gate_vec + k);
      gq[0] = __ldg(p);
      gq[1] = __ldg(p + 1);
    }
  };
  if (k_begin < k_end) fetch(k_begin);
  for (int kb = k_begin; kb < k_end; kb += 32) {
    double xd[MT][8], wd[NTW][8];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (a.x_is_f32) {
        const uint32_t u[8] = {xq[mt][0].x, xq[mt][0].y, xq[mt][0].z, xq[mt][0].w,
                               xq[mt][1].x, xq[mt][1].y, xq[mt][1].z, xq[mt][1].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) xd[mt][j] = (double)__uint_as_float(u[j]);
      } else {
        const uint32_t u[4] = {xq[mt][0].x, xq[mt][0].y, xq[mt][0].z, xq[mt][0].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xd[mt][2 * j] = (double)bf16lo(u[j]);
          xd[mt][2 * j + 1] = (double)bf16hi(u[j]);
        }
      }
    }
#pragma unroll
    for (int jt = 0; jt < NTW; ++jt) {
      const float f[8] = {wq[jt][0].x, wq[jt][0].y, wq[jt][0].z, wq[jt][0].w,
                          wq[jt][1].x, wq[jt][1].y, wq[jt][1].z, wq[jt][1].w};
#pragma unroll
      for (int j = 0; j < 8; ++j) wd[jt][j] = (double)f[j];
    }
    if (do_gate) {
      const float g[8] = {gq[0].x, gq[0].y, gq[0].z, gq[0].w, gq[1].x, gq[1].y, gq[1].z, gq[1].w};
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < 8; ++j) gacc[mt] = fma((double)g[j], xd[mt][j], gacc[mt]);
    }
    if (kb + 32 < k_end) fetch(kb + 32);
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int jt = 0; jt < NTW; ++jt)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) dmma884(acc[mt][jt], xd[mt][j], wd[jt][j]);
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
  for (int t = warp; t < kTok; t += kDW) {
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

template <int E_T>
int launch_direct(const RouterArgs& a, cudaStream_t s) {
  constexpr int NT = E_T / 8;
  constexpr int NW_K = kDW / (NT < kDW ? NT : kDW);
  // k-range of a k-slice: d over the slices, rounded up to whole 32-k steps
  const int kw = ((a.d + NW_K - 1) / NW_K + 31) / 32 * 32;
  if (a.T >= 8192 || (E_T > 16 && a.T >= 2048)) {
    router_dmma_direct_kernel<E_T, 2><<<(a.T + 15) / 16, kDW * 32, 0, s>>>(a, kw);
  } else {
    router_dmma_direct_kernel<E_T, 1><<<(a.T + 7) / 8, kDW * 32, 0, s>>>(a, kw);
  }
  return (int)cudaGetLastError();
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
