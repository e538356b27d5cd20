// Softmax + top-k of one token by one warp, shared by the router kernels.
#pragma once
#include "common.cuh"

namespace atenia {

constexpr int kMaxK = 8;

// Softmax + top-k for one token by one warp.  `lg` holds E f32 logits in shared memory.
// Follows the reference's sequence: f32 maximum, exp((f64)(v - max)) with the subtraction in f32,
// the f64 sum accumulated in ascending expert order by one lane, f32 weights, then k rounds of
// "largest weight, lowest index" and a renormalisation summed in ascending index order.
template <int EPL>
__device__ __forceinline__ int route_one_warp(const float* lg, int E, int k, int renormalize, int lane,
                                              int32_t* idx_out, float* w_out, double* exps /* smem, E */) {
  float mx = -INFINITY;
  bool finite = true;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    int e = lane + 32 * j;
    if (e < E) {
      float v = lg[e];
      if (!isfinite(v)) finite = false;
      mx = fmaxf(mx, v);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (__any_sync(0xffffffffu, !finite)) return ATENIA_ERR_ROUTING;
  double ex[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    int e = lane + 32 * j;
    ex[j] = 0.0;
    if (e < E) {
      ex[j] = exp((double)__fsub_rn(lg[e], mx));
      exps[e] = ex[j];
    }
  }
  __syncwarp();
  double sum = 0.0;
  if (lane == 0)
    for (int e = 0; e < E; ++e) sum += exps[e];
  sum = __shfl_sync(0xffffffffu, sum, 0);
  const double inv = sum > 0.0 ? 1.0 / sum : 0.0;
  float p[EPL];
  bool taken[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    p[j] = (float)(ex[j] * inv);
    taken[j] = (lane + 32 * j) >= E;  // slots past E never compete
  }
  for (int s = 0; s < k; ++s) {
    float bw = -1.0f;  // weights are >= 0
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      if (!taken[j] && p[j] > bw) {  // ascending j = ascending index: strict > keeps the lower one
        bw = p[j];
        bi = lane + 32 * j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ow = __shfl_xor_sync(0xffffffffu, bw, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ow > bw || (ow == bw && oi < bi)) {
        bw = ow;
        bi = oi;
      }
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (lane + 32 * j == bi) taken[j] = true;
  }
  // selected experts in ascending order: rank of each selected slot among the selected
  int m_before = 0;
  double ssum = 0.0;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    bool sel = taken[j] && (lane + 32 * j) < E;
    unsigned mask = __ballot_sync(0xffffffffu, sel);
    int rank = m_before + __popc(mask & ((1u << lane) - 1u));
    if (sel) {
      idx_out[rank] = lane + 32 * j;
      exps[rank] = (double)p[j];  // reuse as the selected-weight list (ascending index)
    }
    m_before += __popc(mask);
  }
  __syncwarp();
  if (lane == 0)
    for (int s = 0; s < k; ++s) ssum += exps[s];
  ssum = __shfl_sync(0xffffffffu, ssum, 0);
  if (!(ssum > 0.0)) return ATENIA_ERR_ROUTING;
  const double scale = renormalize ? 1.0 / ssum : 1.0;
  if (lane < k) w_out[lane] = (float)(exps[lane] * scale);
  __syncwarp();
  return 0;
}

}  // namespace atenia
