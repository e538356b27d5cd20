// Router for small batches: the d-long dot products are cut into 128-wide slices over many CTAs.
//
// router.cu gives every 8 (or 16) tokens one CTA that walks all of d; a CTA takes tens of
// microseconds however few tokens there are, so at decode sizes the router is a large part of a
// layer and runs on one SM.  Here CTA (slice, token block) computes the f64 partial logits of 8 tokens
// over k in [128 slice, 128 slice + 128) and leaves them in a workspace; the last CTA of a token block
// to finish (an atomic counter decides) adds the slices in ascending order, adds the bias, rounds to
// f32 and runs the same softmax + top-k (route_one_warp).  Every order of additions is fixed, so
// results do not depend on scheduling; against router.cu only the order of f64 additions differs.
//
//   warp w of a CTA owns experts w, w + 8, ...; lane l owns k = 128 slice + 4 l .. + 3 for all 8 tokens
//   (x in registers as f64, loaded once per CTA; the router row is one coalesced 512-byte load per
//   expert), partial sums are folded over the lanes with a fixed shuffle tree.
#include "route_warp.cuh"

namespace atenia {
namespace {

constexpr int kSkTok = 8;     // tokens per CTA
constexpr int kSkSlice = 128; // k values per CTA
constexpr int kSkWarps = 8;

template <int E_T>
__global__ void __launch_bounds__(kSkWarps * 32) router_splitk_kernel(RouterArgs a, int ksplit, int n_tb) {
  __shared__ float lg_s[kSkTok][E_T];
  __shared__ double exps_s[kSkWarps][E_T];
  __shared__ int32_t idx_s[kSkTok][kMaxK];
  __shared__ float w_s[kSkTok][kMaxK];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slice = blockIdx.x, tb = blockIdx.y;
  const int t0 = tb * kSkTok;
  const int d = a.d, E = a.E;
  const int k0 = slice * kSkSlice + lane * 4;
  const bool k_ok = k0 < d;  // d is a multiple of 16: four consecutive k are all in or all out

  double xk[kSkTok][4];
#pragma unroll
  for (int t = 0; t < kSkTok; ++t) {
    const int tg = t0 + t;
    xk[t][0] = xk[t][1] = xk[t][2] = xk[t][3] = 0.0;
    if (tg < a.T && k_ok) {
      if (a.x_is_f32) {
        const float4 v = *reinterpret_cast<const float4*>(static_cast<const float*>(a.x) + (size_t)tg * d + k0);
        xk[t][0] = v.x; xk[t][1] = v.y; xk[t][2] = v.z; xk[t][3] = v.w;
      } else {
        const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(a.x) + (size_t)tg * d + k0);
        xk[t][0] = bf16lo(u.x); xk[t][1] = bf16hi(u.x); xk[t][2] = bf16lo(u.y); xk[t][3] = bf16hi(u.y);
      }
    }
  }
  double* part = a.sk_part + ((size_t)slice * n_tb + tb) * kSkTok * E_T;
  auto fold = [&](double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  };
  for (int e = warp; e < E; e += kSkWarps) {
    double w[4] = {0.0, 0.0, 0.0, 0.0};
    if (k_ok) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(a.w_router + (size_t)e * d + k0));
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
#pragma unroll
    for (int t = 0; t < kSkTok; ++t) {
      double acc = w[0] * xk[t][0];
      acc = fma(w[1], xk[t][1], acc);
      acc = fma(w[2], xk[t][2], acc);
      acc = fma(w[3], xk[t][3], acc);
      acc = fold(acc);
      if (lane == 0) part[t * E_T + e] = acc;
    }
  }
  if (a.gate_vec && warp == 0) {  // partial dot products with the shared expert's gate vector
    double g[4] = {0.0, 0.0, 0.0, 0.0};
    if (k_ok) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(a.gate_vec + k0));
      g[0] = v.x; g[1] = v.y; g[2] = v.z; g[3] = v.w;
    }
#pragma unroll
    for (int t = 0; t < kSkTok; ++t) {
      double acc = g[0] * xk[t][0];
      acc = fma(g[1], xk[t][1], acc);
      acc = fma(g[2], xk[t][2], acc);
      acc = fma(g[3], xk[t][3], acc);
      acc = fold(acc);
      if (lane == 0) a.sk_gate[((size_t)slice * n_tb + tb) * kSkTok + t] = acc;
    }
  }
  // the last CTA of this token block to get here finishes the block
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&a.sk_counters[tb], 1u) == (unsigned)(ksplit - 1)) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < kSkTok * E; i += blockDim.x) {
    const int t = i / E, e = i - t * E;
    double v = 0.0;
    for (int s = 0; s < ksplit; ++s) v += __ldcg(a.sk_part + (((size_t)s * n_tb + tb) * kSkTok + t) * E_T + e);
    if (a.bias) v += (double)a.bias[e];  // the bias joins the f64 sum before the rounding to f32
    const float f = (float)v;
    lg_s[t][e] = f;
    const int tg = t0 + t;
    if (a.logits && tg < a.T) a.logits[(size_t)tg * E + e] = f;
  }
  if (a.gate_vec && a.gate_scale && threadIdx.x < kSkTok) {
    const int t = threadIdx.x, tg = t0 + t;
    double v = 0.0;
    for (int s = 0; s < ksplit; ++s) v += __ldcg(a.sk_gate + ((size_t)s * n_tb + tb) * kSkTok + t);
    if (tg < a.T) a.gate_scale[tg] = (float)(1.0 / (1.0 + exp(-v)));
  }
  __syncthreads();
  {
    const int t = warp, tg = t0 + t;  // one warp per token
    if (tg < a.T) {
      int rc = route_one_warp<(E_T + 31) / 32>(lg_s[t], E, a.k, a.renormalize, lane, idx_s[t], w_s[t], exps_s[warp]);
      if (rc) {
        if (lane == 0) report_error(a.err, rc, 1004);
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
  if (threadIdx.x == 0) a.sk_counters[tb] = 0u;  // ready for the next launch (and for graph replay)
}

template <int E_T>
int launch_one(const RouterArgs& a, cudaStream_t s) {
  const int ksplit = (a.d + kSkSlice - 1) / kSkSlice;
  const int n_tb = (a.T + kSkTok - 1) / kSkTok;
  router_splitk_kernel<E_T><<<dim3(ksplit, n_tb), kSkWarps * 32, 0, s>>>(a, ksplit, n_tb);
  return (int)cudaGetLastError();
}

}  // namespace

// Workspace a layer needs for batches of at most `tokens`: doubles for the partial logits and gate
// dot products, counters (zero-initialised by the caller once).
void router_splitk_workspace(int tokens, int d, int E, size_t* part_doubles, size_t* gate_doubles, size_t* counters) {
  const size_t ksplit = (size_t)(d + kSkSlice - 1) / kSkSlice, n_tb = (size_t)(tokens + kSkTok - 1) / kSkTok;
  const size_t e_t = E <= 8 ? 8 : E <= 16 ? 16 : E <= 32 ? 32 : E <= 64 ? 64 : 128;
  *part_doubles = ksplit * n_tb * kSkTok * e_t;
  *gate_doubles = ksplit * n_tb * kSkTok;
  *counters = n_tb;
}

int launch_router_splitk(const RouterArgs& a, cudaStream_t s) {
  if (a.T <= 0) return ATENIA_OK;
  if (a.k > kMaxK || a.E > 128 || a.d % 16 != 0) return ATENIA_ERR_UNSUPPORTED;
  if (!a.sk_part || !a.sk_gate || !a.sk_counters || a.T > a.sk_tokens) return ATENIA_ERR_STATE;
  int rc;
  if (a.E <= 8) rc = launch_one<8>(a, s);
  else if (a.E <= 16) rc = launch_one<16>(a, s);
  else if (a.E <= 32) rc = launch_one<32>(a, s);
  else if (a.E <= 64) rc = launch_one<64>(a, s);
  else rc = launch_one<128>(a, s);
  count_launch();
  return rc;
}

}  // namespace atenia
