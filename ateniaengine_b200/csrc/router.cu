// Router: logits (f64 accumulation) + softmax + top-k with lowest-index tie-break, one launch.
//
// The reference ranks experts by their f32 softmax weight, computed as exp((f64)(v - max)) with the
// subtraction in f32, a sequential f64 sum, a multiply by the f64 reciprocal and a rounding to f32
// (src/moe/dense.rs:172-187); ties go to the lower index (src/moe/sparse.rs:166-175).  Two distinct
// logits can round to one f32 weight, so ranking by logits is not equivalent: the kernel repeats
// the reference's sequence and ranks the rounded weights.  Logits are accumulated in f64 like the
// reference's router matvec (src/moe/dense.rs:97-115, :333), so they round to the same f32 except
// when the f64 sums differ in their last bits across summation orders.
#include "common.cuh"
#include "route_warp.cuh"
#include "v3_route.cuh"

namespace atenia {
namespace {

// softmax + top-k for one token, executed by one thread.  `lg` holds E f32 logits (stride 1).
// Writes k ascending indices and weights.  Returns 0 or a negative status.  `probs` (E floats) may
// alias `lg`: each logit is read before its slot is overwritten.
__device__ int route_one(const float* lg, int E, int k, int renormalize, int32_t* idx_out, float* w_out,
                         float* probs) {
  float mx = -INFINITY;
  bool finite = true;
  for (int e = 0; e < E; ++e) {
    float v = lg[e];
    if (!isfinite(v)) finite = false;
    mx = fmaxf(mx, v);
  }
  if (!finite) return ATENIA_ERR_ROUTING;
  double sum = 0.0;
  for (int e = 0; e < E; ++e) {
    float dl = __fsub_rn(lg[e], mx);
    sum += exp((double)dl);
  }
  double inv = sum > 0.0 ? 1.0 / sum : 0.0;
  for (int e = 0; e < E; ++e) {
    float dl = __fsub_rn(lg[e], mx);
    probs[e] = (float)(exp((double)dl) * inv);
  }
  unsigned long long used[2] = {0ull, 0ull};
  for (int s = 0; s < k; ++s) {
    int best = -1;
    float bw = 0.f;
    for (int e = 0; e < E; ++e) {
      if ((used[e >> 6] >> (e & 63)) & 1ull) continue;
      float w = probs[e];
      if (best < 0 || w > bw) {  // strict >: the lower index keeps a tie
        best = e;
        bw = w;
      }
    }
    used[best >> 6] |= 1ull << (best & 63);
  }
  double ssum = 0.0;
  int m = 0;
  for (int e = 0; e < E; ++e) {
    if ((used[e >> 6] >> (e & 63)) & 1ull) {
      idx_out[m++] = e;
      ssum += (double)probs[e];
    }
  }
  if (!(ssum > 0.0)) return ATENIA_ERR_ROUTING;
  double scale = renormalize ? 1.0 / ssum : 1.0;
  for (int s = 0; s < k; ++s) w_out[s] = (float)((double)probs[idx_out[s]] * scale);
  return 0;
}

// Router kernel.  One CTA (8 warps) handles TOK tokens.
//   * per chunk of KC values of k, the CTA stages x[TOK, KC] as f64 ([k][token]: one 16-byte load
//     gives two tokens at one k) and W_router[E, KC] transposed as f32 ([k][expert]) in shared memory,
//     so global memory is read with full sectors and every operand of the inner loop is a
//     conflict-free shared-memory read;
//   * warp w owns the k-slice [w*KC/8, (w+1)*KC/8) of the chunk; lane l owns experts (l % EL) + EL*j
//     and the contiguous sub-slice l / EL of its warp's slice; it accumulates TOK tokens x EPL experts
//     in f64;
//   * the sub-slices are folded with shuffles inside a warp and through shared memory across warps
//     (one warp after the other, a fixed order);
//   * the warps then route the tokens (route_one_warp).
// E_T: experts rounded up to a power of two in {8,16,32,64,128}.
constexpr int kRWarps = 8;

template <int E_T, int TOK>
struct RouterSmem {
  static constexpr int KC = E_T >= 128 ? 64 : 128;
  static constexpr int kXs = KC * TOK * 8;
  static constexpr int kWs = KC * E_T * 4;
  static constexpr int kAcc = TOK * (E_T + 1) * 8;
  static constexpr int kLg = TOK * E_T * 4;
  static constexpr int kExps = TOK * E_T * 8;
  static constexpr int kGate = kRWarps * TOK * 8;
  static constexpr int kSel = TOK * kMaxK * 8;
  static constexpr int kLoop = kXs + kWs;
  static constexpr int kTail = kAcc + kLg + kExps + kGate + kSel;
  static constexpr int kBytes = kLoop > kTail ? kLoop : kTail;
};

template <int E_T, int TOK>
__global__ void __launch_bounds__(kRWarps * 32) router_kernel(RouterArgs a) {
  using SM = RouterSmem<E_T, TOK>;
  constexpr int KC = SM::KC;
  constexpr int EL = E_T < 32 ? E_T : 32;
  constexpr int KS = 32 / EL;
  constexpr int EPL = E_T / EL;
  constexpr int SLICE = KC / kRWarps;  // k values per warp per chunk
  constexpr int KPL = SLICE / KS;      // k values per lane per chunk
  static_assert(KPL >= 1, "chunk too small for this expert count");
  __shared__ __align__(16) unsigned char smem[SM::kBytes];
  // main-loop view
  double (*xs)[TOK] = reinterpret_cast<double (*)[TOK]>(smem);
  float (*ws)[E_T] = reinterpret_cast<float (*)[E_T]>(smem + SM::kXs);
  // tail view (after the last __syncthreads of the loop)
  double (*acc_s)[E_T + 1] = reinterpret_cast<double (*)[E_T + 1]>(smem);
  float (*lg_s)[E_T] = reinterpret_cast<float (*)[E_T]>(smem + SM::kAcc);
  double (*exps_s)[E_T] = reinterpret_cast<double (*)[E_T]>(smem + SM::kAcc + SM::kLg);
  double (*gate_s)[TOK] = reinterpret_cast<double (*)[TOK]>(smem + SM::kAcc + SM::kLg + SM::kExps);
  int32_t (*idx_s)[kMaxK] = reinterpret_cast<int32_t (*)[kMaxK]>(smem + SM::kAcc + SM::kLg + SM::kExps + SM::kGate);
  float (*w_s)[kMaxK] = reinterpret_cast<float (*)[kMaxK]>(smem + SM::kAcc + SM::kLg + SM::kExps + SM::kGate +
                                                          TOK * kMaxK * 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TOK;
  const int e_lane = lane % EL;
  const int ks = lane / EL;
  const int d = a.d, E = a.E;

  double acc[TOK][EPL];
#pragma unroll
  for (int t = 0; t < TOK; ++t)
#pragma unroll
    for (int j = 0; j < EPL; ++j) acc[t][j] = 0.0;
  double gacc = 0.0;  // lane t (< TOK) of every warp accumulates the gate dot product of token t

  // Global loads of chunk i+1 are issued before the arithmetic of chunk i and land in registers;
  // they are converted and written to shared memory at the top of the next iteration.
  constexpr int XV = (TOK * (KC / 8) + kRWarps * 32 - 1) / (kRWarps * 32);   // 16-byte x loads per thread
  constexpr int WV = (E_T * (KC / 4) + kRWarps * 32 - 1) / (kRWarps * 32);   // float4 W loads per thread
  uint4 xq[XV][2];  // bf16 input uses [.][0] only; f32 input uses both halves
  float4 wq[WV];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int r = 0; r < XV; ++r) {
      const int i = threadIdx.x + r * kRWarps * 32;
      const int g = i / TOK, t = i - g * TOK;
      const int kk = k0 + g * 8, tg = t0 + t;
      xq[r][0] = make_uint4(0, 0, 0, 0);
      xq[r][1] = make_uint4(0, 0, 0, 0);
      if (i < TOK * (KC / 8) && tg < a.T && kk < d) {  // d is a multiple of 16: a group of 8 is all in or out
        if (a.x_is_f32) {
          const uint4* p = reinterpret_cast<const uint4*>(static_cast<const float*>(a.x) + (size_t)tg * d + kk);
          xq[r][0] = p[0];
          xq[r][1] = p[1];
        } else {
          xq[r][0] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.x) + (size_t)tg * d + kk);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < WV; ++r) {
      const int i = threadIdx.x + r * kRWarps * 32;
      const int g = i / E_T, e = i - g * E_T;
      const int kk = k0 + g * 4;
      wq[r] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < E_T * (KC / 4) && e < E && kk < d)
        wq[r] = __ldg(reinterpret_cast<const float4*>(a.w_router + (size_t)e * d + kk));
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < d; k0 += KC) {
    __syncthreads();
    // x as f64, [k][token]: neighbouring threads hold neighbouring tokens, so the stores fall in
    // distinct banks
#pragma unroll
    for (int r = 0; r < XV; ++r) {
      const int i = threadIdx.x + r * kRWarps * 32;
      if (i < TOK * (KC / 8)) {
        const int g = i / TOK, t = i - g * TOK;
        float v[8];
        if (a.x_is_f32) {
          v[0] = __uint_as_float(xq[r][0].x); v[1] = __uint_as_float(xq[r][0].y);
          v[2] = __uint_as_float(xq[r][0].z); v[3] = __uint_as_float(xq[r][0].w);
          v[4] = __uint_as_float(xq[r][1].x); v[5] = __uint_as_float(xq[r][1].y);
          v[6] = __uint_as_float(xq[r][1].z); v[7] = __uint_as_float(xq[r][1].w);
        } else {
          const uint4 u = xq[r][0];
          v[0] = bf16lo(u.x); v[1] = bf16hi(u.x); v[2] = bf16lo(u.y); v[3] = bf16hi(u.y);
          v[4] = bf16lo(u.z); v[5] = bf16hi(u.z); v[6] = bf16lo(u.w); v[7] = bf16hi(u.w);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) xs[g * 8 + j][t] = (double)v[j];
      }
    }
    // W transposed, [k][expert]: neighbouring threads hold neighbouring experts
#pragma unroll
    for (int r = 0; r < WV; ++r) {
      const int i = threadIdx.x + r * kRWarps * 32;
      if (i < E_T * (KC / 4)) {
        const int g = i / E_T, e = i - g * E_T;
        ws[g * 4 + 0][e] = wq[r].x;
        ws[g * 4 + 1][e] = wq[r].y;
        ws[g * 4 + 2][e] = wq[r].z;
        ws[g * 4 + 3][e] = wq[r].w;
      }
    }
    __syncthreads();
    if (k0 + KC < d) fetch(k0 + KC);
    const int kbase = warp * SLICE + ks * KPL;  // within the chunk; rows past d hold zeros
#pragma unroll 4
    for (int c = 0; c < KPL; ++c) {
      const int kc = kbase + c;
      double w[EPL];
#pragma unroll
      for (int j = 0; j < EPL; ++j) w[j] = (double)ws[kc][e_lane + EL * j];
      const double2* xr = reinterpret_cast<const double2*>(&xs[kc][0]);
#pragma unroll
      for (int t2 = 0; t2 < TOK / 2; ++t2) {
        const double2 xv = xr[t2];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          acc[2 * t2][j] = fma(w[j], xv.x, acc[2 * t2][j]);
          acc[2 * t2 + 1][j] = fma(w[j], xv.y, acc[2 * t2 + 1][j]);
        }
      }
    }
    if (a.gate_vec && lane < TOK) {
      for (int c = 0; c < SLICE; ++c) {
        const int kc = warp * SLICE + c;
        if (k0 + kc < d) gacc = fma((double)__ldg(a.gate_vec + k0 + kc), xs[kc][lane], gacc);
      }
    }
  }
  // fold the k sub-slices inside the warp
#pragma unroll
  for (int t = 0; t < TOK; ++t) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      double v = acc[t][j];
#pragma unroll
      for (int o = EL; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[t][j] = v;
    }
  }
  __syncthreads();  // the loop's shared-memory view is dead from here on
  // fold the warps, one after the other
  for (int w = 0; w < kRWarps; ++w) {
    if (warp == w && ks == 0) {
#pragma unroll
      for (int t = 0; t < TOK; ++t)
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          const int e = e_lane + EL * j;
          if (e < E) acc_s[t][e] = (w == 0 ? 0.0 : acc_s[t][e]) + acc[t][j];
        }
    }
    __syncthreads();
  }
  if (a.gate_vec && lane < TOK) gate_s[warp][lane] = gacc;
  // logits: bias joins the f64 sum before the rounding to f32
  for (int i = threadIdx.x; i < TOK * E; i += blockDim.x) {
    const int t = i / E, e = i - t * E;
    double v = acc_s[t][e];
    if (a.bias) v += (double)a.bias[e];
    const float f = (float)v;
    lg_s[t][e] = f;
    const int tg = t0 + t;
    if (a.logits && tg < a.T) a.logits[(size_t)tg * E + e] = f;
  }
  __syncthreads();
  if (a.gate_vec && a.gate_scale && threadIdx.x < TOK) {
    const int t = threadIdx.x, tg = t0 + t;
    double v = 0.0;
    for (int w = 0; w < kRWarps; ++w) v += gate_s[w][t];
    if (tg < a.T) a.gate_scale[tg] = (float)(1.0 / (1.0 + exp(-v)));
  }
  for (int t = warp; t < TOK; t += kRWarps) {
    const int tg = t0 + t;
    if (tg >= a.T) continue;
    int rc = route_one_warp<(E_T + 31) / 32>(lg_s[t], E, a.k, a.renormalize, lane, idx_s[t], w_s[t], exps_s[t]);
    if (rc) {
      if (lane == 0) report_error(a.err, rc, 1000);
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

__global__ void route_from_logits_kernel(const float* __restrict__ logits, int T, int E, int k, int renormalize,
                                         int32_t* __restrict__ topk_idx, float* __restrict__ topk_w,
                                         DeviceError* err) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  int32_t idx[kMaxK];
  float w[kMaxK];
  float probs[128];
  int rc = route_one(logits + (size_t)t * E, E, k, renormalize, idx, w, probs);
  if (rc) {
    report_error(err, rc, 1001);
    for (int s = 0; s < k; ++s) {
      idx[s] = s;
      w[s] = 0.f;
    }
  }
  for (int s = 0; s < k; ++s) {
    topk_idx[(size_t)t * k + s] = idx[s];
    topk_w[(size_t)t * k + s] = w[s];
  }
}

__global__ void __launch_bounds__(128) v3_route_kernel(const float* __restrict__ logits,
                                                        const float* __restrict__ e_score_bias, int T,
                                                        V3RouteParams p, int32_t* __restrict__ topk_idx,
                                                        float* __restrict__ topk_w, DeviceError* err) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  double scores[kV3MaxExperts], choice[kV3MaxExperts];
  int32_t idx[kV3MaxTopK];
  float w[kV3MaxTopK];
  const int rc = v3_route_one(logits + (size_t)t * p.n, e_score_bias, p, idx, w, scores, choice);
  if (rc) {
    report_error(err, ATENIA_ERR_ROUTING, 1002);
    for (int s = 0; s < p.top_k; ++s) {  // keep downstream kernels in bounds
      idx[s] = s;
      w[s] = 0.f;
    }
  }
  for (int s = 0; s < p.top_k; ++s) {
    topk_idx[(size_t)t * p.top_k + s] = idx[s];
    topk_w[(size_t)t * p.top_k + s] = w[s];
  }
}

}  // namespace

int launch_v3_route(const float* logits, const float* e_score_bias, int T, int E, int k, int n_group, int topk_group,
                    int norm_topk_prob, float scaling, int32_t* topk_idx, float* topk_w, DeviceError* err,
                    cudaStream_t s) {
  if (T <= 0) return ATENIA_OK;
  V3RouteParams p{E, k, n_group, topk_group, norm_topk_prob, (double)scaling};
  if (v3_validate(p) != 0) return ATENIA_ERR_SHAPE;
  v3_route_kernel<<<(T + 127) / 128, 128, 0, s>>>(logits, e_score_bias, T, p, topk_idx, topk_w, err);
  count_launch();
  return (int)cudaGetLastError();
}

int launch_router(const RouterArgs& a, cudaStream_t s) {
  if (a.T <= 0) return ATENIA_OK;
  if (a.k > kMaxK || a.E > 128) return ATENIA_ERR_UNSUPPORTED;
  // variant -1: choose by size (see atenia_moe_create)
  if ((a.variant == 2 || a.variant == -1) && a.T <= a.sk_tokens && a.sk_part) return launch_router_splitk(a, s);
  if (a.variant == 1 || (a.variant == -1 && a.d % 16 == 0)) return launch_router_dmma(a, s);
  dim3 block(kRWarps * 32);
  // more tokens per CTA for many experts: the router matrix is re-read once per CTA
  if (a.E <= 8) router_kernel<8, 8><<<(a.T + 7) / 8, block, 0, s>>>(a);
  else if (a.E <= 16) router_kernel<16, 8><<<(a.T + 7) / 8, block, 0, s>>>(a);
  else if (a.E <= 32) router_kernel<32, 8><<<(a.T + 7) / 8, block, 0, s>>>(a);
  else if (a.E <= 64) router_kernel<64, 16><<<(a.T + 15) / 16, block, 0, s>>>(a);
  else router_kernel<128, 16><<<(a.T + 15) / 16, block, 0, s>>>(a);
  count_launch();
  return (int)cudaGetLastError();
}

int launch_route_from_logits(const float* logits, int T, int E, int k, int renormalize, int32_t* topk_idx,
                             float* topk_w, DeviceError* err, cudaStream_t s) {
  if (T <= 0) return ATENIA_OK;
  if (k > kMaxK || E > 128) return ATENIA_ERR_UNSUPPORTED;
  route_from_logits_kernel<<<(T + 127) / 128, 128, 0, s>>>(logits, T, E, k, renormalize, topk_idx, topk_w, err);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace atenia
