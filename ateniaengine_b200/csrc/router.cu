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

namespace atenia {
namespace {

constexpr int kTokPerWarp = 8;
constexpr int kWarps = 4;
constexpr int kTokPerBlock = kTokPerWarp * kWarps;  // 32
constexpr int kChunk = 64;                          // k elements staged per step
constexpr int kMaxK = 8;

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

// E_T: experts rounded up to a power of two in {8,16,32,64,128}.
// Lane l of a warp owns experts (l % EL) + EL*j, j < EPL, and the k-slice l / EL of KS slices.
template <int E_T>
__global__ void __launch_bounds__(kWarps * 32) router_kernel(RouterArgs a) {
  constexpr int EL = E_T < 32 ? E_T : 32;
  constexpr int KS = 32 / EL;
  constexpr int EPL = E_T / EL;
  __shared__ double xs[kTokPerBlock][kChunk + 1];  // +1: the token-major reads below stay conflict-light
  __shared__ float lg_s[kTokPerBlock][E_T];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t_block = blockIdx.x * kTokPerBlock;
  const int t_warp = t_block + warp * kTokPerWarp;
  const int e_lane = lane % EL;
  const int ks = lane / EL;
  const int d = a.d, E = a.E;

  double acc[kTokPerWarp][EPL];
#pragma unroll
  for (int t = 0; t < kTokPerWarp; ++t)
#pragma unroll
    for (int j = 0; j < EPL; ++j) acc[t][j] = 0.0;
  double gacc[kTokPerWarp];
#pragma unroll
  for (int t = 0; t < kTokPerWarp; ++t) gacc[t] = 0.0;

  for (int k0 = 0; k0 < d; k0 += kChunk) {
    const int kc = min(kChunk, d - k0);
    __syncthreads();
    // stage x[t_block .. +32, k0 .. +kc] as f64
    for (int i = threadIdx.x; i < kTokPerBlock * kChunk; i += blockDim.x) {
      int t = i / kChunk, c = i - t * kChunk;
      double v = 0.0;
      int tg = t_block + t;
      if (tg < a.T && c < kc) {
        size_t off = (size_t)tg * d + k0 + c;
        v = a.x_is_f32 ? (double)static_cast<const float*>(a.x)[off]
                       : (double)__bfloat162float(static_cast<const __nv_bfloat16*>(a.x)[off]);
      }
      xs[t][c] = v;
    }
    __syncthreads();
    // this lane's k values: c = ks, ks + KS, ...
    for (int c = ks; c < kc; c += KS) {
      double w[EPL];
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        int e = e_lane + EL * j;
        w[j] = e < E ? (double)__ldg(a.w_router + (size_t)e * d + k0 + c) : 0.0;
      }
#pragma unroll
      for (int t = 0; t < kTokPerWarp; ++t) {
        double xv = xs[warp * kTokPerWarp + t][c];
#pragma unroll
        for (int j = 0; j < EPL; ++j) acc[t][j] = fma(w[j], xv, acc[t][j]);
      }
    }
    if (a.gate_vec) {
      for (int c = lane; c < kc; c += 32) {
        double gv = (double)__ldg(a.gate_vec + k0 + c);
#pragma unroll
        for (int t = 0; t < kTokPerWarp; ++t) gacc[t] = fma(gv, xs[warp * kTokPerWarp + t][c], gacc[t]);
      }
    }
  }
  // reduce the k-slices (lanes with equal e_lane)
#pragma unroll
  for (int t = 0; t < kTokPerWarp; ++t) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      double v = acc[t][j];
#pragma unroll
      for (int o = EL; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[t][j] = v;
    }
    if (a.gate_vec) {
      double v = gacc[t];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      gacc[t] = v;
    }
  }
  if (ks == 0) {
#pragma unroll
    for (int t = 0; t < kTokPerWarp; ++t)
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        int e = e_lane + EL * j;
        if (e < E) {
          double v = acc[t][j];
          if (a.bias) v += (double)a.bias[e];
          lg_s[warp * kTokPerWarp + t][e] = (float)v;
        }
      }
  }
  if (a.gate_vec && a.gate_scale && lane < kTokPerWarp) {
    // every lane holds all eight sums after the butterfly; lane t writes token t
    double v = 0.0;
#pragma unroll
    for (int t = 0; t < kTokPerWarp; ++t)
      if (lane == t) v = gacc[t];
    int tg = t_warp + lane;
    if (tg < a.T) a.gate_scale[tg] = (float)(1.0 / (1.0 + exp(-v)));
  }
  __syncthreads();
  if (threadIdx.x < kTokPerBlock) {
    int tg = t_block + threadIdx.x;
    if (tg < a.T) {
      int32_t idx[kMaxK];
      float w[kMaxK];
      if (a.logits)
        for (int e = 0; e < E; ++e) a.logits[(size_t)tg * E + e] = lg_s[threadIdx.x][e];
      int rc = route_one(lg_s[threadIdx.x], E, a.k, a.renormalize, idx, w, lg_s[threadIdx.x]);
      if (rc) {
        report_error(a.err, rc, 1000);
        for (int s = 0; s < a.k; ++s) {  // keep downstream kernels in bounds
          idx[s] = s;
          w[s] = 0.f;
        }
      }
      for (int s = 0; s < a.k; ++s) {
        a.topk_idx[(size_t)tg * a.k + s] = idx[s];
        a.topk_w[(size_t)tg * a.k + s] = w[s];
      }
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

}  // namespace

int launch_router(const RouterArgs& a, cudaStream_t s) {
  if (a.T <= 0) return ATENIA_OK;
  if (a.k > kMaxK || a.E > 128) return ATENIA_ERR_UNSUPPORTED;
  dim3 grid((a.T + kTokPerBlock - 1) / kTokPerBlock), block(kWarps * 32);
  if (a.E <= 8) router_kernel<8><<<grid, block, 0, s>>>(a);
  else if (a.E <= 16) router_kernel<16><<<grid, block, 0, s>>>(a);
  else if (a.E <= 32) router_kernel<32><<<grid, block, 0, s>>>(a);
  else if (a.E <= 64) router_kernel<64><<<grid, block, 0, s>>>(a);
  else router_kernel<128><<<grid, block, 0, s>>>(a);
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
