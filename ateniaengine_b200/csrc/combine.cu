// Combine: gate-weighted sum of a token's expert outputs back in token order, plus the shared expert.
//
// The reference accumulates out[d] += w * y_e[d] over the selected experts in ascending expert order
// with an f32 multiply followed by an f32 add (src/moe/sparse.rs:227-233), then adds scale * shared
// (src/moe/layer.rs:415-429).  The kernel gathers each token's k rows from the dispatch-ordered
// buffer in slot order (slots are ascending experts) and repeats that arithmetic, so the result does
// not depend on scheduling: no atomics.
//
// Also here: the small elementwise kernels of the library (int8 per-row quantiser, f32 to bf16 conversion).
#include "common.cuh"

namespace atenia {
namespace {

// One block per token, one 16-byte vector of the row per thread and step.  K is the top-k count (a
// compile-time bound so that the k row loads of a vector are all issued before the first is used);
// the arithmetic order does not depend on it.
template <int K>
__global__ void __launch_bounds__(256) combine_kernel(CombineArgs a) {
  const int t = blockIdx.x;
  const int nvec = a.d / 8;
  int rows[K];
  float w[K];
#pragma unroll
  for (int s = 0; s < K; ++s) {
    rows[s] = s < a.k ? a.inv_perm[(size_t)t * a.k + s] : -1;
    w[s] = s < a.k ? a.topk_w[(size_t)t * a.k + s] : 0.f;
  }
  const float scale = a.gate_scale ? a.gate_scale[t] : 1.0f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 y[K];
#pragma unroll
    for (int s = 0; s < K; ++s)
      if (rows[s] >= 0) y[s] = *reinterpret_cast<const uint4*>(a.y_rows + (size_t)rows[s] * a.d + v * 8);
    uint4 ysh = make_uint4(0, 0, 0, 0);
    if (a.y_shared) ysh = *reinterpret_cast<const uint4*>(a.y_shared + (size_t)t * a.d + v * 8);
    float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0;
    if (a.residual) {
      const float4* r = reinterpret_cast<const float4*>(a.residual + (size_t)t * a.d + v * 8);
      r0 = r[0];
      r1 = r[1];
    }
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int s = 0; s < K; ++s) {
      if (rows[s] < 0) continue;  // slot past k, or an entry without a row (invalid expert id, reported by the dispatch)
      const uint32_t p[4] = {y[s].x, y[s].y, y[s].z, y[s].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(w[s], bf16lo(p[j])));
        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(w[s], bf16hi(p[j])));
      }
    }
    if (a.y_shared) {
      const uint32_t p[4] = {ysh.x, ysh.y, ysh.z, ysh.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(scale, bf16lo(p[j])));
        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(scale, bf16hi(p[j])));
      }
    }
    if (a.residual) {
      acc[0] = __fadd_rn(acc[0], r0.x); acc[1] = __fadd_rn(acc[1], r0.y);
      acc[2] = __fadd_rn(acc[2], r0.z); acc[3] = __fadd_rn(acc[3], r0.w);
      acc[4] = __fadd_rn(acc[4], r1.x); acc[5] = __fadd_rn(acc[5], r1.y);
      acc[6] = __fadd_rn(acc[6], r1.z); acc[7] = __fadd_rn(acc[7], r1.w);
    }
    if (a.out_is_f32) {
      float4* o = reinterpret_cast<float4*>(static_cast<float*>(a.out) + (size_t)t * a.d + v * 8);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      uint4* o = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + (size_t)t * a.d + v * 8);
      *o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                      pack_bf16x2(acc[6], acc[7]));
    }
  }
}

// One block per row: scale = max|row| / 127 (1 for a zero row), q = clamp(round_half_away(w * (1/scale))).
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ w, int64_t cols,
                                                             int8_t* __restrict__ q, float* __restrict__ scales) {
  __shared__ float red[8];
  __shared__ float s_scale;
  const int64_t r = blockIdx.x;
  const float* row = w + r * cols;
  float amax = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) amax = fmaxf(amax, fabsf(row[c]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    float sc = m > 0.f ? __fdiv_rn(m, 127.0f) : 1.0f;
    s_scale = sc;
    scales[r] = sc;
  }
  __syncthreads();
  const float inv = __fdiv_rn(1.0f, s_scale);
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = roundf(__fmul_rn(row[c], inv));  // roundf: halves away from zero, like Rust's f32::round
    v = fminf(fmaxf(v, -127.0f), 127.0f);
    q[r * cols + c] = (int8_t)v;
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = __float2bfloat16(src[i]);
}

}  // namespace

int launch_combine(const CombineArgs& a, cudaStream_t s) {
  if (a.T <= 0) return ATENIA_OK;
  // d / 8 vectors per token: narrow rows take narrower blocks
  const int nvec = a.d / 8;
  const int threads = nvec >= 256 ? 256 : nvec >= 128 ? 128 : 64;
  if (a.k <= 2) combine_kernel<2><<<a.T, threads, 0, s>>>(a);
  else if (a.k <= 4) combine_kernel<4><<<a.T, threads, 0, s>>>(a);
  else if (a.k <= 6) combine_kernel<6><<<a.T, threads, 0, s>>>(a);
  else combine_kernel<8><<<a.T, threads, 0, s>>>(a);
  count_launch();
  return (int)cudaGetLastError();
}

__global__ void set_pair_kernel(int32_t* p, int32_t a, int32_t b) {
  p[0] = a;
  p[1] = b;
}

int launch_set_pair(int32_t* p, int32_t a, int32_t b, cudaStream_t s) {
  set_pair_kernel<<<1, 1, 0, s>>>(p, a, b);
  count_launch();
  return (int)cudaGetLastError();
}

int launch_f32_to_bf16(const float* src, __nv_bfloat16* dst, int64_t n, cudaStream_t s) {
  if (n <= 0) return ATENIA_OK;
  int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  f32_to_bf16_kernel<<<blocks, 256, 0, s>>>(src, dst, n);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace atenia

extern "C" int atenia_quantize_per_row_i8(const float* w, int64_t rows, int64_t cols, int8_t* q, float* scales,
                                          void* stream) {
  if (!w || !q || !scales) return ATENIA_ERR_NULL;
  if (rows < 0 || cols <= 0 || rows > 0x7fffffff) return ATENIA_ERR_SHAPE;
  if (rows == 0) return ATENIA_OK;
  atenia::quantize_rows_kernel<<<(unsigned)rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, cols, q, scales);
  atenia::count_launch();
  return (int)cudaGetLastError();
}
