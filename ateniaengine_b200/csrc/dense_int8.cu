// Dense W8A16 weight quantiser and its materialising dequant: the [K, N] row-major layout with one
// scale per (group of consecutive rows, column) that the reference uses for non-MoE linear weights
// (src/tensor/quantizer.rs:67-118 per channel, :176-246 per group; src/cuda/int8_to_bf16.cu:24-40,
// :99-117).  The MoE tiers use the per-row layout of combine.cu instead.
//
// All three passes are streaming, HBM-bound work:
//   amax      read K*N*4 bytes; a block covers 128 columns x up to 256 rows of one group, reduces its
//             8 row lanes in shared memory and merges with atomicMax on the bit pattern (non-negative
//             floats order like unsigned integers, so the result does not depend on scheduling)
//   finalize  scale = max(amax / 127, 1e-12), in place
//   quantize  read K*N*4, write K*N bytes: q = clamp(round_half_away(w / scale), -127, 127), NaN -> 0
//   dequant   read K*N, write K*N*2 bytes: bf16 = high half of (float)q * scale (truncation, as the
//             reference's kernel does)
#include "common.cuh"

namespace atenia {
namespace {

constexpr int COLS_PER_BLOCK = 128;  // 32 threads x 4 columns
constexpr int ROW_LANES = 8;
constexpr int ROWS_PER_BLOCK = 256;

struct Cols4 {
  float v[4];
};

// Four consecutive columns of row r starting at c0; columns >= N read as 0.
__device__ __forceinline__ Cols4 load_cols4(const float* __restrict__ w, int64_t r, int64_t c0, int64_t N, bool vec) {
  Cols4 o;
  if (vec) {
    const float4 f = *reinterpret_cast<const float4*>(w + r * N + c0);
    o.v[0] = f.x; o.v[1] = f.y; o.v[2] = f.z; o.v[3] = f.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) o.v[j] = (c0 + j < N) ? w[r * N + c0 + j] : 0.f;
  }
  return o;
}

__global__ void __launch_bounds__(256) amax_kernel(const float* __restrict__ w, int64_t K, int64_t N, int64_t G,
                                                    int64_t strips, int64_t chunks_per_group, int vec,
                                                    unsigned int* __restrict__ amax_bits) {
  __shared__ float red[ROW_LANES][COLS_PER_BLOCK];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t strip = blockIdx.x % strips, y = blockIdx.x / strips;
  const int64_t g = y / chunks_per_group, ch = y % chunks_per_group;
  const int64_t lo = g * G + ch * ROWS_PER_BLOCK;
  int64_t hi = lo + ROWS_PER_BLOCK;
  if (hi > (g + 1) * G) hi = (g + 1) * G;
  if (hi > K) hi = K;
  const int64_t c0 = strip * COLS_PER_BLOCK + tx * 4;
  float m[4] = {0.f, 0.f, 0.f, 0.f};
  if (c0 < N) {
    for (int64_t r = lo + ty; r < hi; r += ROW_LANES) {
      const Cols4 x = load_cols4(w, r, c0, N, vec != 0);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = fabsf(x.v[j]);
        if (a > m[j]) m[j] = a;  // a NaN never compares greater: skipped, as in the reference
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) red[ty][tx * 4 + j] = m[j];
  __syncthreads();
  if (threadIdx.x < COLS_PER_BLOCK) {
    const int64_t c = strip * COLS_PER_BLOCK + threadIdx.x;
    if (c < N && lo < hi) {
      float a = red[0][threadIdx.x];
#pragma unroll
      for (int l = 1; l < ROW_LANES; ++l) a = fmaxf(a, red[l][threadIdx.x]);
      if (a > 0.f) atomicMax(&amax_bits[g * N + c], __float_as_uint(a));
    }
  }
}

__global__ void finalize_scales_kernel(float* __restrict__ scales, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i < n; i += (int64_t)gridDim.x * blockDim.x) scales[i] = fmaxf(__fdiv_rn(scales[i], 127.0f), 1e-12f);
}

__device__ __forceinline__ int quantize_one(float w, float s) {
  float v = roundf(__fdiv_rn(w, s));  // roundf: halves away from zero, like Rust's f32::round
  if (v != v) return 0;               // Rust's `as i32` sends NaN to 0
  v = fminf(fmaxf(v, -127.0f), 127.0f);
  return (int)v;
}

__global__ void __launch_bounds__(256) quantize_kernel(const float* __restrict__ w, const float* __restrict__ scales,
                                                        int64_t K, int64_t N, int64_t G, int vec,
                                                        int8_t* __restrict__ q) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    const int64_t n4 = K * N / 4;
    for (; i < n4; i += stride) {
      const int64_t e = i * 4, r = e / N, c = e % N;
      const float4 x = *reinterpret_cast<const float4*>(w + e);
      const float4 s = *reinterpret_cast<const float4*>(scales + (r / G) * N + c);
      const uint32_t b0 = (uint32_t)quantize_one(x.x, s.x) & 0xffu, b1 = (uint32_t)quantize_one(x.y, s.y) & 0xffu,
                     b2 = (uint32_t)quantize_one(x.z, s.z) & 0xffu, b3 = (uint32_t)quantize_one(x.w, s.w) & 0xffu;
      *reinterpret_cast<uint32_t*>(q + e) = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
    }
  } else {
    const int64_t n = K * N;
    for (; i < n; i += stride) {
      const int64_t r = i / N, c = i % N;
      q[i] = (int8_t)quantize_one(w[i], scales[(r / G) * N + c]);
    }
  }
}

__device__ __forceinline__ uint32_t trunc_bf16(int q, float s) {
  return __float_as_uint(__fmul_rn((float)q, s)) >> 16;
}

__global__ void __launch_bounds__(256) dequant_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                                       int64_t K, int64_t N, int64_t G, int vec,
                                                       uint16_t* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    const int64_t n8 = K * N / 8;
    for (; i < n8; i += stride) {
      const int64_t e = i * 8, r = e / N, c = e % N;
      const uint2 p = *reinterpret_cast<const uint2*>(q + e);
      const float* srow = scales + (r / G) * N + c;
      const float4 s0 = *reinterpret_cast<const float4*>(srow), s1 = *reinterpret_cast<const float4*>(srow + 4);
      const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      uint32_t h[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t word = j < 4 ? p.x : p.y;
        h[j] = trunc_bf16((int)(int8_t)((word >> (8 * (j & 3))) & 0xffu), s[j]);
      }
      *reinterpret_cast<uint4*>(out + e) =
          make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
    }
  } else {
    const int64_t n = K * N;
    for (; i < n; i += stride) {
      const int64_t r = i / N, c = i % N;
      out[i] = (uint16_t)trunc_bf16((int)q[i], scales[(r / G) * N + c]);
    }
  }
}

inline unsigned grid_for(int64_t work_items) {
  const int64_t blocks = (work_items + 255) / 256;
  const int64_t cap = 148LL * 32;  // enough blocks in flight to cover HBM latency; the loops stride
  return (unsigned)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace atenia

extern "C" {

int atenia_quantize_per_group_i8(const float* w, int64_t K, int64_t N, int64_t group_size, int8_t* q, float* scales,
                                 void* stream) {
  using namespace atenia;
  if (K < 0 || N < 0 || group_size < 0) return ATENIA_ERR_SHAPE;
  if (K == 0 || N == 0) return ATENIA_OK;
  if (!w || !q || !scales) return ATENIA_ERR_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t G = (group_size == 0 || group_size > K) ? K : group_size;
  const int64_t groups = (K + G - 1) / G;
  const int64_t strips = (N + COLS_PER_BLOCK - 1) / COLS_PER_BLOCK;
  const int64_t cpg = (G + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
  const int64_t blocks = strips * groups * cpg;
  if (blocks > 0x7fffffffLL || groups * N > 0x7fffffffLL * 4) return ATENIA_ERR_SHAPE;
  ATENIA_CUDA_TRY(cudaMemsetAsync(scales, 0, (size_t)(groups * N) * sizeof(float), s));
  const int vec_w = (N % 4 == 0 && aligned16(w)) ? 1 : 0;
  amax_kernel<<<(unsigned)blocks, 256, 0, s>>>(w, K, N, G, strips, cpg, vec_w, reinterpret_cast<unsigned int*>(scales));
  count_launch();
  ATENIA_CUDA_TRY(cudaGetLastError());
  finalize_scales_kernel<<<grid_for(groups * N), 256, 0, s>>>(scales, groups * N);
  count_launch();
  ATENIA_CUDA_TRY(cudaGetLastError());
  const int vec_q = (vec_w && aligned16(scales) && (reinterpret_cast<uintptr_t>(q) & 3u) == 0) ? 1 : 0;
  quantize_kernel<<<grid_for(vec_q ? K * N / 4 : K * N), 256, 0, s>>>(w, scales, K, N, G, vec_q, q);
  count_launch();
  return (int)cudaGetLastError();
}

int atenia_int8_to_bf16_per_group(const int8_t* q, const float* scales, int64_t K, int64_t N, int64_t group_size,
                                  uint16_t* out_bf16, void* stream) {
  using namespace atenia;
  if (K < 0 || N < 0 || group_size < 0) return ATENIA_ERR_SHAPE;
  if (K == 0 || N == 0) return ATENIA_OK;
  if (!q || !scales || !out_bf16) return ATENIA_ERR_NULL;
  const int64_t G = (group_size == 0 || group_size > K) ? K : group_size;
  const int vec = (N % 8 == 0 && aligned16(out_bf16) && aligned16(scales) && (reinterpret_cast<uintptr_t>(q) & 7u) == 0)
                      ? 1
                      : 0;
  dequant_kernel<<<grid_for(vec ? K * N / 8 : K * N), 256, 0, static_cast<cudaStream_t>(stream)>>>(q, scales, K, N, G,
                                                                                                      vec, out_bf16);
  count_launch();
  return (int)cudaGetLastError();
}

}  // extern "C"
