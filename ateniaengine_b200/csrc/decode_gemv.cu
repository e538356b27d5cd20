// Expert products for one or two rows (decode at batch 1): a CUDA-core matrix-vector kernel.
//
// With a row or two in the whole call the work is reading the touched experts' weights once:
// 2 F d + d F weights per expert for a few flops each.  A tensor-core tile of 128 weight rows spends
// its time on staging (and, for INT8, on the widening chain) rather than on the stream; here every
// warp streams whole weight rows with 16-byte loads -- per lane 32 bytes of each of four rows (two of
// each matrix) per step, the next step's vectors requested before the current ones are multiplied --
// and multiplies them with the group's rows as f32.  No shared memory, no barriers: the kernel is bound
// by HBM (bytes in flight per SM: 2 blocks x 256 lanes x 128 bytes, all the time).  INT8 codes become f32 exactly with one byte permute and one
// subtraction (0x4B0000uu is 2^23 + u for the biased code u = q + 128), and the per-row scale
// multiplies the finished sum ((q s) . x = s (q . x)).
//
//   grid   = (ceil(N / 16), groups); a block of 8 warps, each warp two output features
//   kSwiGLU: out[r, n] = silu(s0[n] (W0[n, :] . x[r, :])) * (s1[n] (W1[n, :] . x[r, :]))
//   kPlain:  out[r, n] = s0[n] (W0[n, :] . x[r, :])
// f32 accumulation over k in a fixed order (lane-strided partial sums, then a shuffle tree).
#include "common.cuh"

namespace atenia {
namespace {

constexpr int kGvWarps = 8;
constexpr int kGvRowsPerWarp = 2;
constexpr int kGvRowsPerBlock = kGvWarps * kGvRowsPerWarp;  // 16 output features
constexpr int kGvMaxRows = 4;                               // token rows per call (kernel forms for 2 and 4)

// sixteen weights of one lane as f32
__device__ __forceinline__ void unpack16_i8(const uint4& v, float (&f)[16]) {
  const uint32_t w[4] = {v.x ^ 0x80808080u, v.y ^ 0x80808080u, v.z ^ 0x80808080u, v.w ^ 0x80808080u};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bytes {u, 00, 00, 4B}: the f32 2^23 + u; minus 2^23 + 128 gives the code q = u - 128 exactly
    f[4 * i + 0] = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7540)) - 8388736.0f;
    f[4 * i + 1] = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7541)) - 8388736.0f;
    f[4 * i + 2] = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7542)) - 8388736.0f;
    f[4 * i + 3] = __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7543)) - 8388736.0f;
  }
}
__device__ __forceinline__ void unpack8_bf16(const uint4& v, float* f) {
  f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}

// A lane's share of one step: U units of 16 consecutive k per weight row (INT8: two units = 32 bytes,
// bf16: one unit = 32 bytes), for NM matrices x kGvRowsPerWarp output features.
template <int NM, bool W8>
struct GvStep {
  static constexpr int U = W8 ? 2 : 1;
  static constexpr int V = W8 ? 1 : 2;  // 16-byte vectors per unit
  uint4 q[U][NM][kGvRowsPerWarp][V];
};

template <int MODE, bool W8, int MAXR>
__global__ void __launch_bounds__(kGvWarps * 32, MAXR <= 2 ? 2 : 1) grouped_gemv_kernel(GroupedGemmCheckArgs a) {
  constexpr int NM = (MODE == kSwiGLU) ? 2 : 1;  // matrices
  using Step = GvStep<NM, W8>;
  constexpr int CH = 16 * Step::U;               // k per lane and step
  const int g = blockIdx.y;
  const int r0 = a.group_offsets[g];
  int R = a.group_offsets[g + 1] - r0;
  if (R <= 0) return;
  if (R > MAXR) R = MAXR;  // the launcher only takes calls of at most MAXR rows in all
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_base = blockIdx.x * kGvRowsPerBlock + warp * kGvRowsPerWarp;
  if (n_base >= a.N) return;
  const int K = a.K;
  const size_t esz = W8 ? 1 : 2;
  const uint8_t* wrow[NM][kGvRowsPerWarp];
#pragma unroll
  for (int j = 0; j < kGvRowsPerWarp; ++j) {
    const int n = n_base + j < a.N ? n_base + j : a.N - 1;
    wrow[0][j] = static_cast<const uint8_t*>(a.b0[g]) + (size_t)n * K * esz;
    if (NM == 2) wrow[NM - 1][j] = static_cast<const uint8_t*>(a.b1[g]) + (size_t)n * K * esz;
  }

  float acc[NM][kGvRowsPerWarp][MAXR];
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int j = 0; j < kGvRowsPerWarp; ++j)
#pragma unroll
      for (int r = 0; r < MAXR; ++r) acc[m][j][r] = 0.f;

  // all weight vectors of a step are requested before any is used; K is a multiple of 16, so a unit
  // is all inside or all outside
  auto load = [&](Step& st, int k) {
#pragma unroll
    for (int u = 0; u < Step::U; ++u)
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int j = 0; j < kGvRowsPerWarp; ++j) {
          const int ku = k + 16 * u;
          const uint4* p = reinterpret_cast<const uint4*>(wrow[m][j] + (size_t)ku * esz);
#pragma unroll
          for (int v = 0; v < Step::V; ++v) st.q[u][m][j][v] = ku < K ? p[v] : make_uint4(0, 0, 0, 0);
        }
  };
  auto compute = [&](const Step& st, int k) {
#pragma unroll
    for (int u = 0; u < Step::U; ++u) {
      const int ku = k + 16 * u;
      if (ku >= K) break;
      // rows two at a time (a decode call rarely has more than two per expert): their 16 k-values as f32
#pragma unroll
      for (int rp = 0; rp < MAXR; rp += 2) {
        if (rp >= R) break;
        float xf[2][16];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (rp + q < R) {
            const uint4* p = reinterpret_cast<const uint4*>(a.a + (size_t)(r0 + rp + q) * K + ku);
            const uint4 x0 = __ldg(p), x1 = __ldg(p + 1);
            unpack8_bf16(x0, xf[q]);
            unpack8_bf16(x1, xf[q] + 8);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) xf[q][i] = 0.f;
          }
        }
#pragma unroll
        for (int m = 0; m < NM; ++m)
#pragma unroll
          for (int j = 0; j < kGvRowsPerWarp; ++j) {
            float wf[16];
            if (W8) {
              unpack16_i8(st.q[u][m][j][0], wf);
            } else {
              unpack8_bf16(st.q[u][m][j][0], wf);
              unpack8_bf16(st.q[u][m][j][Step::V - 1], wf + 8);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              acc[m][j][rp] = fmaf(wf[i], xf[0][i], acc[m][j][rp]);
              acc[m][j][rp + 1] = fmaf(wf[i], xf[1][i], acc[m][j][rp + 1]);
            }
          }
      }
    }
  };

  // two steps in flight: the vectors of the next step are requested before the current one is multiplied
  constexpr int STRIDE = 32 * CH;  // k per warp and step
  Step s0, s1;
  int k = lane * CH;
  if (k < K) load(s0, k);
  for (; k < K; k += 2 * STRIDE) {
    const bool more1 = k + STRIDE < K;
    if (more1) load(s1, k + STRIDE);
    compute(s0, k);
    if (more1) {
      if (k + 2 * STRIDE < K) load(s0, k + 2 * STRIDE);
      compute(s1, k + STRIDE);
    }
  }
  // fold the lanes (fixed tree)
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int j = 0; j < kGvRowsPerWarp; ++j)
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        float v = acc[m][j][r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[m][j][r] = v;
      }
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < kGvRowsPerWarp; ++j) {
      const int n = n_base + j;
      if (n >= a.N) continue;
      const float s0f = a.scale0 ? a.scale0[g][n] : 1.0f;
      const float s1f = (NM == 2 && a.scale1) ? a.scale1[g][n] : 1.0f;
#pragma unroll
      for (int r = 0; r < MAXR; ++r) {
        if (r >= R) continue;
        float v;
        if (MODE == kSwiGLU) {
          const float gt = acc[0][j][r] * s0f, up = acc[NM - 1][j][r] * s1f;
          v = __fdividef(gt * up, 1.0f + __expf(-gt));
        } else {
          v = acc[0][j][r] * s0f;
        }
        a.out[(size_t)(r0 + r) * a.N + n] = __float2bfloat16(v);
      }
    }
  }
}

template <int MODE, bool W8>
void launch_gv(const GroupedGemmCheckArgs& a, dim3 grid, dim3 block, cudaStream_t s) {
  if (a.max_rows <= 2) grouped_gemv_kernel<MODE, W8, 2><<<grid, block, 0, s>>>(a);
  else grouped_gemv_kernel<MODE, W8, 4><<<grid, block, 0, s>>>(a);
}

}  // namespace

// Same arguments as the CUDA-core checking contraction (raw matrix pointers per group); the call must
// have at most kGvMaxRows rows in total (a.max_rows), so that every group has at most that many.  The
// layer sends calls of at most kGemvMaxRows = 2 rows here: measured on B200 (Mixtral shape, one token)
// bf16 0.189 -> 0.183 ms, INT8 0.174 -> 0.166 ms, a DeepSeek-shaped layer with its shared expert
// 0.182 -> 0.156 ms; with four rows the tensor-core decode kernels are as fast or faster.
int launch_grouped_gemv(const GroupedGemmCheckArgs& a, cudaStream_t s) {
  if (a.num_groups <= 0 || a.max_rows <= 0) return ATENIA_OK;
  if (a.max_rows > kGvMaxRows || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (a.b_is_int8 && (!a.scale0 || (a.mode == kSwiGLU && !a.scale1))) return ATENIA_ERR_NULL;
  const dim3 grid((a.N + kGvRowsPerBlock - 1) / kGvRowsPerBlock, a.num_groups), block(kGvWarps * 32);
  if (a.mode == kSwiGLU) {
    if (a.b_is_int8) launch_gv<kSwiGLU, true>(a, grid, block, s);
    else launch_gv<kSwiGLU, false>(a, grid, block, s);
  } else {
    if (a.b_is_int8) launch_gv<kPlain, true>(a, grid, block, s);
    else launch_gv<kPlain, false>(a, grid, block, s);
  }
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace atenia
