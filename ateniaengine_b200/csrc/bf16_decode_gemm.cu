// Grouped expert GEMM at decode sizes, sm_100a: bf16 weights (groups of at most 128 rows) and INT8
// weights multiplied as integers (calls of at most 128 rows).
//
// At a batch of a few tokens the work is streaming the touched experts' weights once; what decides
// the speed is whether every SM streams the same number of bytes.  The 128-row-tile kernels of
// grouped_gemm.cu give a batch of one token on a Mixtral layer 112 gate/up tiles and 64 down tiles for
// 148 SMs.  This kernel cuts the flattened list of (tile, k-block) pairs into one contiguous span per
// CTA ("stream-K", as w8_gemm.cu does for INT8): partial pieces leave raw f32 accumulators in a
// two-slot-per-CTA workspace and bf16_splitk_reduce_kernel adds the pieces of a tile in CTA order
// (deterministic) before the activation and the store.
//
// The contraction is computed transposed, D[f, t] = sum_k W[f, k] * X[t, k]: 128 weight rows are the
// M side of the MMA, the token tile its N side, so the MMA width follows the row count (N = rows
// rounded up to 16) and the per-lane epilogue handles one output feature.  Both operands come from
// shared memory (bf16 tiles, 128B swizzle, by TMA).
//
//   tile      = up to 128 tokens of one expert x { 128 gate rows + 128 up rows (kSwiGLU) | 256 down rows (kPlain) }
//   k-block   = 64: two 16 KiB weight tiles + one 16 KiB token tile per stage, 4 stages
//   TMEM      = two buffers of two 128-column accumulators: the epilogue of a piece overlaps the
//               main loop of the next
//   warps     : 0 TMA, 1 MMA + TMEM alloc, 4..11 epilogue (two warps per TMEM lane quarter)
// All waits are bounded as in grouped_gemm.cu.
// (A form of this kernel with 256-row token tiles for groups of a few hundred rows -- one tile per expert
// instead of a full and a nearly empty 128-row tile -- was measured on B200 against the 128-row-tile kernel
// of grouped_gemm.cu: Qwen1.5-MoE shape 2048 tokens 0.400 vs 0.416 ms, Mixtral shape 512 tokens 0.603 vs
// 0.640 ms, but Mixtral 1024 tokens 0.993 vs 0.899 ms and DeepSeek-V2-Lite 4096 tokens 0.743 vs 0.649 ms;
// it was removed.)
//
// INT8 form (template parameter I8).  Widening int8 codes to bf16 costs two to three instructions per
// weight, and at decode sizes those instructions, not HBM, set the pace of the widening kernels (w8_gemm.cu,
// decode_gemv.cu: 44 - 52 % of the copy rate).  Here no weight is ever widened: the MMA is
// tcgen05.mma.kind::i8 on the codes as they lie in memory, and the bf16 ACTIVATIONS are turned into
// integers instead -- a handful of rows per call.  quantize_digits_kernel writes every token row as four
// planes of balanced base-128 digits of X = rint(x 2^(26 - e)), e = the row's exponent (|x| < 2^e):
//   x = 2^(e - 26) (d0 + 128 d1 + 128^2 d2 + 128^3 d3),   d_i in [-64, 63]
// (exact for every element within 2^-19 of the row's largest; below that the element is rounded to
// 2^-27 of the largest, far finer than the bf16 product it replaces).  The four planes of a token tile
// are four column blocks of ONE MMA (N = 4 x tokens rounded to 16), the int32 accumulators are exact,
// and the epilogue folds them, v = a0 + 128 (a1 + 128 (a2 + 128 a3)), and multiplies by the weight
// row's scale and the token's 2^(e - 26).  Per k-block of 128 codes a stage holds two 16 KiB weight tiles
// and at most 16 KiB of digits; token tiles are 32 rows.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int DTN = 128;     // token tile (MMA N at most)
constexpr int DROWS = 128;   // weight rows per A tile (MMA M)
constexpr int D_STAGES = 4;
constexpr int D_W_BYTES = DROWS * BK * 2;  // 16 KiB
constexpr int D_X_BYTES = DTN * BK * 2;    // 16 KiB
constexpr int D_STAGE_BYTES = 2 * D_W_BYTES + D_X_BYTES;  // 48 KiB
constexpr int D_THREADS = 384;
constexpr int D_SMEM_BYTES = D_STAGES * D_STAGE_BYTES + 1024 + 256;
constexpr int D_TMEM_COLS = 512;
constexpr int D_SLOT_FLOATS = 2 * DTN * DROWS;  // [accumulator][token][feature]
static_assert(D_SLOT_FLOATS == (int)kW8SplitKSlotFloats, "the layer sizes one workspace for both stream-K kernels");

struct __align__(8) BarriersDec {
  uint64_t full[D_STAGES];   // TMA landed (1 arrival + bytes)
  uint64_t empty[D_STAGES];  // the MMAs that read the stage are done (commit)
  uint64_t acc_full[2];      // all MMAs of the piece done (commit)
  uint64_t acc_empty[2];     // 8 epilogue warps drained the buffer
  uint32_t tmem_base;
  int abort_flag;
};

// Instruction descriptor: D f32, A = B = bf16, K-major, M = 128, N given at run time.
__device__ __forceinline__ uint32_t idesc_dec(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(DROWS >> 4) << 24);
}
// The same for kind::i8: D s32 (format 2), A = B = signed 8-bit (format 1).
__device__ __forceinline__ uint32_t idesc_dec_i8(int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(DROWS >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
constexpr int ITOK = 32;        // INT8 form: token tile (four digit planes = 128 MMA columns)
constexpr int IBK = 128;        // INT8 form: codes per k-block (128 bytes of a row, as for bf16)
constexpr int kDigitPlanes = 4;

// Work of one CTA: whole tiles dealt round-robin, or (stream-K) one contiguous span of the flattened
// (tile, k-block) list.  A span has at most one partial piece at its start (slot 0) and one at its end
// (slot 1).
struct DecPieces {
  bool splitk;
  int num_kb, n_tiles, num_groups, bn_out, tile_rows;
  const int32_t* off;
  TileCursor cur;
  int tile, stride;
  long long g, g0, g_end;
  TileCoord tc;
  int kb0, nkb, slot;  // slot -1: the piece is a whole tile
  int tile_id;         // stream-K: index of the piece's tile in the flattened tile list
  long long span;      // stream-K: k-blocks per CTA

  __device__ void init(bool sk, int num_kb_, int n_tiles_, int num_groups_, int bn_out_, const int32_t* off_,
                       int tile_rows_) {
    splitk = sk;
    tile_rows = tile_rows_;
    num_kb = num_kb_;
    n_tiles = n_tiles_;
    num_groups = num_groups_;
    bn_out = bn_out_;
    off = off_;
    cur.group = 0;
    cur.base = 0;
    if (num_groups > 0) cursor_load(cur, off, tile_rows);
    tile = blockIdx.x;
    stride = gridDim.x;
    g = g0 = g_end = 0;
    tile_id = 0;
    span = 1;
    if (splitk) {
      long long total_tiles = 0;
      for (int gi = 0; gi < num_groups; ++gi)
        total_tiles += (long long)((off[gi + 1] - off[gi] + tile_rows - 1) / tile_rows) * n_tiles;
      const long long total = total_tiles * num_kb;
      span = (total + gridDim.x - 1) / gridDim.x;
      g0 = g = (long long)blockIdx.x * span;
      g_end = g0 + span < total ? g0 + span : total;
    }
  }
  __device__ bool next() {
    if (num_groups <= 0) return false;
    if (!splitk) {
      if (!cursor_seek(cur, tile, n_tiles, num_groups, off, tc, bn_out, tile_rows)) return false;
      tile += stride;
      kb0 = 0;
      nkb = num_kb;
      slot = -1;
      return true;
    }
    if (g >= g_end) return false;
    const int t = (int)(g / num_kb);
    tile_id = t;
    kb0 = (int)(g - (long long)t * num_kb);
    const long long left = g_end - g;
    nkb = (num_kb - kb0) < left ? (num_kb - kb0) : (int)left;
    if (!cursor_seek(cur, t, n_tiles, num_groups, off, tc, bn_out, tile_rows)) return false;
    slot = (nkb == num_kb) ? -1 : (g == g0 ? 0 : 1);
    g += nkb;
    return true;
  }
  __device__ int rows() const {
    const int r = tc.row_end - tc.row0;
    return r > tile_rows ? tile_rows : r;
  }
};

// I8: tmap_x is the digit-plane map (uint8, box {128, 16}; plane p of row r at row p * plane_rows + r),
// tmap_w0 / tmap_w1 are int8 maps with box {128, 128} and the 128-byte swizzle, scale0 / scale1 the
// weight rows' scales per group and tok_scale the token rows' 2^(e - 26).
template <int MODE, bool I8>
__global__ void __launch_bounds__(D_THREADS, 1)
grouped_gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_x, const CUtensorMap* __restrict__ tmap_w0,
                           const CUtensorMap* __restrict__ tmap_w1, const int32_t* __restrict__ group_offsets,
                           int num_groups, int N, int K, __nv_bfloat16* __restrict__ out, DeviceError* err,
                           int splitk, float* __restrict__ ws, const float* const* __restrict__ scale0,
                           const float* const* __restrict__ scale1, const float* __restrict__ tok_scale,
                           int plane_rows, unsigned int* __restrict__ tile_cnt) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int BN_OUT = (MODE == kSwiGLU) ? DROWS : 2 * DROWS;
  constexpr int BKE = I8 ? IBK : BK;      // k elements per k-block
  constexpr int TROWS = I8 ? ITOK : DTN;  // token rows per tile
  constexpr int ACOLS = DTN;              // tensor-memory columns of one accumulator
  constexpr int STAGES = D_STAGES;
  constexpr int STAGE_BYTES = D_STAGE_BYTES;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  BarriersDec* bars = reinterpret_cast<BarriersDec*>(smem_aligned + D_STAGES * D_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BKE - 1) / BKE;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars->acc_full[b]), 1);
      mbar_init(smem_u32(&bars->acc_empty[b]), 8);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&bars->tmem_base)),
                 "r"(D_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  DecPieces it;
  it.init(splitk != 0, num_kb, n_tiles, num_groups, BN_OUT, group_offsets, TROWS);
  const TileCoord& tc = it.tc;

  if (warp == 0) {
    // ================= TMA producer =================
    // All lanes of the warp walk the same piece list.  Lane 0 waits for the stage and arms its barrier;
    // then lane c issues copy c of the stage (0 and 1: the two weight tiles, 2 and up: the token rows), so
    // that the issue latencies of a stage's copies overlap instead of adding up in one thread (a stage of
    // the INT8 form has up to ten copies).  Measured: no different from one issuing thread.
    {
      uint32_t idx = 0;
      int last_group = -1;
      uint32_t armed = 0;
      bool ok = true;
      while (ok && it.next()) {
        const CUtensorMap* m0 = &tmap_w0[tc.group];
        const CUtensorMap* m1 = (MODE == kSwiGLU) ? &tmap_w1[tc.group] : m0;
        if (tc.group != last_group) {
          if (lane == 0) tmap_acquire(m0);
          if (lane == 1) tmap_acquire(m1);
          last_group = tc.group;
        }
        const int n1 = (MODE == kSwiGLU) ? tc.n0 : tc.n0 + DROWS;
        // copies of token rows per stage, and the stage's bytes
        const int tokp = (it.rows() + 15) & ~15;
        const int cpp = tokp / 16;  // INT8: copies per digit plane (16 rows each)
        const int n_x = I8 ? kDigitPlanes * cpp : 1;
        const uint32_t bytes = I8 ? 2 * D_W_BYTES + kDigitPlanes * tokp * 128 : (uint32_t)D_STAGE_BYTES;
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++idx) {
          const int stage = idx % STAGES;
          const uint32_t phase = (idx / STAGES) & 1u;
          int got = 1;
          if (lane == 0) got = mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag) ? 1 : 0;
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) {
            if (lane == 0) {
              report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2600 + stage);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sw = smem_base + stage * STAGE_BYTES;
          if (lane == 0) mbar_expect_tx(full, bytes);
          __syncwarp();
          if (lane == 0) {
            tma_load_2d(sw, m0, full, kb * BKE, tc.n0);
          } else if (lane == 1) {
            tma_load_2d(sw + D_W_BYTES, m1, full, kb * BKE, n1);
          } else if (lane - 2 < n_x) {
            const int c = lane - 2;
            if (I8) {
              // digit plane p, token rows 16 cc .. 16 cc + 15 of the tile: MMA columns p * tokp + 16 cc ...
              const int p = c / cpp, cc = (c - p * cpp) * 16;
              tma_load_2d(sw + 2 * D_W_BYTES + (p * tokp + cc) * 128, &tmap_x, full, kb * BKE,
                          p * plane_rows + tc.row0 + cc);
            } else {
              tma_load_2d(sw + 2 * D_W_BYTES, &tmap_x, full, kb * BKE, tc.row0);
            }
          }
          armed |= 1u << stage;
        }
      }
      if (lane == 0 && *abort_flag) {
        const int stage = idx % STAGES;
        const uint32_t phase = (idx / STAGES) & 1u;
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(smem_u32(&bars->full[s]), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      uint32_t idx = 0;
      int acc = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      while (ok && it.next()) {
        if (!mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase[acc] ^ 1u, abort_flag)) {
          report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2700 + acc);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const int tokp = (it.rows() + 15) & ~15;
        const uint32_t idesc = I8 ? idesc_dec_i8(kDigitPlanes * tokp) : idesc_dec(tokp);
        const uint32_t d0 = tmem_base + acc * 2 * ACOLS, d1 = d0 + ACOLS;
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++idx) {
          const int stage = idx % STAGES;
          const uint32_t phase = (idx / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2710 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sw = smem_base + stage * STAGE_BYTES;
          const uint64_t da0 = make_smem_desc(sw), da1 = make_smem_desc(sw + D_W_BYTES);
          const uint64_t db = make_smem_desc(sw + 2 * D_W_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accum = (kb > it.kb0 || k > 0) ? 1u : 0u;
            // 16 bf16 (32 int8) of K = 32 bytes along a swizzled row = 2 in descriptor address units
            if (I8) {
              tc_mma_i8(d0, da0 + 2 * k, db + 2 * k, idesc, accum);
              tc_mma_i8(d1, da1 + 2 * k, db + 2 * k, idesc, accum);
            } else {
              tc_mma_bf16(d0, da0 + 2 * k, db + 2 * k, idesc, accum);
              tc_mma_bf16(d1, da1 + 2 * k, db + 2 * k, idesc, accum);
            }
          }
          tc_commit(smem_u32(&bars->empty[stage]));
        }
        if (ok) tc_commit(smem_u32(&bars->acc_full[acc]));
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else if (warp >= 4) {
    // ================= epilogue =================
    // Lane f of the two accumulators is output feature n0 + f (first weight tile) / the matching row
    // of the second tile; column t is token row0 + t.  For a fixed token the 32 lanes of a warp write
    // 64 contiguous bytes.
    const int quarter = warp & 3;
    const int f = quarter * 32 + lane;
    const int half = (warp - 4) >> 2;  // which of the two warps of this lane quarter
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    while (it.next()) {
      if (!mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase[acc], abort_flag)) {
        if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2900 + acc);
        *abort_flag = 1;
        break;
      }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int rows = it.rows();
      const uint32_t t0 = tmem_base + (uint32_t(quarter * 32) << 16) + acc * 2 * ACOLS, t1 = t0 + ACOLS;
      if (I8) {
        // INT8 form: column p * tokp + t of an accumulator is digit plane p of token t (int32, exact)
        const int tokp = (rows + 15) & ~15;
        auto fold16 = [&](uint32_t t, int c, float (&v)[16]) {
          uint32_t a[16];
          tc_ld16(t + 3 * tokp + c, a);
          tc_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = (float)(int32_t)a[j];
#pragma unroll
          for (int p = 2; p >= 0; --p) {
            tc_ld16(t + p * tokp + c, a);
            tc_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = fmaf(v[j], 128.0f, (float)(int32_t)a[j]);
          }
        };
        const int n_lo = tc.n0 + f, n_hi = tc.n0 + DROWS + f;
        const bool lo_ok = n_lo < N, hi_ok = (MODE == kSwiGLU) ? lo_ok : n_hi < N;
        float sa = 0.f, sb = 0.f;  // weight-row scales of this lane's two accumulator rows
        if (it.slot < 0) {
          if (lo_ok) sa = scale0[tc.group][n_lo];
          if (MODE == kSwiGLU) {
            if (lo_ok) sb = scale1[tc.group][n_lo];
          } else if (hi_ok) {
            sb = scale0[tc.group][n_hi];
          }
        }
        float* slot = it.slot >= 0 ? ws + ((size_t)blockIdx.x * 2 + it.slot) * D_SLOT_FLOATS : nullptr;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          float va[16], vb[16];
          fold16(t0, c, va);
          fold16(t1, c, vb);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c + j >= rows) continue;
            if (slot) {  // partial piece: folded, unscaled sums, [accumulator][token][feature]
              slot[(size_t)(c + j) * DROWS + f] = va[j];
              slot[(size_t)(DTN + c + j) * DROWS + f] = vb[j];
              continue;
            }
            const float ts = tok_scale[tc.row0 + c + j];
            const float a = va[j] * sa * ts, b = vb[j] * sb * ts;
            if (MODE == kSwiGLU) {
              if (lo_ok) obase[(size_t)(c + j) * N + n_lo] = __float2bfloat16(silu_mul(a, b));
            } else {
              if (lo_ok) obase[(size_t)(c + j) * N + n_lo] = __float2bfloat16(a);
              if (hi_ok) obase[(size_t)(c + j) * N + n_hi] = __float2bfloat16(b);
            }
          }
        }
      } else if (it.slot >= 0) {
        // partial piece: raw accumulators to this CTA's workspace slot, [accumulator][token][feature]
        float* slot = ws + ((size_t)blockIdx.x * 2 + it.slot) * D_SLOT_FLOATS;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t a[16], b[16];
          tc_ld16(t0 + c, a);
          tc_ld16(t1 + c, b);
          tc_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c + j < rows) {
              slot[(size_t)(c + j) * DROWS + f] = __uint_as_float(a[j]);
              slot[(size_t)(DTN + c + j) * DROWS + f] = __uint_as_float(b[j]);
            }
          }
        }
      } else if (MODE == kSwiGLU) {
        const int n = tc.n0 + f;
        const bool n_ok = n < N;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N + n;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t g[16], u[16];
          tc_ld16(t0 + c, g);
          tc_ld16(t1 + c, u);
          tc_ld_wait();
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < rows)
                obase[(size_t)(c + j) * N] = __float2bfloat16(silu_mul(__uint_as_float(g[j]), __uint_as_float(u[j])));
          }
        }
      } else {
        const int n_lo = tc.n0 + f, n_hi = tc.n0 + DROWS + f;
        const bool lo_ok = n_lo < N, hi_ok = n_hi < N;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t a[16], b[16];
          tc_ld16(t0 + c, a);
          tc_ld16(t1 + c, b);
          tc_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c + j < rows) {
              if (lo_ok) obase[(size_t)(c + j) * N + n_lo] = __float2bfloat16(__uint_as_float(a[j]));
              if (hi_ok) obase[(size_t)(c + j) * N + n_hi] = __float2bfloat16(__uint_as_float(b[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
      acc ^= 1;
      // ---- fix-up of a tile that stream-K cut across CTAs, without a second kernel.  Every piece of such
      // a tile is partial and every CTA's warp with this warp's role (lane quarter, token half) has written
      // the same portion of its slot.  A counter per (tile, role) counts those warps; the one that arrives
      // last adds the portions of all pieces in CTA order (fixed, whoever is last) and finishes them as
      // the whole-tile epilogue would.  Nothing waits for anything: a warp that is not last just goes on.
      if (tile_cnt != nullptr && it.slot >= 0) {
        const long long tkb = (long long)it.tile_id * num_kb;
        const int c0 = (int)(tkb / it.span), c1 = (int)((tkb + num_kb - 1) / it.span);
        __threadfence();  // this thread's slot stores, before the count
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          unsigned int* cnt = tile_cnt + (size_t)it.tile_id * 8 + (warp - 4);
          last = atomicAdd(cnt, 1u) == (unsigned)(c1 - c0) ? 1 : 0;
          if (last) *cnt = 0u;  // ready for the next launch (and for graph replay)
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();  // the other pieces' stores, after the count
          const int n_lo = tc.n0 + f, n_hi = tc.n0 + DROWS + f;
          const bool lo_ok = n_lo < N, hi_ok = (MODE == kSwiGLU) ? lo_ok : n_hi < N;
          float sa = 1.f, sb = 1.f;
          if (I8) {
            sa = lo_ok ? scale0[tc.group][n_lo] : 0.f;
            sb = (MODE == kSwiGLU) ? (lo_ok ? scale1[tc.group][n_lo] : 0.f) : (hi_ok ? scale0[tc.group][n_hi] : 0.f);
          }
          __nv_bfloat16* obase = out + (size_t)tc.row0 * N;
#pragma unroll 1
          for (int c = half * 16; c < rows; c += 32) {
            for (int j = 0; j < 16 && c + j < rows; ++j) {
              float a = 0.f, b = 0.f;
              for (int cc = c0; cc <= c1; ++cc) {
                const int sl = (it.tile_id == (int)(((long long)cc * it.span) / num_kb)) ? 0 : 1;
                const float* p = ws + ((size_t)cc * 2 + sl) * D_SLOT_FLOATS;
                a += __ldcg(p + (size_t)(c + j) * DROWS + f);
                b += __ldcg(p + (size_t)(DTN + c + j) * DROWS + f);
              }
              if (I8) {
                const float ts = tok_scale[tc.row0 + c + j];
                a = a * sa * ts;
                b = b * sb * ts;
              }
              if (MODE == kSwiGLU) {
                if (lo_ok) obase[(size_t)(c + j) * N + n_lo] = __float2bfloat16(silu_mul(a, b));
              } else {
                if (lo_ok) obase[(size_t)(c + j) * N + n_lo] = __float2bfloat16(a);
                if (hi_ok) obase[(size_t)(c + j) * N + n_hi] = __float2bfloat16(b);
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(D_TMEM_COLS)
                 : "memory");
  }
}

// Adds the partial pieces of every tile that stream-K cut across CTAs, in CTA order, then applies the
// main kernel's activation and store.  One block per tile; thread (f, y) takes weight row (feature) f and
// every kReduceTokLanes-th token, so that the dependent loads of one thread are few.
constexpr int kReduceTokLanes = 8;
constexpr int kReduceMaxGroups = 256;
template <int MODE, bool I8>
__global__ void __launch_bounds__(DROWS * kReduceTokLanes) decode_splitk_reduce_kernel(const int32_t* __restrict__ group_offsets_g,
                                                                      int num_groups, int N, int K,
                                                                      __nv_bfloat16* __restrict__ out,
                                                                      const float* __restrict__ ws, int num_ctas,
                                                                      const float* const* __restrict__ scale0,
                                                                      const float* const* __restrict__ scale1,
                                                                      const float* __restrict__ tok_scale) {
  constexpr int BN_OUT = (MODE == kSwiGLU) ? DROWS : 2 * DROWS;
  constexpr int BKE = I8 ? IBK : BK;
  constexpr int TROWS = I8 ? ITOK : DTN;
  const int num_kb = (K + BKE - 1) / BKE;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;
  // the group offsets once, side by side, into shared memory: the walks below are chains of dependent reads
  __shared__ int32_t off_s[kReduceMaxGroups + 1];
  const bool in_smem = num_groups <= kReduceMaxGroups;
  if (in_smem) {
    for (int i = threadIdx.y * DROWS + threadIdx.x; i <= num_groups; i += DROWS * kReduceTokLanes)
      off_s[i] = group_offsets_g[i];
    __syncthreads();
  }
  const int32_t* group_offsets = in_smem ? off_s : group_offsets_g;
  long long total_tiles = 0;
  for (int gi = 0; gi < num_groups; ++gi)
    total_tiles += (long long)((group_offsets[gi + 1] - group_offsets[gi] + TROWS - 1) / TROWS) * n_tiles;
  const long long t = blockIdx.x;
  if (t >= total_tiles) return;
  const long long total = total_tiles * num_kb;
  const long long span = (total + num_ctas - 1) / num_ctas;
  const int c0 = (int)((t * num_kb) / span), c1 = (int)(((t + 1) * num_kb - 1) / span);
  if (c0 == c1) return;  // the tile was computed whole by one CTA
  TileCursor cur;
  cur.group = 0;
  cur.base = 0;
  cursor_load(cur, group_offsets, TROWS);
  TileCoord tc;
  if (!cursor_seek(cur, (int)t, n_tiles, num_groups, group_offsets, tc, BN_OUT, TROWS)) return;
  const int f = threadIdx.x;
  int rows = tc.row_end - tc.row0;
  if (rows > TROWS) rows = TROWS;
  const int n_lo = tc.n0 + f, n_hi = tc.n0 + DROWS + f;
  const bool ok_a = n_lo < N, ok_b = (MODE == kSwiGLU) ? ok_a : n_hi < N;
  float sa = 1.f, sb = 1.f;
  if (I8) {
    sa = ok_a ? scale0[tc.group][n_lo] : 0.f;
    sb = (MODE == kSwiGLU) ? (ok_a ? scale1[tc.group][n_lo] : 0.f) : (ok_b ? scale0[tc.group][n_hi] : 0.f);
  }
  for (int tok = threadIdx.y; tok < rows; tok += kReduceTokLanes) {
    float a = 0.f, b = 0.f;
    for (int c = c0; c <= c1; ++c) {
      const int slot = (t == ((long long)c * span) / num_kb) ? 0 : 1;
      const float* p = ws + ((size_t)c * 2 + slot) * D_SLOT_FLOATS;
      a += p[(size_t)tok * DROWS + f];
      b += p[(size_t)(DTN + tok) * DROWS + f];
    }
    if (I8) {
      const float ts = tok_scale[tc.row0 + tok];
      a = a * sa * ts;
      b = b * sb * ts;
    }
    __nv_bfloat16* orow = out + (size_t)(tc.row0 + tok) * N;
    if (MODE == kSwiGLU) {
      if (ok_a) orow[n_lo] = __float2bfloat16(silu_mul(a, b));
    } else {
      if (ok_a) orow[n_lo] = __float2bfloat16(a);
      if (ok_b) orow[n_hi] = __float2bfloat16(b);
    }
  }
}

constexpr int kFixupMaxRows = 32;  // rows (tokens x top-k) up to which the kernel adds split tiles itself

template <int MODE, bool I8>
int launch_dec_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_decode_kernel<MODE, I8>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, D_SMEM_BYTES));
  }
  // stream-K where a workspace slot can hold every piece (bf16: every group fits one 128-token tile;
  // INT8: tiles are 32 tokens) and the tiles that can exist are too few to balance the SMs
  constexpr int BN_OUT = (MODE == kSwiGLU) ? DROWS : 2 * DROWS;
  constexpr int TROWS = I8 ? ITOK : DTN;
  const int n_tiles = (a.N + BN_OUT - 1) / BN_OUT;
  const int active_groups = a.max_rows < a.num_groups ? a.max_rows : a.num_groups;
  const int max_tok_tiles = I8 ? active_groups + a.max_rows / TROWS : active_groups;
  // (up to eight rounds of whole tiles: below that the idle SMs of the last round cost more than the
  // reduce pass -- Mixtral shape, 8 tokens, INT8 gate/up product: 448 tiles on 148 SMs are 3.03 rounds)
  const bool splitk = a.splitk_ws != nullptr && (I8 || a.max_rows <= DTN) && max_tok_tiles * n_tiles < 8 * num_sms;
  // With tile counters the kernel finishes the split tiles itself.  That saves the second launch, and pays
  // for calls of a few rows (Mixtral INT8 shape, 1 token: 0.136 against 0.146 ms per layer); from about a
  // hundred rows on the last warp's serial sum costs what the launch saved, so the reduce kernel stays.
  const bool fixup = splitk && a.splitk_cnt != nullptr && a.max_rows <= kFixupMaxRows &&
                     max_tok_tiles * n_tiles <= kSplitKMaxTiles;
  grouped_gemm_decode_kernel<MODE, I8><<<dim3(num_sms), dim3(D_THREADS), D_SMEM_BYTES, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.err, splitk ? 1 : 0, a.splitk_ws, a.scale0, a.scale1, a.tok_scale, a.plane_rows,
      fixup ? a.splitk_cnt : nullptr);
  int rc = (int)cudaGetLastError();
  if (rc || !splitk || fixup) return rc;
  decode_splitk_reduce_kernel<MODE, I8><<<dim3(max_tok_tiles * n_tiles), dim3(DROWS, kReduceTokLanes), 0, s>>>(
      a.group_offsets, a.num_groups, a.N, a.K, a.out, a.splitk_ws, num_sms, a.scale0, a.scale1, a.tok_scale);
  count_launch();
  return (int)cudaGetLastError();
}

// One block per token row: the row's exponent, then its four digit planes (see the head of this file).
// The row is read once: a thread keeps its (up to kQVecs) 16-byte vectors in registers between the two
// passes; longer rows read the rest again.
constexpr int kQThreads = 1024;
constexpr int kQVecs = 2;  // 8 bf16 each: rows of up to 16 384 elements stay in registers

__device__ __forceinline__ void digits_of_vector(const uint4& q, float mul, int8_t* __restrict__ prow, size_t plane,
                                                 int v) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint32_t d[kDigitPlanes][2] = {};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float xv = (i & 1) ? bf16hi(w[i >> 1]) : bf16lo(w[i >> 1]);
    int X = __float2int_rn(xv * mul);  // |X| <= 2^26
#pragma unroll
    for (int p = 0; p < kDigitPlanes; ++p) {
      const int dg = ((X + 64) & 127) - 64;  // balanced digit in [-64, 63]
      X = (X - dg) >> 7;
      d[p][i >> 2] |= (uint32_t)(dg & 0xff) << (8 * (i & 3));
    }
  }
#pragma unroll
  for (int p = 0; p < kDigitPlanes; ++p)
    *reinterpret_cast<uint2*>(prow + p * plane + (size_t)v * 8) = make_uint2(d[p][0], d[p][1]);
}

__device__ __forceinline__ void amax_of_vector(const uint4& q, float& amax, bool& bad) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = fabsf(bf16lo(w[i])), b = fabsf(bf16hi(w[i]));
    bad = bad || !(a <= 3.0e38f) || !(b <= 3.0e38f);  // inf or NaN
    amax = fmaxf(amax, fmaxf(a, b));
  }
}

__global__ void __launch_bounds__(kQThreads) quantize_digits_kernel(DigitSource src,
                                                                    const int32_t* __restrict__ n_rows_dev, int n_rows,
                                                                    int K, int plane_rows, int8_t* __restrict__ planes,
                                                                    float* __restrict__ tok_scale) {
  const int row = blockIdx.x;
  // rows the dispatch did not place (invalid expert ids) hold nothing: skip them
  const int placed = n_rows_dev ? (*n_rows_dev < n_rows ? *n_rows_dev : n_rows) : n_rows;
  if (row >= placed) return;
  // dispatch row `row` is token perm[row] / k of the caller's batch (gather and digits in one pass)
  const int srow = src.perm ? src.perm[row] / src.k : row;
  if (srow < 0 || srow >= src.n_src_rows) return;
  __shared__ float red[kQThreads / 32];
  __shared__ float mul_s;
  // vector v of the row: eight consecutive elements as bf16 (f32 input is rounded to nearest even first,
  // as the row gather does)
  auto load_vec = [&](int v) -> uint4 {
    if (src.x_is_f32) {
      const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(src.x) + (size_t)srow * K) + 2 * v;
      const float4 a = p[0], b = p[1];
      return make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y), pack_bf16x2(b.z, b.w));
    }
    return reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(src.x) + (size_t)srow * K)[v];
  };
  const int nvec = K / 8;
  uint4 keep[kQVecs];
  float amax = 0.f;
  bool bad = false;
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) {
    const int v = threadIdx.x + j * kQThreads;
    keep[j] = v < nvec ? load_vec(v) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) amax_of_vector(keep[j], amax, bad);
  for (int v = threadIdx.x + kQVecs * kQThreads; v < nvec; v += kQThreads) amax_of_vector(load_vec(v), amax, bad);
  if (bad) amax = __int_as_float(0x7f800000);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float m = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (threadIdx.x == 0) {
      float mul = 0.f, ts = 0.f;
      if (!(m <= 3.0e38f)) {
        ts = __int_as_float(0x7fc00000);  // a non-finite activation makes the token's outputs NaN
      } else if (m > 0.f) {
        int e = ilogbf(m) + 1;  // m < 2^e
        if (e < -100) e = -100;
        mul = ldexpf(1.0f, 26 - e);
        ts = ldexpf(1.0f, e - 26);
      }
      mul_s = mul;
      tok_scale[row] = ts;
    }
  }
  __syncthreads();
  const float mul = mul_s;
  const size_t plane = (size_t)plane_rows * K;
  int8_t* prow = planes + (size_t)row * K;
#pragma unroll
  for (int j = 0; j < kQVecs; ++j) {
    const int v = threadIdx.x + j * kQThreads;
    if (v < nvec) digits_of_vector(keep[j], mul, prow, plane, v);
  }
  for (int v = threadIdx.x + kQVecs * kQThreads; v < nvec; v += kQThreads)
    digits_of_vector(load_vec(v), mul, prow, plane, v);
}

}  // namespace

int launch_grouped_gemm_bf16_decode(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  int rc = a.mode == kSwiGLU ? launch_dec_one<kSwiGLU, false>(a, num_sms, s) : launch_dec_one<kPlain, false>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

int launch_grouped_gemm_w8_i8_decode(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0 || a.max_rows > kI8DecodeMaxRows) return ATENIA_ERR_SHAPE;
  if (!a.scale0 || (a.mode == kSwiGLU && !a.scale1) || !a.tok_scale || a.plane_rows < a.max_rows) return ATENIA_ERR_NULL;
  int rc = a.mode == kSwiGLU ? launch_dec_one<kSwiGLU, true>(a, num_sms, s) : launch_dec_one<kPlain, true>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

int launch_quantize_digits(const DigitSource& src, const int32_t* n_rows_dev, int n_rows, int K, int plane_rows,
                           int8_t* planes, float* tok_scale, cudaStream_t s) {
  if (n_rows <= 0) return ATENIA_OK;
  if (K % 16 != 0 || n_rows > plane_rows || !src.x || (src.perm && src.k < 1)) return ATENIA_ERR_SHAPE;
  quantize_digits_kernel<<<n_rows, kQThreads, 0, s>>>(src, n_rows_dev, n_rows, K, plane_rows, planes, tok_scale);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace atenia
