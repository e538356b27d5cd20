// Grouped expert GEMM for INT8 weights (W8A16) at decode sizes (groups of at most 128 rows), sm_100a:
// weights widened into shared memory, transposed product, stream-K.
//
// At a batch of a few tokens the work is streaming the touched experts' int8 weights once, and the
// widening to bf16 has to keep up with that stream.  The contraction is computed transposed,
// D[f, t] = sum_k W[f, k] * X[t, k]: 128 weight rows are the M side of the MMA, the token tile its N side
// (N = rows rounded up to 16, so the MMA of a k-block is a few dozen cycles and a batch of 8 does not
// pay for 128 columns).  Per k-block the TMA brings two 128-row tiles of codes (16 KiB) and the bf16
// token tile; sixteen warps in two groups, taking alternate k-blocks, widen the codes (exact: |q| <= 127)
// into a 128B-swizzled bf16 tile pair of their group's buffer, which is the MMA's A operand.  The
// shared-memory traffic of a k-block (about 114 KiB for 16 KiB of weights) is what bounds the kernel, at
// roughly four fifths of the HBM rate; the per-row scale multiplies the f32 sums in the epilogue, one
// scalar per lane in this orientation.  As in bf16_decode_gemm.cu the flattened list of (tile, k-block)
// pairs is cut into one contiguous span per CTA when there are too few tiles to balance the SMs
// (stream-K); partial pieces leave raw f32 accumulators in a two-slot-per-CTA workspace and
// w8_decode_splitk_reduce_kernel adds the pieces of a tile in CTA order (deterministic) before scale,
// activation and store.
//
//   tile      = up to 128 tokens of one expert x { 128 gate rows + 128 up rows (kSwiGLU) | 256 down rows (kPlain) }
//   k-block   = 64: two 8 KiB int8 weight tiles + one 16 KiB bf16 token tile per stage, 4 stages;
//               2 buffers of 32 KiB for the widened tile pair (one per widening group)
//   TMEM      = two buffers of two 128-column accumulators: the epilogue of a piece overlaps the
//               main loop of the next
//   warps     : 0 TMA, 1 MMA + TMEM alloc, 4..11 epilogue (two warps per TMEM lane quarter),
//               12..19 and 20..27 the two widening groups
// All waits are bounded as in grouped_gemm.cu.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int DTN = 128;     // token tile (MMA N at most)
constexpr int DROWS = 128;   // weight rows per A tile (MMA M)
constexpr int D_STAGES = 4;
constexpr int D_W_BYTES = DROWS * BK * 2;  // 16 KiB: one widened weight tile
constexpr int D_Q_BYTES = DROWS * BK;      // 8 KiB: one tile of codes
constexpr int D_X_BYTES = DTN * BK * 2;    // 16 KiB
constexpr int D_STAGE_BYTES = 2 * D_Q_BYTES + D_X_BYTES;  // 32 KiB
constexpr int D_CONV = 2;                 // widened tile pairs, one per widening group
constexpr int D_GROUP_WARPS = 8;
constexpr int D_CONV_BYTES = 2 * D_W_BYTES;  // 32 KiB
constexpr int D_CONV_OFF = D_STAGES * D_STAGE_BYTES;
constexpr int D_FIRST_CONV_WARP = 12;
constexpr int D_THREADS = (D_FIRST_CONV_WARP + D_CONV * D_GROUP_WARPS) * 32;  // 896
constexpr int D_SMEM_BYTES = D_CONV_OFF + D_CONV * D_CONV_BYTES + 1024 + 256;
constexpr int D_TMEM_COLS = 512;
constexpr int D_SLOT_FLOATS = 2 * DTN * DROWS;  // [accumulator][token][feature]
static_assert(D_SLOT_FLOATS == (int)kW8SplitKSlotFloats, "the layer sizes one workspace for both stream-K kernels");

struct __align__(8) BarriersDec {
  uint64_t full[D_STAGES];   // TMA landed (1 arrival + bytes)
  uint64_t empty[D_STAGES];  // MMA commit (token tile read) + the 8 warps of one widening group (codes read)
  uint64_t conv_full[D_CONV];   // widened tile pair written (8 warps of the owning group)
  uint64_t conv_empty[D_CONV];  // the MMAs that read it are done (commit)
  uint64_t acc_full[2];      // all MMAs of the piece done (commit)
  uint64_t acc_empty[2];     // 8 epilogue warps drained the buffer
  uint32_t tmem_base;
  int abort_flag;
};

// Instruction descriptor: D f32, A = B = bf16, K-major, M = 128, N given at run time.
__device__ __forceinline__ uint32_t idesc_dec(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(DROWS >> 4) << 24);
}

// Work of one CTA: whole tiles dealt round-robin, or (stream-K) one contiguous span of the flattened
// (tile, k-block) list.  A span has at most one partial piece at its start (slot 0) and one at its end
// (slot 1).
struct DecPieces {
  bool splitk;
  int num_kb, n_tiles, num_groups, bn_out;
  const int32_t* off;
  TileCursor cur;
  int tile, stride;
  long long g, g0, g_end;
  TileCoord tc;
  int kb0, nkb, slot;  // slot -1: the piece is a whole tile

  __device__ void init(bool sk, int num_kb_, int n_tiles_, int num_groups_, int bn_out_, const int32_t* off_) {
    splitk = sk;
    num_kb = num_kb_;
    n_tiles = n_tiles_;
    num_groups = num_groups_;
    bn_out = bn_out_;
    off = off_;
    cur.group = 0;
    cur.base = 0;
    if (num_groups > 0) cursor_load(cur, off);
    tile = blockIdx.x;
    stride = gridDim.x;
    g = g0 = g_end = 0;
    if (splitk) {
      long long total_tiles = 0;
      for (int gi = 0; gi < num_groups; ++gi)
        total_tiles += (long long)((off[gi + 1] - off[gi] + BM - 1) / BM) * n_tiles;
      const long long total = total_tiles * num_kb;
      const long long span = (total + gridDim.x - 1) / gridDim.x;
      g0 = g = (long long)blockIdx.x * span;
      g_end = g0 + span < total ? g0 + span : total;
    }
  }
  __device__ bool next() {
    if (num_groups <= 0) return false;
    if (!splitk) {
      if (!cursor_seek(cur, tile, n_tiles, num_groups, off, tc, bn_out)) return false;
      tile += stride;
      kb0 = 0;
      nkb = num_kb;
      slot = -1;
      return true;
    }
    if (g >= g_end) return false;
    const int t = (int)(g / num_kb);
    kb0 = (int)(g - (long long)t * num_kb);
    const long long left = g_end - g;
    nkb = (num_kb - kb0) < left ? (num_kb - kb0) : (int)left;
    if (!cursor_seek(cur, t, n_tiles, num_groups, off, tc, bn_out)) return false;
    slot = (nkb == num_kb) ? -1 : (g == g0 ? 0 : 1);
    g += nkb;
    return true;
  }
  __device__ int rows() const {
    const int r = tc.row_end - tc.row0;
    return r > DTN ? DTN : r;
  }
};

template <int MODE>
__global__ void __launch_bounds__(D_THREADS, 1)
grouped_gemm_w8_decode_kernel(const __grid_constant__ CUtensorMap tmap_x, const CUtensorMap* __restrict__ tmap_w0,
                              const CUtensorMap* __restrict__ tmap_w1, const int32_t* __restrict__ group_offsets,
                              int num_groups, int N, int K, __nv_bfloat16* __restrict__ out,
                              const float* const* __restrict__ scale0, const float* const* __restrict__ scale1,
                              DeviceError* err, int splitk, float* __restrict__ ws) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int BN_OUT = (MODE == kSwiGLU) ? DROWS : 2 * DROWS;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  BarriersDec* bars = reinterpret_cast<BarriersDec*>(smem_aligned + D_CONV_OFF + D_CONV * D_CONV_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < D_STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1 + D_GROUP_WARPS);
    }
    for (int c = 0; c < D_CONV; ++c) {
      mbar_init(smem_u32(&bars->conv_full[c]), D_GROUP_WARPS);
      mbar_init(smem_u32(&bars->conv_empty[c]), 1);
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
  it.init(splitk != 0, num_kb, n_tiles, num_groups, BN_OUT, group_offsets);
  const TileCoord& tc = it.tc;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      uint32_t idx = 0;
      int last_group = -1;
      uint32_t armed = 0;
      bool ok = true;
      while (ok && it.next()) {
        if (tc.group != last_group) {
          tmap_acquire(&tmap_w0[tc.group]);
          if (MODE == kSwiGLU) tmap_acquire(&tmap_w1[tc.group]);
          last_group = tc.group;
        }
        const CUtensorMap* m0 = &tmap_w0[tc.group];
        const CUtensorMap* m1 = (MODE == kSwiGLU) ? &tmap_w1[tc.group] : m0;
        const int n1 = (MODE == kSwiGLU) ? tc.n0 : tc.n0 + DROWS;
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++idx) {
          const int stage = idx % D_STAGES;
          const uint32_t phase = (idx / D_STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2600 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sw = smem_base + stage * D_STAGE_BYTES;
          mbar_expect_tx(full, D_STAGE_BYTES);
          tma_load_2d(sw, m0, full, kb * BK, tc.n0);
          tma_load_2d(sw + D_Q_BYTES, m1, full, kb * BK, n1);
          tma_load_2d(sw + 2 * D_Q_BYTES, &tmap_x, full, kb * BK, tc.row0);
          armed |= 1u << stage;
        }
      }
      if (*abort_flag) {
        const int stage = idx % D_STAGES;
        const uint32_t phase = (idx / D_STAGES) & 1u;
        for (int s = 0; s < D_STAGES; ++s) {
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
        const uint32_t idesc = idesc_dec((it.rows() + 15) & ~15);
        const uint32_t d0 = tmem_base + acc * 2 * DTN, d1 = d0 + DTN;
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++idx) {
          const int stage = idx % D_STAGES;
          const uint32_t phase = (idx / D_STAGES) & 1u;
          const int cbuf = idx % D_CONV;
          const uint32_t cphase = (idx / D_CONV) & 1u;
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
              !mbar_wait(smem_u32(&bars->conv_full[cbuf]), cphase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2710 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sw = smem_base + stage * D_STAGE_BYTES;
          const uint32_t sc = smem_base + D_CONV_OFF + cbuf * D_CONV_BYTES;
          const uint64_t da0 = make_smem_desc(sc), da1 = make_smem_desc(sc + D_W_BYTES);
          const uint64_t db = make_smem_desc(sw + 2 * D_Q_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accum = (kb > it.kb0 || k > 0) ? 1u : 0u;
            // 16 bf16 of K = 32 bytes along a swizzled row = 2 in descriptor address units
            tc_mma_bf16(d0, da0 + 2 * k, db + 2 * k, idesc, accum);
            tc_mma_bf16(d1, da1 + 2 * k, db + 2 * k, idesc, accum);
          }
          tc_commit(smem_u32(&bars->empty[stage]));
          tc_commit(smem_u32(&bars->conv_empty[cbuf]));
        }
        if (ok) tc_commit(smem_u32(&bars->acc_full[acc]));
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else if (warp >= D_FIRST_CONV_WARP) {
    // ================= int8 -> bf16 widening =================
    // Group g takes the k-blocks with idx % 2 == g and owns widened buffer g.  Per k-block 256 rows x 64
    // codes (two tiles, contiguous in the stage) = 1024 16-byte pieces for the group's 256 threads: thread
    // t takes pieces (row, c) with row = (t >> 2) + 64 i, c = t & 3.  Sixteen codes become two 16-byte
    // pieces of the row's 128-byte bf16 line, stored at the 128B-swizzled position (piece index XOR row
    // mod 8) the MMA descriptor expects; rows 128..255 form the second tile, 16 KiB further on.
    const int ct = (threadIdx.x - D_FIRST_CONV_WARP * 32) % (D_GROUP_WARPS * 32);
    const int grp = (threadIdx.x - D_FIRST_CONV_WARP * 32) / (D_GROUP_WARPS * 32);
    uint32_t idx = 0;
    bool ok = true;
    while (ok && it.next()) {
      for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++idx) {
        if ((int)(idx % D_CONV) != grp) continue;
        const int stage = idx % D_STAGES;
        const uint32_t phase = (idx / D_STAGES) & 1u, cphase = (idx / D_CONV) & 1u;
        if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
            !mbar_wait(smem_u32(&bars->conv_empty[grp]), cphase ^ 1u, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 2800 + warp);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint8_t* q = smem_aligned + stage * D_STAGE_BYTES;
        uint8_t* b = smem_aligned + D_CONV_OFF + grp * D_CONV_BYTES;
        const int c = ct & 3;
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = *reinterpret_cast<const uint4*>(q + ((ct >> 2) + 64 * i) * BK + c * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = (ct >> 2) + 64 * i;
          uint4 o0, o1;
          widen4(v[i].x, o0.x, o0.y);
          widen4(v[i].y, o0.z, o0.w);
          widen4(v[i].z, o1.x, o1.y);
          widen4(v[i].w, o1.z, o1.w);
          uint8_t* line = b + row * 128;  // row 128 starts the second tile: 128 x 128 bytes = D_W_BYTES further
          *reinterpret_cast<uint4*>(line + (((2 * c) ^ (row & 7)) << 4)) = o0;
          *reinterpret_cast<uint4*>(line + (((2 * c + 1) ^ (row & 7)) << 4)) = o1;
        }
        fence_proxy_async();  // generic-proxy writes above must be visible to the MMA's async-proxy reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bars->conv_full[grp]));
          mbar_arrive(smem_u32(&bars->empty[stage]));  // the codes of this stage have been read
        }
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
      const uint32_t t0 = tmem_base + (uint32_t(quarter * 32) << 16) + acc * 2 * DTN, t1 = t0 + DTN;
      if (it.slot >= 0) {
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
        const float sg = n_ok ? scale0[tc.group][n] : 0.f, su = n_ok ? scale1[tc.group][n] : 0.f;
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
                obase[(size_t)(c + j) * N] = __float2bfloat16(silu_mul(__uint_as_float(g[j]) * sg, __uint_as_float(u[j]) * su));
          }
        }
      } else {
        const int n_lo = tc.n0 + f, n_hi = tc.n0 + DROWS + f;
        const bool lo_ok = n_lo < N, hi_ok = n_hi < N;
        const float s_lo = lo_ok ? scale0[tc.group][n_lo] : 0.f, s_hi = hi_ok ? scale0[tc.group][n_hi] : 0.f;
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
              if (lo_ok) obase[(size_t)(c + j) * N + n_lo] = __float2bfloat16(__uint_as_float(a[j]) * s_lo);
              if (hi_ok) obase[(size_t)(c + j) * N + n_hi] = __float2bfloat16(__uint_as_float(b[j]) * s_hi);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
      acc ^= 1;
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
// main kernel's activation and store.  One block per tile, one thread per weight row (feature).
template <int MODE>
__global__ void __launch_bounds__(DROWS) w8_decode_splitk_reduce_kernel(const int32_t* __restrict__ group_offsets,
                                                                  int num_groups, int N, int K,
                                                                  __nv_bfloat16* __restrict__ out,
                                                                  const float* const* __restrict__ scale0,
                                                                  const float* const* __restrict__ scale1,
                                                                  const float* __restrict__ ws, int num_ctas) {
  constexpr int BN_OUT = (MODE == kSwiGLU) ? DROWS : 2 * DROWS;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;
  long long total_tiles = 0;
  for (int gi = 0; gi < num_groups; ++gi)
    total_tiles += (long long)((group_offsets[gi + 1] - group_offsets[gi] + BM - 1) / BM) * n_tiles;
  const long long t = blockIdx.x;
  if (t >= total_tiles) return;
  const long long total = total_tiles * num_kb;
  const long long span = (total + num_ctas - 1) / num_ctas;
  const int c0 = (int)((t * num_kb) / span), c1 = (int)(((t + 1) * num_kb - 1) / span);
  if (c0 == c1) return;  // the tile was computed whole by one CTA
  TileCursor cur;
  cur.group = 0;
  cur.base = 0;
  cursor_load(cur, group_offsets);
  TileCoord tc;
  if (!cursor_seek(cur, (int)t, n_tiles, num_groups, group_offsets, tc, BN_OUT)) return;
  const int f = threadIdx.x;
  int rows = tc.row_end - tc.row0;
  if (rows > DTN) rows = DTN;
  const int n_lo = tc.n0 + f, n_hi = tc.n0 + DROWS + f;
  const bool ok_a = n_lo < N, ok_b = (MODE == kSwiGLU) ? ok_a : n_hi < N;
  const float s_a = ok_a ? scale0[tc.group][n_lo] : 0.f;
  const float s_b = (MODE == kSwiGLU) ? (ok_a ? scale1[tc.group][n_lo] : 0.f) : (ok_b ? scale0[tc.group][n_hi] : 0.f);
  for (int tok = 0; tok < rows; ++tok) {
    float a = 0.f, b = 0.f;
    for (int c = c0; c <= c1; ++c) {
      const int slot = (t == ((long long)c * span) / num_kb) ? 0 : 1;
      const float* p = ws + ((size_t)c * 2 + slot) * D_SLOT_FLOATS;
      a += p[(size_t)tok * DROWS + f];
      b += p[(size_t)(DTN + tok) * DROWS + f];
    }
    __nv_bfloat16* orow = out + (size_t)(tc.row0 + tok) * N;
    if (MODE == kSwiGLU) {
      if (ok_a) orow[n_lo] = __float2bfloat16(silu_mul(a * s_a, b * s_b));
    } else {
      if (ok_a) orow[n_lo] = __float2bfloat16(a * s_a);
      if (ok_b) orow[n_hi] = __float2bfloat16(b * s_b);
    }
  }
}

template <int MODE>
int launch_w8dec_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_w8_decode_kernel<MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, D_SMEM_BYTES));
  }
  // stream-K where every group fits one token tile (one workspace slot holds 128 tokens) and the
  // tiles that can exist are too few to balance the SMs
  constexpr int BN_OUT = (MODE == kSwiGLU) ? DROWS : 2 * DROWS;
  const int n_tiles = (a.N + BN_OUT - 1) / BN_OUT;
  const int active_groups = a.max_rows < a.num_groups ? a.max_rows : a.num_groups;
  const bool splitk = a.splitk_ws != nullptr && a.max_rows <= DTN && active_groups * n_tiles < 4 * num_sms;
  grouped_gemm_w8_decode_kernel<MODE><<<dim3(num_sms), dim3(D_THREADS), D_SMEM_BYTES, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.scale0, a.scale1, a.err, splitk ? 1 : 0, a.splitk_ws);
  int rc = (int)cudaGetLastError();
  if (rc || !splitk) return rc;
  const int max_tiles = a.num_groups * n_tiles;  // every group has at most one token tile here
  w8_decode_splitk_reduce_kernel<MODE><<<dim3(max_tiles), dim3(DROWS), 0, s>>>(a.group_offsets, a.num_groups, a.N, a.K, a.out,
                                                                        a.scale0, a.scale1, a.splitk_ws, num_sms);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

int launch_grouped_gemm_w8_decode(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (!a.scale0 || (a.mode == kSwiGLU && !a.scale1)) return ATENIA_ERR_NULL;
  int rc = a.mode == kSwiGLU ? launch_w8dec_one<kSwiGLU>(a, num_sms, s) : launch_w8dec_one<kPlain>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

}  // namespace atenia
