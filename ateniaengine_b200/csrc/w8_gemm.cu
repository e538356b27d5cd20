// Grouped expert GEMM for INT8 weights (W8A16) on sm_100a: weights as the TMEM-resident operand.
//
// The contraction is computed transposed, D[f, t] = sum_k W[f, k] * X[t, k]: 128 weight rows are
// the M side of the MMA, a tile of up to 128 tokens is the N side.  The int8 weight tile arrives by
// TMA (one byte per weight through HBM, L2 and shared memory), each of 256 threads widens one weight
// row of a k-block to bf16 in registers (exact: |q| <= 127) and stores it with tcgen05.st into
// tensor memory, and tcgen05.mma reads A from tensor memory and B (the bf16 token tile, 128B-swizzled
// by TMA) from shared memory.  The widened weights never touch shared memory, which is the scarce
// resource of this kernel: per k-block the shared-memory traffic is 80 KiB instead of the 128 KiB of
// a widen-into-shared-memory design.  The per-row scale multiplies the f32 accumulator in the
// epilogue ((q*s).x = s*(q.x) exactly); in this orientation it is one scalar per thread.
//
//   tile      = 128 tokens of one expert x { 128 gate rows + 128 up rows (kSwiGLU) | 256 down rows (kPlain) }
//   k-block   = 64: two 8 KiB int8 weight tiles + one 16 KiB bf16 token tile per stage, 6 stages
//   TMEM      = columns [0,128) accumulator 0, [128,256) accumulator 1,
//               [256,512) four stages of the widened weight tiles (2 x 32 columns each)
//   MMA       = M128 x N x K16 with N = the tile's token count rounded up to 16: a decode batch does
//               not pay for 128 columns
//   warps     : 0 TMA, 1 MMA + TMEM alloc, 4..7 widen both weight tiles of the even k-blocks, 8..11 of the
//               odd ones, 12..19 epilogue (two warps per TMEM lane quarter, each taking every other
//               16-token chunk)
//
// The two groups of widening warps take ALTERNATE k-blocks: a warp's chain wait -> ld.shared -> widen ->
// tcgen05.st -> wait::st -> arrive then has two k-block periods to complete, and two k-blocks are in
// flight.  (With every warp serving every k-block, that chain, not HBM, set the k-block period at decode
// sizes, where the MMA of a k-block is a few dozen cycles: measured on B200, a Mixtral-shaped layer at
// 8 / 64 tokens takes 0.309 / 0.531 ms this way against 0.318 / 0.549 ms.)
//
// The accumulator is single-buffered (TMEM is full); the TMA ring and the widening run ahead into the
// next tile while the epilogue drains.  All waits are bounded as in grouped_gemm.cu.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int TN = 128;            // token tile (MMA N, at most)
constexpr int WROWS = 128;         // weight rows per A tile (MMA M)
constexpr int S_STAGES = 6;        // shared-memory ring
constexpr int T_STAGES = 4;        // tensor-memory ring of widened weight tiles
constexpr int WQ_TILE_BYTES = WROWS * BK;      // 8 KiB of int8
constexpr int X_TILE_BYTES = TN * BK * 2;      // 16 KiB of bf16
constexpr int S_STAGE_BYTES = 2 * WQ_TILE_BYTES + X_TILE_BYTES;  // 32 KiB
constexpr int NUM_THREADS_W8 = 640;
constexpr int SMEM_BYTES_W8 = S_STAGES * S_STAGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS_W8 = 512;
constexpr int ACC1_COL = 128;
constexpr int A_RING_COL = 256;
constexpr int A_TILE_COLS = BK / 2;  // 64 bf16 per row = 32 columns of 32 bits

struct __align__(8) BarriersW8 {
  uint64_t full[S_STAGES];    // TMA landed (1 arrival + bytes)
  uint64_t empty[S_STAGES];   // 4 widening warps (one group) read the int8 tiles + MMA commit read the token tile
  uint64_t a_full[T_STAGES];  // widened tiles stored to TMEM (4 widening warps: one group)
  uint64_t a_empty[T_STAGES]; // MMAs that read them are done (commit)
  uint64_t acc_full;          // all MMAs of the tile done (commit)
  uint64_t acc_empty;         // 8 epilogue warps drained the accumulators
  uint32_t tmem_base;
  int abort_flag;
};

// Instruction descriptor: D f32, A = B = bf16, K-major, M = 128, N given at run time.
__device__ __forceinline__ uint32_t idesc_for(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(WROWS >> 4) << 24);
}

// ---- work decomposition ---------------------------------------------------------------------------
// Whole tiles dealt round-robin (large batches), or "stream-K": the flattened list of (tile, k-block)
// pairs is cut into one contiguous span per CTA, so that every SM streams the same number of weight
// bytes even when there are fewer tiles than SMs (decode batches).  A span covers at most one partial
// piece at its start and one at its end; partial pieces leave their raw f32 accumulators in a
// workspace slot (2 per CTA) and a second kernel adds the pieces of a tile in CTA order.
constexpr int SLOT_FLOATS = 2 * TN * WROWS;  // [accumulator][token][feature]

struct PieceIter {
  bool splitk;
  int num_kb, n_tiles, num_groups, bn_out;
  const int32_t* off;
  TileCursor cur;
  int tile, stride;       // round-robin mode
  long long g, g0, g_end; // stream-K mode: flattened k-block range of this CTA
  // current piece
  TileCoord tc;
  int kb0, nkb, slot;     // slot: -1 = the piece is a whole tile, else the workspace slot of this CTA

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
};

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS_W8, 1)
grouped_gemm_w8_tmem_kernel(const __grid_constant__ CUtensorMap tmap_x, const CUtensorMap* __restrict__ tmap_w0,
                            const CUtensorMap* __restrict__ tmap_w1, const int32_t* __restrict__ group_offsets,
                            int num_groups, int N, int K, __nv_bfloat16* __restrict__ out,
                            const float* const* __restrict__ scale0, const float* const* __restrict__ scale1,
                            DeviceError* err, int splitk, float* __restrict__ ws) {
  extern __shared__ uint8_t smem_raw[];
  // kSwiGLU: 128 output columns per tile (gate rows and up rows of the same 128 features);
  // kPlain: 256 output columns per tile (two 128-row halves of W_down).
  constexpr int BN_OUT = (MODE == kSwiGLU) ? WROWS : 2 * WROWS;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  BarriersW8* bars = reinterpret_cast<BarriersW8*>(smem_aligned + S_STAGES * S_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S_STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 5);
    }
    for (int c = 0; c < T_STAGES; ++c) {
      mbar_init(smem_u32(&bars->a_full[c]), 4);
      mbar_init(smem_u32(&bars->a_empty[c]), 1);
    }
    mbar_init(smem_u32(&bars->acc_full), 1);
    mbar_init(smem_u32(&bars->acc_empty), 8);
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS_W8)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  PieceIter it;
  it.init(splitk != 0, num_kb, n_tiles, num_groups, BN_OUT, group_offsets);
  TileCoord& tc = it.tc;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
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
        const int n1 = (MODE == kSwiGLU) ? tc.n0 : tc.n0 + WROWS;
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 600 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sw = smem_base + stage * S_STAGE_BYTES;
          mbar_expect_tx(full, S_STAGE_BYTES);
          tma_load_2d(sw, m0, full, kb * BK, tc.n0);
          tma_load_2d(sw + WQ_TILE_BYTES, m1, full, kb * BK, n1);
          tma_load_2d(sw + 2 * WQ_TILE_BYTES, &tmap_x, full, kb * BK, tc.row0);
          armed |= 1u << stage;
          if (++stage == S_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_flag) {
        for (int s = 0; s < S_STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          uint32_t par = (s < stage) ? phase : (phase ^ 1u);
          for (uint32_t i = 0; i < (1u << 20); ++i)
            if (mbar_try_wait(smem_u32(&bars->full[s]), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      int stage = 0, tstage = 0;
      uint32_t phase = 0, tphase = 0, acc_phase = 0;
      bool ok = true;
      while (ok && it.next()) {
        if (!mbar_wait(smem_u32(&bars->acc_empty), acc_phase ^ 1u, abort_flag)) {
          report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 700);
          *abort_flag = 1;
          break;
        }
        acc_phase ^= 1u;
        tc_fence_after();
        int rows = tc.row_end - tc.row0;
        if (rows > TN) rows = TN;
        const uint32_t idesc = idesc_for((rows + 15) & ~15);
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
              !mbar_wait(smem_u32(&bars->a_full[tstage]), tphase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 710 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t db = make_smem_desc(smem_base + stage * S_STAGE_BYTES + 2 * WQ_TILE_BYTES);
          const uint32_t a0 = tmem_base + A_RING_COL + tstage * 2 * A_TILE_COLS;
          const uint32_t a1 = a0 + A_TILE_COLS;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accum = (kb > it.kb0 || k > 0) ? 1u : 0u;
            // 16 bf16 of K = 8 TMEM columns of the A tile, 32 bytes of the swizzled B row
            tc_mma_bf16_tmem_a(tmem_base, a0 + k * (UMMA_K / 2), db + 2 * k, idesc, accum);
            tc_mma_bf16_tmem_a(tmem_base + ACC1_COL, a1 + k * (UMMA_K / 2), db + 2 * k, idesc, accum);
          }
          tc_commit(smem_u32(&bars->empty[stage]));     // token tile of this stage consumed
          tc_commit(smem_u32(&bars->a_empty[tstage]));  // widened tiles of this TMEM stage consumed
          if (++stage == S_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
          if (++tstage == T_STAGES) {
            tstage = 0;
            tphase ^= 1u;
          }
        }
        if (ok) tc_commit(smem_u32(&bars->acc_full));
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ================= int8 -> bf16 widening into tensor memory =================
    // Group (warp - 4) / 4 takes the k-blocks of its parity and widens both weight tiles of them; warp
    // quarter w % 4 owns TMEM lanes [32q, 32q + 32); a thread widens one row of each tile: 64 int8 =
    // four 16-byte pieces.  The TMA box is 64B-swizzled (piece index XOR (row / 2) mod 4), which makes
    // the 32 row-strided reads of a warp conflict-free.
    const uint32_t group = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int sw = (row >> 1) & 3;
    // The TMEM stores of one k-block stay in flight while this group's next k-block is read and
    // widened; their completion is awaited (and the barriers signalled) just before the next store.
    uint32_t idx = 0;  // k-blocks of this CTA so far, both groups counted
    int pend_stage = -1, pend_tstage = -1;
    bool ok = true;
    auto retire = [&]() {
      if (pend_stage < 0) return;
      tc_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bars->a_full[pend_tstage]));
        mbar_arrive(smem_u32(&bars->empty[pend_stage]));
      }
      pend_stage = -1;
    };
    auto widen_row = [&](const uint8_t* q, uint32_t (&v)[32]) {
      uint4 p[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) p[c] = *reinterpret_cast<const uint4*>(q + ((c ^ sw) << 4));
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        widen4(p[c].x, v[8 * c + 0], v[8 * c + 1]);
        widen4(p[c].y, v[8 * c + 2], v[8 * c + 3]);
        widen4(p[c].z, v[8 * c + 4], v[8 * c + 5]);
        widen4(p[c].w, v[8 * c + 6], v[8 * c + 7]);
      }
    };
    while (ok && it.next()) {
      for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++idx) {
        if ((idx & 1u) != group) continue;
        const int stage = idx % S_STAGES, tstage = idx % T_STAGES;
        const uint32_t phase = (idx / S_STAGES) & 1u, tphase = (idx / T_STAGES) & 1u;
        if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 800 + warp);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint8_t* q0 = smem_aligned + stage * S_STAGE_BYTES + row * BK;
        uint32_t v[32];
        widen_row(q0, v);
        retire();
        if (!mbar_wait(smem_u32(&bars->a_empty[tstage]), tphase ^ 1u, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 820 + warp);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + A_RING_COL + tstage * 2 * A_TILE_COLS;
        tc_st32(taddr, v);
        widen_row(q0 + WQ_TILE_BYTES, v);  // the store above read its registers when it was issued
        tc_st32(taddr + A_TILE_COLS, v);
        pend_stage = stage;
        pend_tstage = tstage;
      }
    }
    retire();
  } else if (warp >= 12) {
    // ================= epilogue =================
    // Lane f of the accumulators is output feature n0 + f (tile 0) / the matching row of tile 1;
    // column t is token row0 + t.  For a fixed token the 32 lanes of a warp write 64 contiguous bytes.
    const int quarter = warp & 3;
    const int f = quarter * 32 + lane;
    const int half = (warp - 12) >> 2;  // which of the two warps of this lane quarter
    uint32_t acc_phase = 0;
    while (it.next()) {
      if (!mbar_wait(smem_u32(&bars->acc_full), acc_phase, abort_flag)) {
        if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 900);
        *abort_flag = 1;
        break;
      }
      acc_phase ^= 1u;
      tc_fence_after();
      int rows = tc.row_end - tc.row0;
      if (rows > TN) rows = TN;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16);
      const float* sc0 = scale0[tc.group];
      if (it.slot >= 0) {
        // partial piece: raw accumulators to this CTA's workspace slot, [accumulator][token][feature]
        float* slot = ws + ((size_t)blockIdx.x * 2 + it.slot) * SLOT_FLOATS;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t a[16], b[16];
          tc_ld16(taddr + c, a);
          tc_ld16(taddr + ACC1_COL + c, b);
          tc_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (c + j < rows) {
              slot[(size_t)(c + j) * WROWS + f] = __uint_as_float(a[j]);
              slot[(size_t)(TN + c + j) * WROWS + f] = __uint_as_float(b[j]);
            }
          }
        }
      } else if (MODE == kSwiGLU) {
        const int n = tc.n0 + f;
        const bool n_ok = n < N;
        const float sg = n_ok ? sc0[n] : 0.f;
        const float su = n_ok ? scale1[tc.group][n] : 0.f;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N + n;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t g[16], u[16];
          tc_ld16(taddr + c, g);
          tc_ld16(taddr + ACC1_COL + c, u);
          tc_ld_wait();
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c + j < rows) {
                const float gv = __uint_as_float(g[j]) * sg, uv = __uint_as_float(u[j]) * su;
                obase[(size_t)(c + j) * N] = __float2bfloat16(silu_mul(gv, uv));
              }
            }
          }
        }
      } else {
        const int n_lo = tc.n0 + f, n_hi = tc.n0 + WROWS + f;
        const bool lo_ok = n_lo < N, hi_ok = n_hi < N;
        const float s_lo = lo_ok ? sc0[n_lo] : 0.f;
        const float s_hi = hi_ok ? sc0[n_hi] : 0.f;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t a[16], b[16];
          tc_ld16(taddr + c, a);
          tc_ld16(taddr + ACC1_COL + c, b);
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
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS_W8)
                 : "memory");
  }
}

// Adds the partial pieces of every tile that stream-K cut across CTAs, in CTA order, and applies the
// same scale / activation / store as the main kernel's epilogue.  One block per tile, one thread per
// weight row (feature).
template <int MODE>
__global__ void __launch_bounds__(WROWS * 8) w8_splitk_reduce_kernel(const int32_t* __restrict__ group_offsets,
                                                                  int num_groups, int N, int K,
                                                                  __nv_bfloat16* __restrict__ out,
                                                                  const float* const* __restrict__ scale0,
                                                                  const float* const* __restrict__ scale1,
                                                                  const float* __restrict__ ws, int num_ctas) {
  constexpr int BN_OUT = (MODE == kSwiGLU) ? WROWS : 2 * WROWS;
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
  if (rows > TN) rows = TN;
  const float* sc0 = scale0[tc.group];
  const int n_lo = tc.n0 + f, n_hi = tc.n0 + WROWS + f;
  float s_a, s_b;
  bool ok_a, ok_b;
  if (MODE == kSwiGLU) {
    ok_a = ok_b = n_lo < N;
    s_a = ok_a ? sc0[n_lo] : 0.f;
    s_b = ok_a ? scale1[tc.group][n_lo] : 0.f;
  } else {
    ok_a = n_lo < N;
    ok_b = n_hi < N;
    s_a = ok_a ? sc0[n_lo] : 0.f;
    s_b = ok_b ? sc0[n_hi] : 0.f;
  }
  // (thread (f, y) takes every blockDim.y-th token: few dependent loads per thread)
  for (int tok = threadIdx.y; tok < rows; tok += blockDim.y) {
    float a = 0.f, b = 0.f;
    for (int c = c0; c <= c1; ++c) {
      const int slot = (t == ((long long)c * span) / num_kb) ? 0 : 1;
      const float* p = ws + ((size_t)c * 2 + slot) * SLOT_FLOATS;
      a += p[(size_t)tok * WROWS + f];
      b += p[(size_t)(TN + tok) * WROWS + f];
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
int launch_w8_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_w8_tmem_kernel<MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_W8));
  }
  // stream-K only where groups fit one token tile (decode: one workspace slot holds 128 tokens) and
  // the tiles that can exist (groups that can have a row x column tiles) are too few to balance SMs
  constexpr int BN_OUT_H = (MODE == kSwiGLU) ? WROWS : 2 * WROWS;
  const int active_groups = a.max_rows < a.num_groups ? a.max_rows : a.num_groups;
  const int tile_bound = active_groups * ((a.N + BN_OUT_H - 1) / BN_OUT_H);
  const bool splitk = a.splitk_ws != nullptr && a.max_rows <= TN && tile_bound < 4 * num_sms;
  grouped_gemm_w8_tmem_kernel<MODE><<<dim3(num_sms), dim3(NUM_THREADS_W8), SMEM_BYTES_W8, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.scale0, a.scale1, a.err, splitk ? 1 : 0, a.splitk_ws);
  int rc = (int)cudaGetLastError();
  if (rc || !splitk) return rc;
  constexpr int BN_OUT = (MODE == kSwiGLU) ? WROWS : 2 * WROWS;
  const int n_tiles = (a.N + BN_OUT - 1) / BN_OUT;
  const int max_tiles = a.num_groups * n_tiles;  // every group has at most one token tile here
  w8_splitk_reduce_kernel<MODE><<<dim3(max_tiles), dim3(WROWS, 8), 0, s>>>(a.group_offsets, a.num_groups, a.N, a.K, a.out,
                                                                         a.scale0, a.scale1, a.splitk_ws, num_sms);
  count_launch();
  return (int)cudaGetLastError();
}

}  // namespace

int launch_grouped_gemm_w8_tmem(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (!a.scale0 || (a.mode == kSwiGLU && !a.scale1)) return ATENIA_ERR_NULL;
  int rc = a.mode == kSwiGLU ? launch_w8_one<kSwiGLU>(a, num_sms, s) : launch_w8_one<kPlain>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

}  // namespace atenia
