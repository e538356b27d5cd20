// Grouped expert GEMM for INT8 weights (W8A16) at large batches: one widened weight tile per k-block
// serves up to 192 tokens.
//
// Same transposed contraction as w8_gemm.cu (D[f, t] = sum_k W[f, k] * X[t, k], weights widened in
// registers and stored to tensor memory, tokens from shared memory), re-balanced for groups of
// hundreds of rows, where the cost of widening per MMA cycle decides the speed:
//   * a k-block carries ONE 128-row weight tile (not a gate tile and an up tile) and up to 192 token
//     columns, so 8 KiB of codes are widened per 384 MMA cycles instead of 16 KiB per 512;
//   * gate and up rows of the same features share the tile: TMEM lanes 32q + l hold gate feature
//     n0 + 16q + l for l < 16 and up feature n0 + 16q + (l - 16) otherwise, so the SwiGLU partner of a
//     lane is lane ^ 16 of the same warp and the epilogue pairs them with one shuffle;
//   * two groups of four widening warps take alternate k-blocks, so the chain
//     wait -> ld.shared -> widen -> tcgen05.st -> wait::st -> arrive of one k-block overlaps the
//     next k-block's;
//   * the accumulator is double-buffered (2 x 192 columns), the epilogue of a tile overlaps the
//     main loop of the next.
//
//   tile      = up to 192 tokens of one expert x { 64 features: 64 gate + 64 up rows (kSwiGLU) |
//               128 rows of W_down (kPlain) }
//   k-block   = 64: two 64-row int8 boxes (8 KiB, 64B swizzle) + up to three 64-row bf16 token boxes
//               (24 KiB, 128B swizzle) per stage, 6 stages
//   TMEM      = columns [0,192) accumulator 0, [192,384) accumulator 1, [384,512) four stages of the
//               widened weight tile (32 columns each)
//   MMA       = M128 x N x K16, A from tensor memory, N = the tile's token count rounded up to 16
//   warps     : 0 TMA, 1 MMA + TMEM alloc, 4..7 widen even k-blocks, 8..11 widen odd k-blocks,
//               12..19 epilogue (two warps per TMEM lane quarter, alternate 16-token chunks)
// All waits are bounded as in grouped_gemm.cu.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int WTN = 192;                 // token tile (MMA N at most)
constexpr int WBOX = 64;                 // rows per TMA box, weights and tokens
constexpr int W_S_STAGES = 6;            // shared-memory ring
constexpr int W_T_STAGES = 4;            // tensor-memory ring of widened weight tiles
constexpr int W_WQ_BYTES = 128 * BK;     // 8 KiB of int8: two boxes
constexpr int W_BOX_X_BYTES = WBOX * BK * 2;  // 8 KiB of bf16 per token box
constexpr int W_X_BYTES = WTN * BK * 2;  // 24 KiB
constexpr int W_STAGE_BYTES = W_WQ_BYTES + W_X_BYTES;  // 32 KiB
constexpr int W_THREADS = 640;
constexpr int W_SMEM_BYTES = W_S_STAGES * W_STAGE_BYTES + 1024 + 256;
constexpr int W_TMEM_COLS = 512;
constexpr int W_RING_COL = 2 * WTN;      // 384
constexpr int W_A_COLS = BK / 2;         // 64 bf16 per row = 32 columns of 32 bits
static_assert(W_RING_COL + W_T_STAGES * W_A_COLS <= W_TMEM_COLS, "tensor memory layout");

struct __align__(8) BarriersWide {
  uint64_t full[W_S_STAGES];     // TMA landed (1 arrival + bytes)
  uint64_t empty[W_S_STAGES];    // 4 widening warps read the int8 tile + MMA commit read the token tile
  uint64_t a_full[W_T_STAGES];   // widened tile stored to TMEM (4 widening warps)
  uint64_t a_empty[W_T_STAGES];  // the MMAs that read it are done (commit)
  uint64_t acc_full[2];          // all MMAs of the tile done (commit)
  uint64_t acc_empty[2];         // 8 epilogue warps drained the accumulator
  uint32_t tmem_base;
  int abort_flag;
};

// Instruction descriptor: D f32, A = B = bf16, K-major, M = 128, N given at run time.
__device__ __forceinline__ uint32_t idesc_wide(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24);
}

// Every role walks the same tile list: tile i of this CTA is blockIdx.x + i * gridDim.x.
struct TileWalk {
  TileCursor cur;
  TileCoord tc;
  int tile, n_tiles, num_groups, bn_out;
  const int32_t* off;
  __device__ void init(int n_tiles_, int num_groups_, int bn_out_, const int32_t* off_) {
    n_tiles = n_tiles_;
    num_groups = num_groups_;
    bn_out = bn_out_;
    off = off_;
    cur.group = 0;
    cur.base = 0;
    if (num_groups > 0) cursor_load(cur, off, WTN);
    tile = blockIdx.x;
  }
  __device__ bool next() {
    if (num_groups <= 0) return false;
    if (!cursor_seek(cur, tile, n_tiles, num_groups, off, tc, bn_out, WTN)) return false;
    tile += gridDim.x;
    return true;
  }
  __device__ int rows() const {
    const int r = tc.row_end - tc.row0;
    return r > WTN ? WTN : r;
  }
};

template <int MODE>
__global__ void __launch_bounds__(W_THREADS, 1)
grouped_gemm_w8_wide_kernel(const __grid_constant__ CUtensorMap tmap_x, const CUtensorMap* __restrict__ tmap_w0,
                            const CUtensorMap* __restrict__ tmap_w1, const int32_t* __restrict__ group_offsets,
                            int num_groups, int N, int K, __nv_bfloat16* __restrict__ out,
                            const float* const* __restrict__ scale0, const float* const* __restrict__ scale1,
                            DeviceError* err) {
  extern __shared__ uint8_t smem_raw[];
  // kSwiGLU: 64 output features per tile (64 gate rows + 64 up rows); kPlain: 128 output rows.
  constexpr int BN_OUT = (MODE == kSwiGLU) ? 64 : 128;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  BarriersWide* bars = reinterpret_cast<BarriersWide*>(smem_aligned + W_S_STAGES * W_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < W_S_STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 5);
    }
    for (int c = 0; c < W_T_STAGES; ++c) {
      mbar_init(smem_u32(&bars->a_full[c]), 4);
      mbar_init(smem_u32(&bars->a_empty[c]), 1);
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
                 "r"(W_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  TileWalk it;
  it.init(n_tiles, num_groups, BN_OUT, group_offsets);
  const TileCoord& tc = it.tc;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      uint32_t idx = 0;  // k-blocks issued by this CTA so far
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
        const int n1 = (MODE == kSwiGLU) ? tc.n0 : tc.n0 + WBOX;
        const int nbox = (it.rows() + WBOX - 1) / WBOX;
        for (int kb = 0; kb < num_kb; ++kb, ++idx) {
          const int stage = idx % W_S_STAGES;
          const uint32_t phase = (idx / W_S_STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1600 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sw = smem_base + stage * W_STAGE_BYTES;
          mbar_expect_tx(full, W_WQ_BYTES + nbox * W_BOX_X_BYTES);
          tma_load_2d(sw, m0, full, kb * BK, tc.n0);
          tma_load_2d(sw + W_WQ_BYTES / 2, m1, full, kb * BK, n1);
          for (int b = 0; b < nbox; ++b)
            tma_load_2d(sw + W_WQ_BYTES + b * W_BOX_X_BYTES, &tmap_x, full, kb * BK, tc.row0 + b * WBOX);
          armed |= 1u << stage;
        }
      }
      if (*abort_flag) {
        // copies in flight must land before the CTA exits: wait (bounded) for every armed stage
        const int stage = idx % W_S_STAGES;
        const uint32_t phase = (idx / W_S_STAGES) & 1u;
        for (int s = 0; s < W_S_STAGES; ++s) {
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
          report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1700 + acc);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t idesc = idesc_wide((it.rows() + 15) & ~15);
        const uint32_t d_tmem = tmem_base + acc * WTN;
        for (int kb = 0; kb < num_kb; ++kb, ++idx) {
          const int stage = idx % W_S_STAGES, tstage = idx % W_T_STAGES;
          const uint32_t phase = (idx / W_S_STAGES) & 1u, tphase = (idx / W_T_STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
              !mbar_wait(smem_u32(&bars->a_full[tstage]), tphase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1710 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t db = make_smem_desc(smem_base + stage * W_STAGE_BYTES + W_WQ_BYTES);
          const uint32_t a0 = tmem_base + W_RING_COL + tstage * W_A_COLS;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            // 16 bf16 of K = 8 TMEM columns of the A tile, 32 bytes of the swizzled B row
            tc_mma_bf16_tmem_a(d_tmem, a0 + k * (UMMA_K / 2), db + 2 * k, idesc, accum);
          }
          tc_commit(smem_u32(&bars->empty[stage]));     // token tile of this stage consumed
          tc_commit(smem_u32(&bars->a_empty[tstage]));  // widened tile of this TMEM stage consumed
        }
        if (ok) tc_commit(smem_u32(&bars->acc_full[acc]));
        acc_phase[acc] ^= 1u;
        acc ^= 1;
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ================= int8 -> bf16 widening into tensor memory =================
    // Group (warp - 4) / 4 takes the k-blocks of its parity; warp quarter w % 4 owns TMEM lanes
    // [32q, 32q + 32); each thread widens one weight row of the k-block: 64 int8 = four 16-byte
    // pieces.  The boxes are 64B-swizzled (piece index XOR (row / 2) mod 4): the eight lanes of one
    // shared-memory wavefront read eight consecutive rows, which touch every bank once.
    const uint32_t group = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int srow = (MODE == kSwiGLU) ? ((lane < 16) ? quarter * 16 + lane : 64 + quarter * 16 + (lane - 16))
                                       : quarter * 32 + lane;
    const int sw = (srow >> 1) & 3;
    uint32_t idx = 0;
    int pend_stage = -1, pend_tstage = -1;
    bool ok = true;
    // The TMEM store of one k-block stays in flight while this group's next k-block is read and
    // widened; its completion is awaited (and the barriers signalled) just before the next store.
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
    while (ok && it.next()) {
      for (int kb = 0; kb < num_kb; ++kb, ++idx) {
        if ((idx & 1u) != group) continue;
        const int stage = idx % W_S_STAGES, tstage = idx % W_T_STAGES;
        const uint32_t phase = (idx / W_S_STAGES) & 1u, tphase = (idx / W_T_STAGES) & 1u;
        if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1800 + warp);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint8_t* q = smem_aligned + stage * W_STAGE_BYTES + srow * BK;
        uint4 p[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) p[c] = *reinterpret_cast<const uint4*>(q + ((c ^ sw) << 4));
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          widen4(p[c].x, v[8 * c + 0], v[8 * c + 1]);
          widen4(p[c].y, v[8 * c + 2], v[8 * c + 3]);
          widen4(p[c].z, v[8 * c + 4], v[8 * c + 5]);
          widen4(p[c].w, v[8 * c + 6], v[8 * c + 7]);
        }
        retire();
        if (!mbar_wait(smem_u32(&bars->a_empty[tstage]), tphase ^ 1u, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1820 + warp);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + W_RING_COL + tstage * W_A_COLS;
        tc_st32(taddr, v);
        pend_stage = stage;
        pend_tstage = tstage;
      }
    }
    retire();
  } else if (warp >= 12) {
    // ================= epilogue =================
    // Column t of an accumulator is token row0 + t.  kSwiGLU: lane l < 16 of quarter q holds the gate
    // row of feature n0 + 16q + l, lane l + 16 its up row; the two exchange their scaled values and
    // share the work (lanes < 16 finish even columns, lanes >= 16 odd ones), so for one token the 16
    // storing lanes of a warp write 32 contiguous bytes.  kPlain: lane l holds output row n0 + 32q + l.
    const int quarter = warp & 3;
    const int half = (warp - 12) >> 2;  // which of the two warps of this lane quarter
    const int upper = lane >> 4;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    while (it.next()) {
      if (!mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase[acc], abort_flag)) {
        if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1900 + acc);
        *abort_flag = 1;
        break;
      }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int rows = it.rows();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * WTN;
      if (MODE == kSwiGLU) {
        const int n = tc.n0 + quarter * 16 + (lane & 15);
        const bool n_ok = n < N;
        const float sc = n_ok ? (upper ? scale1[tc.group][n] : scale0[tc.group][n]) : 0.f;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N + n;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t a[16];
          tc_ld16(taddr + c, a);
          tc_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float mine = __uint_as_float(a[j]) * sc;
            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
            const float gv = upper ? other : mine, uv = upper ? mine : other;
            if ((j & 1) == upper && n_ok && c + j < rows) obase[(size_t)(c + j) * N] = __float2bfloat16(silu_mul(gv, uv));
          }
        }
      } else {
        const int n = tc.n0 + quarter * 32 + lane;
        const bool n_ok = n < N;
        const float sc = n_ok ? scale0[tc.group][n] : 0.f;
        __nv_bfloat16* obase = out + (size_t)tc.row0 * N + n;
#pragma unroll 1
        for (int c = half * 16; c < rows; c += 32) {
          uint32_t a[16];
          tc_ld16(taddr + c, a);
          tc_ld_wait();
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c + j < rows) obase[(size_t)(c + j) * N] = __float2bfloat16(__uint_as_float(a[j]) * sc);
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(W_TMEM_COLS)
                 : "memory");
  }
}

template <int MODE>
int launch_wide_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_w8_wide_kernel<MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES));
  }
  grouped_gemm_w8_wide_kernel<MODE><<<dim3(num_sms), dim3(W_THREADS), W_SMEM_BYTES, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.scale0, a.scale1, a.err);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_grouped_gemm_w8_wide(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (!a.scale0 || (a.mode == kSwiGLU && !a.scale1)) return ATENIA_ERR_NULL;
  int rc = a.mode == kSwiGLU ? launch_wide_one<kSwiGLU>(a, num_sms, s) : launch_wide_one<kPlain>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

}  // namespace atenia
