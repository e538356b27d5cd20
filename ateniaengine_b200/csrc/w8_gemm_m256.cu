// Grouped expert GEMM for INT8 weights (W8A16) at large batches: 256 token rows per CTA share every
// widened weight tile.
//
// Widening int8 codes to bf16 on chip costs shared-memory bandwidth, which is what bounds the kernels
// that widen into shared memory: per k-block the 128-row tile of grouped_gemm.cu moves 16 KiB of
// codes in, reads them, writes 32 KiB of bf16 back and lets the MMA read those 32 KiB again, for
// 128 x 256 x 64 multiply-adds (measured: 1280 cycles per k-block, the tensor pipe 40 % busy).  Here one
// CTA owns a 256-row token tile: the widened 256 x 64 weight tile is written once and read by TWO
// M128 x N256 MMAs (token rows 0..127 and 128..255), so the widening traffic per multiply-add is halved
// and a k-block's shared-memory traffic (192 KiB for 256 x 256 x 64) is about what the two MMAs take
// anyway.  The two f32 accumulators fill tensor memory (2 x 256 columns), so the accumulator is not
// double-buffered: the epilogue of a tile (8 warps) runs while the TMA ring and the widening warps
// already work on the next tile's first k-blocks, and the MMAs resume when it has drained.
//
//   tile      = 256 tokens of one expert x { 128 gate + 128 up rows (kSwiGLU) | 256 down rows (kPlain) }
//   k-block   = 64: 32 KiB of bf16 tokens (two 128-row boxes, 128B swizzle) + 16 KiB of int8 weights
//               (two 128-row boxes, no swizzle) per stage, 3 stages; 2 buffers of 32 KiB for the widened
//               weight tile (128B swizzle, written by the widening warps)
//   TMEM      = columns [0,256) rows 0..127 of the tile, [256,512) rows 128..255
//   warps     : 0 TMA, 1 MMA + TMEM alloc, 2..5 epilogue of the first accumulator, 6..13 and 14..21 the
//               two widening groups (alternate k-blocks, one buffer each), 22..25 epilogue of the second
// (q * s) . x = s * (q . x) exactly and |q| <= 127 is exact in bf16: the MMA runs on the codes and the
// per-row scale multiplies the accumulator column in the epilogue.  All waits are bounded.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int M_ROWS = 256;                    // token rows per tile
constexpr int M_BN = 256;                      // MMA N
constexpr int M_STAGES = 3;                    // TMA ring
constexpr int M_CONV = 2;                      // widened weight tiles, one per widening group
constexpr int M_GROUP_WARPS = 8;
constexpr int M_A_BYTES = M_ROWS * BK * 2;     // 32 KiB
constexpr int M_Q_BYTES = M_BN * BK;           // 16 KiB
constexpr int M_STAGE_BYTES = M_A_BYTES + M_Q_BYTES;
constexpr int M_B_BYTES = M_BN * BK * 2;       // 32 KiB
constexpr int M_CONV_OFF = M_STAGES * M_STAGE_BYTES;
constexpr int M_THREADS = 26 * 32;
constexpr int M_SMEM_BYTES = M_CONV_OFF + M_CONV * M_B_BYTES + 1024 + 256;
constexpr int M_TMEM_COLS = 512;
constexpr int M_FIRST_CONV_WARP = 6;
constexpr int M_SECOND_EPI_WARP = M_FIRST_CONV_WARP + 2 * M_GROUP_WARPS;  // 22

struct __align__(8) BarriersM256 {
  uint64_t full[M_STAGES];     // TMA landed (1 arrival + bytes)
  uint64_t empty[M_STAGES];    // MMA commit (token tile read) + the 8 warps of one widening group (codes read)
  uint64_t conv_full[M_CONV];  // widened tile written (8 warps of the group that owns the buffer)
  uint64_t conv_empty[M_CONV]; // the MMAs that read it are done (commit)
  uint64_t acc_full;           // all MMAs of the tile done (commit)
  uint64_t acc_empty;          // 8 epilogue warps drained both accumulators
  uint32_t tmem_base;
  int abort_flag;
};

// D f32, A = B = bf16, K-major, M = 128, N = 256
constexpr uint32_t kInstrDescM = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(M_BN >> 3) << 17) | (uint32_t(128 >> 4) << 24);

template <int MODE>
__global__ void __launch_bounds__(M_THREADS, 1)
grouped_gemm_w8_m256_kernel(const __grid_constant__ CUtensorMap tmap_a, const CUtensorMap* __restrict__ tmap_b0,
                            const CUtensorMap* __restrict__ tmap_b1, const int32_t* __restrict__ group_offsets,
                            int num_groups, int N, int K, __nv_bfloat16* __restrict__ out,
                            const float* const* __restrict__ scale0, const float* const* __restrict__ scale1,
                            DeviceError* err) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int BN_OUT = (MODE == kSwiGLU) ? M_BN / 2 : M_BN;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  BarriersM256* bars = reinterpret_cast<BarriersM256*>(smem_aligned + M_CONV_OFF + M_CONV * M_B_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < M_STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1 + M_GROUP_WARPS);
    }
    for (int c = 0; c < M_CONV; ++c) {
      mbar_init(smem_u32(&bars->conv_full[c]), M_GROUP_WARPS);
      mbar_init(smem_u32(&bars->conv_empty[c]), 1);
    }
    mbar_init(smem_u32(&bars->acc_full), 1);
    mbar_init(smem_u32(&bars->acc_empty), 8);
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&bars->tmem_base)),
                 "r"(M_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  TileCursor cur;
  cur.group = 0;
  cur.base = 0;
  if (num_groups > 0) cursor_load(cur, group_offsets, M_ROWS);
  TileCoord tc;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      uint32_t gk = 0;  // k-blocks issued so far, across tiles
      int last_group = -1;
      uint32_t armed = 0;
      bool ok = true;
      for (int tile = blockIdx.x;
           ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, M_ROWS); tile += gridDim.x) {
        if (tc.group != last_group) {
          tmap_acquire(&tmap_b0[tc.group]);
          if (MODE == kSwiGLU) tmap_acquire(&tmap_b1[tc.group]);
          last_group = tc.group;
        }
        const CUtensorMap* mb0 = &tmap_b0[tc.group];
        const CUtensorMap* mb1 = (MODE == kSwiGLU) ? &tmap_b1[tc.group] : mb0;
        const int n1 = (MODE == kSwiGLU) ? tc.n0 : tc.n0 + M_BN / 2;
        for (int kb = 0; kb < num_kb; ++kb, ++gk) {
          const int stage = gk % M_STAGES;
          const uint32_t phase = (gk / M_STAGES) & 1u;
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 3100 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sa = smem_base + stage * M_STAGE_BYTES;
          const uint32_t sq = sa + M_A_BYTES;
          mbar_expect_tx(full, M_STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, full, kb * BK, tc.row0);
          tma_load_2d(sa + M_A_BYTES / 2, &tmap_a, full, kb * BK, tc.row0 + 128);
          tma_load_2d(sq, mb0, full, kb * BK, tc.n0);
          tma_load_2d(sq + M_Q_BYTES / 2, mb1, full, kb * BK, n1);
          armed |= 1u << stage;
        }
      }
      if (*abort_flag) {
        // copies already issued must land before the CTA's shared memory is released
        const int stage = gk % M_STAGES;
        const uint32_t phase = (gk / M_STAGES) & 1u;
        for (int s = 0; s < M_STAGES; ++s) {
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
      uint32_t gk = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x;
           ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, M_ROWS); tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars->acc_empty), acc_phase ^ 1u, abort_flag)) {
          report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 3200);
          *abort_flag = 1;
          break;
        }
        acc_phase ^= 1u;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb, ++gk) {
          const int stage = gk % M_STAGES, cstage = gk % M_CONV;
          const uint32_t phase = (gk / M_STAGES) & 1u, cphase = (gk / M_CONV) & 1u;
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
              !mbar_wait(smem_u32(&bars->conv_full[cstage]), cphase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 3300 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * M_STAGE_BYTES;
          const uint64_t da0 = make_smem_desc(sa), da1 = make_smem_desc(sa + M_A_BYTES / 2);
          const uint64_t db = make_smem_desc(smem_base + M_CONV_OFF + cstage * M_B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
            // 16 bf16 of K = 32 bytes inside the swizzled row: +2 in descriptor address units
            tc_mma_bf16(tmem_base, da0 + 2 * k, db + 2 * k, kInstrDescM, accum);
            tc_mma_bf16(tmem_base + M_BN, da1 + 2 * k, db + 2 * k, kInstrDescM, accum);
          }
          tc_commit(smem_u32(&bars->empty[stage]));
          tc_commit(smem_u32(&bars->conv_empty[cstage]));
        }
        if (ok) tc_commit(smem_u32(&bars->acc_full));
      }
    }
  } else if (warp >= M_FIRST_CONV_WARP && warp < M_SECOND_EPI_WARP) {
    // ================= int8 -> bf16 widening =================
    // Group g takes the k-blocks with gk % 2 == g and owns widened buffer g.  Per k-block 256 rows x 64
    // codes = 1024 16-byte pieces for the group's 256 threads: thread t takes pieces (row, c) with
    // row = (t >> 2) + 64 i, c = t & 3.  Sixteen codes become two 16-byte pieces of the row's 128-byte bf16
    // line, stored at the 128B-swizzled position (piece index XOR row mod 8) the MMA descriptor expects.
    const int ct = (threadIdx.x - M_FIRST_CONV_WARP * 32) % (M_GROUP_WARPS * 32);
    const int grp = (threadIdx.x - M_FIRST_CONV_WARP * 32) / (M_GROUP_WARPS * 32);
    uint32_t gk = 0;
    bool ok = true;
    for (int tile = blockIdx.x;
         ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, M_ROWS); tile += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb, ++gk) {
        if ((int)(gk % M_CONV) != grp) continue;
        const int stage = gk % M_STAGES;
        const uint32_t phase = (gk / M_STAGES) & 1u, cphase = (gk / M_CONV) & 1u;
        if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
            !mbar_wait(smem_u32(&bars->conv_empty[grp]), cphase ^ 1u, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 3500 + warp);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint8_t* q = smem_aligned + stage * M_STAGE_BYTES + M_A_BYTES;
        uint8_t* b = smem_aligned + M_CONV_OFF + grp * M_B_BYTES;
        const int c = ct & 3;
        uint4 v[M_BN / (M_GROUP_WARPS * 8)];
#pragma unroll
        for (int i = 0; i < M_BN / (M_GROUP_WARPS * 8); ++i)
          v[i] = *reinterpret_cast<const uint4*>(q + ((ct >> 2) + M_GROUP_WARPS * 8 * i) * BK + c * 16);
#pragma unroll
        for (int i = 0; i < M_BN / (M_GROUP_WARPS * 8); ++i) {
          const int row = (ct >> 2) + M_GROUP_WARPS * 8 * i;
          uint4 o0, o1;
          widen4(v[i].x, o0.x, o0.y);
          widen4(v[i].y, o0.z, o0.w);
          widen4(v[i].z, o1.x, o1.y);
          widen4(v[i].w, o1.z, o1.w);
          uint8_t* line = b + row * 128;
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
  } else {
    // ================= epilogue: warps 2..5 rows 0..127, warps 22..25 rows 128..255 =================
    const int half = warp >= M_SECOND_EPI_WARP ? 1 : 0;
    const int quarter = warp & 3;  // TMEM lanes [32 quarter, 32 quarter + 32) belong to this warp
    const int row_in_tile = half * 128 + quarter * 32 + lane;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, M_ROWS);
         tile += gridDim.x) {
      if (!mbar_wait(smem_u32(&bars->acc_full), acc_phase, abort_flag)) {
        if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 3400 + warp);
        *abort_flag = 1;
        break;
      }
      acc_phase ^= 1u;
      tc_fence_after();
      const int grow = tc.row0 + row_in_tile;
      const bool row_ok = grow < tc.row_end;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + half * M_BN;
      __nv_bfloat16* orow = out + (size_t)grow * N;
      const float* sc0 = scale0[tc.group];
      if (MODE == kSwiGLU) {
        const float* sc1 = scale1[tc.group];
#pragma unroll 1
        for (int c = 0; c < BN_OUT; c += 16) {
          uint32_t g[16], u[16];
          tc_ld16(taddr + c, g);
          tc_ld16(taddr + BN_OUT + c, u);
          tc_ld_wait();
          const int n = tc.n0 + c;
          if (row_ok && n < N) {
            uint32_t p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = __uint_as_float(g[2 * j]) * sc0[n + 2 * j], g1 = __uint_as_float(g[2 * j + 1]) * sc0[n + 2 * j + 1];
              const float u0 = __uint_as_float(u[2 * j]) * sc1[n + 2 * j], u1 = __uint_as_float(u[2 * j + 1]) * sc1[n + 2 * j + 1];
              p[j] = pack_bf16x2(silu_mul(g0, u0), silu_mul(g1, u1));
            }
            uint4* dst = reinterpret_cast<uint4*>(orow + n);
            dst[0] = make_uint4(p[0], p[1], p[2], p[3]);
            dst[1] = make_uint4(p[4], p[5], p[6], p[7]);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN_OUT; c += 16) {
          uint32_t v[16];
          tc_ld16(taddr + c, v);
          tc_ld_wait();
          const int n = tc.n0 + c;
          if (row_ok && n < N) {
            uint32_t p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              p[j] = pack_bf16x2(__uint_as_float(v[2 * j]) * sc0[n + 2 * j], __uint_as_float(v[2 * j + 1]) * sc0[n + 2 * j + 1]);
            uint4* dst = reinterpret_cast<uint4*>(orow + n);
            dst[0] = make_uint4(p[0], p[1], p[2], p[3]);
            dst[1] = make_uint4(p[4], p[5], p[6], p[7]);
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(M_TMEM_COLS)
                 : "memory");
  }
}

template <int MODE>
int launch_m256_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_w8_m256_kernel<MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, M_SMEM_BYTES));
  }
  grouped_gemm_w8_m256_kernel<MODE><<<dim3(num_sms), dim3(M_THREADS), M_SMEM_BYTES, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.scale0, a.scale1, a.err);
  return (int)cudaGetLastError();
}

}  // namespace

// tmap_a: the bf16 token matrix with box {64, 128} (128B swizzle); tmap_b0 / b1: int8 maps with box {64, 128},
// unswizzled -- the maps of launch_grouped_gemm_tcgen05 with w8 set.
int launch_grouped_gemm_w8_m256(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (!a.scale0 || (a.mode == kSwiGLU && !a.scale1)) return ATENIA_ERR_NULL;
  int rc = a.mode == kSwiGLU ? launch_m256_one<kSwiGLU>(a, num_sms, s) : launch_m256_one<kPlain>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

}  // namespace atenia
