// Grouped expert GEMM for sm_100a: TMA-fed tcgen05.mma with TMEM accumulators.
//
// One launch covers every expert of a layer.  A persistent grid (one CTA per SM) walks a tile list
// derived on the device from the dispatch offsets, so the host never reads routing results.
//
//   tile            = 128 rows of one expert  x  BN_OUT output columns
//   kSwiGLU         : B tile = 128 rows of W_gate || 128 rows of W_up  -> one M128 x N256 MMA,
//                     epilogue h = silu(g) * u, BN_OUT = 128
//   kPlain          : B tile = 256 rows of W_down                       -> one M128 x N256 MMA,
//                     BN_OUT = 256
//   k-block         = 64 bf16 (128 bytes: exactly one 128B-swizzle row), 4 MMAs of K = 16
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer,
// warps 2..5 = epilogue (each owns the 32 TMEM lanes its warp id modulo 4 selects).
// The accumulator is double buffered (2 x 256 TMEM columns), so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// INT8 weights (W8A16, template flag W8): the weight tiles arrive by TMA as int8 (16 KiB per stage
// instead of 32), four extra warps widen them to bf16 in registers and write the 128B-swizzled
// operand tile the MMA reads; the per-row scale multiplies the f32 accumulator column in the
// epilogue ((q*s).x = s*(q.x) exactly, and |q| <= 127 is exact in bf16).  HBM and L2 see one byte per
// weight.
//
// Every wait is bounded: a wait that runs out records ATENIA_ERR_DEVICE_TIMEOUT with a site id and
// the CTA leaves its loops, waits (bounded) for its own TMA copies, frees TMEM and returns.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int BN = 256;  // MMA N
constexpr int STAGES = 4;
constexpr int ACC_BUFS = 2;
constexpr int TMEM_COLS = 512;
constexpr int A_STAGE_BYTES = BM * BK * 2;      // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;      // 32 KiB
constexpr int B_HALF_BYTES = B_STAGE_BYTES / 2; // 16 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
// W8A16 variant: TMA ring of {A bf16 16 KiB, B int8 16 KiB} x 3 and a ring of widened bf16 B tiles x 3.
constexpr int Q_STAGE_BYTES = BN * BK;               // 16 KiB of int8
constexpr int Q_HALF_BYTES = Q_STAGE_BYTES / 2;
constexpr int W8_STAGE_BYTES = A_STAGE_BYTES + Q_STAGE_BYTES;  // 32 KiB
constexpr int W8_STAGES = 3;
constexpr int CONV_STAGES = 3;  // must not be a multiple of CONV_GROUPS apart from 1 (groups rotate through the ring)
constexpr int CONV_GROUPS = 2;       // groups of widening warps, taking k-blocks in turn
constexpr int CONV_GROUP_WARPS = 8;  // warps per group
constexpr int CONV_WARPS = CONV_GROUPS * CONV_GROUP_WARPS;
constexpr int W8_NUM_THREADS = 192 + CONV_WARPS * 32;  // + warps 6..21: widen int8 -> bf16
constexpr int W8_SMEM_BYTES = W8_STAGES * W8_STAGE_BYTES + CONV_STAGES * B_STAGE_BYTES + 1024 + 256;


// Instruction descriptor, kind::f16: D = f32 (bit 4), A = B = bf16 (bits 7, 10), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN >> 3) << 17) |
                                (uint32_t(BM >> 4) << 24);


struct __align__(8) SharedBarriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t conv_full[CONV_STAGES];   // W8: widened tile ready (every widening warp arrives)
  uint64_t conv_empty[CONV_STAGES];  // W8: MMAs that read the widened tile are done
  uint64_t acc_full[ACC_BUFS];
  uint64_t acc_empty[ACC_BUFS];
  uint32_t tmem_base;
  int abort_flag;
};


template <int MODE, bool W8>
__global__ void __launch_bounds__(W8 ? W8_NUM_THREADS : NUM_THREADS, 1)
grouped_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const CUtensorMap* __restrict__ tmap_b0,
                            const CUtensorMap* __restrict__ tmap_b1, const int32_t* __restrict__ group_offsets_g,
                            int num_groups, int N, int K, __nv_bfloat16* __restrict__ out,
                            const float* const* __restrict__ scale0, const float* const* __restrict__ scale1,
                            DeviceError* err) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int32_t goff_s[kMaxGroupsShared + 1];
  const int32_t* group_offsets = stage_group_offsets(group_offsets_g, num_groups, goff_s);
  constexpr int BN_OUT = (MODE == kSwiGLU) ? BN / 2 : BN;
  // 1024-byte alignment is required by the 128B swizzle atoms.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  // ring strides: bf16 weights keep A and B of a stage together; W8 keeps {A, int8 B} in the TMA ring
  // and the widened B tiles in a second ring behind it
  constexpr int RING_STRIDE = W8 ? W8_STAGE_BYTES : STAGE_BYTES;
  constexpr int TX_BYTES = RING_STRIDE;
  constexpr int NS = W8 ? W8_STAGES : STAGES;  // depth of the TMA ring
  constexpr uint32_t CONV_BASE_OFF = W8_STAGES * W8_STAGE_BYTES;
  constexpr int TOTAL_TILE_BYTES = W8 ? W8_STAGES * W8_STAGE_BYTES + CONV_STAGES * B_STAGE_BYTES : STAGES * STAGE_BYTES;
  SharedBarriers* bars = reinterpret_cast<SharedBarriers*>(smem_aligned + TOTAL_TILE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), W8 ? 1 + CONV_GROUP_WARPS : 1);  // MMA commit (+ one widening group)
    }
    for (int c = 0; c < CONV_STAGES; ++c) {
      mbar_init(smem_u32(&bars->conv_full[c]), CONV_GROUP_WARPS);
      mbar_init(smem_u32(&bars->conv_empty[c]), 1);
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      mbar_init(smem_u32(&bars->acc_full[b]), 1);
      mbar_init(smem_u32(&bars->acc_empty[b]), 4);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS)
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
  if (num_groups > 0) cursor_load(cur, group_offsets);
  TileCoord tc;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int last_group = -1;
      uint32_t armed = 0;  // stages with a copy possibly in flight
      bool ok = true;
      for (int tile = blockIdx.x; ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT);
           tile += gridDim.x) {
        if (tc.group != last_group) {
          tmap_acquire(&tmap_b0[tc.group]);
          if (MODE == kSwiGLU) tmap_acquire(&tmap_b1[tc.group]);
          last_group = tc.group;
        }
        const CUtensorMap* mb0 = &tmap_b0[tc.group];
        const CUtensorMap* mb1 = (MODE == kSwiGLU) ? &tmap_b1[tc.group] : mb0;
        const int n1 = (MODE == kSwiGLU) ? tc.n0 : tc.n0 + BN / 2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 100 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bars->full[stage]);
          const uint32_t sa = smem_base + stage * RING_STRIDE;
          const uint32_t sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(full, TX_BYTES);
          tma_load_2d(sa, &tmap_a, full, kb * BK, tc.row0);
          tma_load_2d(sb, mb0, full, kb * BK, tc.n0);
          tma_load_2d(sb + (W8 ? Q_HALF_BYTES : B_HALF_BYTES), mb1, full, kb * BK, n1);
          armed |= 1u << stage;
          if (++stage == NS) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (*abort_flag) {
        // Let copies already issued land before the CTA's shared memory is released.
        for (int s = 0; s < NS; ++s) {
          if (!(armed & (1u << s))) continue;
          uint32_t par = (s < stage) ? phase : (phase ^ 1u);
          mbar_wait(smem_u32(&bars->full[s]), par, abort_flag + 0 * s, 1u << 20);
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int cstage = 0;
      uint32_t cphase = 0;
      uint32_t acc_phase[ACC_BUFS] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT);
           tile += gridDim.x, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase[acc] ^ 1u, abort_flag)) {
          report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 200 + acc);
          *abort_flag = 1;
          break;
        }
        acc_phase[acc] ^= 1u;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 300 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (W8 && !mbar_wait(smem_u32(&bars->conv_full[cstage]), cphase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 350 + cstage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * RING_STRIDE;
          const uint32_t sb = W8 ? smem_base + CONV_BASE_OFF + cstage * B_STAGE_BYTES : sa + A_STAGE_BYTES;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 bf16 = 32 bytes along K inside the swizzle row: +2 in address>>4 units
            tc_mma_bf16(d_tmem, da + 2 * k, db + 2 * k, kInstrDesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(smem_u32(&bars->empty[stage]));  // frees the stage once these MMAs have read it
          if (W8) {
            tc_commit(smem_u32(&bars->conv_empty[cstage]));
            if (++cstage == CONV_STAGES) {
              cstage = 0;
              cphase ^= 1u;
            }
          }
          if (++stage == NS) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(smem_u32(&bars->acc_full[acc]));
      }
    }
  } else if (W8 && warp >= 6) {
    // ================= int8 -> bf16 widening (warps 6.., W8 only) =================
    // Per k-block: 256 rows x 64 int8.  Thread t of the CONV_WARPS * 32 handles 16-byte pieces (row, c)
    // with row = (t >> 2) + CONV_WARPS * 8 * i, c = t & 3 (each warp is latency-bound on its own chain of
    // load, widen, store, so many warps with little work each beat few warps with a lot): sixteen codes become two 16-byte pieces of the row's 128-byte
    // bf16 line, stored at the 128B-swizzled position (piece index XOR row mod 8) the MMA expects.
    // The widening warps form CONV_GROUPS groups that take k-blocks in turn: a group's chain of wait,
    // load, widen, store, proxy fence and arrive has a latency of several hundred cycles, and groups
    // working on different k-blocks overlap those chains.
    const int ct = (threadIdx.x - 192) % (CONV_GROUP_WARPS * 32);
    const int grp = (threadIdx.x - 192) / (CONV_GROUP_WARPS * 32);
    const int cw = (threadIdx.x - 192) >> 5;
    uint32_t gk = 0;  // k-blocks seen so far, across tiles
    bool ok = true;
    for (int tile = blockIdx.x; ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT);
         tile += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb, ++gk) {
        if ((int)(gk % CONV_GROUPS) != grp) continue;
        const int stage = gk % NS, cstage = gk % CONV_STAGES;
        const uint32_t phase = (gk / NS) & 1u, cphase = (gk / CONV_STAGES) & 1u;
        if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag) ||
            !mbar_wait(smem_u32(&bars->conv_empty[cstage]), cphase ^ 1u, abort_flag)) {
          if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 500 + cw);
          *abort_flag = 1;
          ok = false;
          break;
        }
        const uint8_t* q = smem_aligned + stage * W8_STAGE_BYTES + A_STAGE_BYTES;
        uint8_t* b = smem_aligned + CONV_BASE_OFF + cstage * B_STAGE_BYTES;
        const int c = ct & 3;
#pragma unroll
        for (int i = 0; i < BN / (CONV_GROUP_WARPS * 8); ++i) {
          const int row = (ct >> 2) + CONV_GROUP_WARPS * 8 * i;
          const uint4 v = *reinterpret_cast<const uint4*>(q + row * BK + c * 16);
          uint4 o0, o1;
          widen4(v.x, o0.x, o0.y);
          widen4(v.y, o0.z, o0.w);
          widen4(v.z, o1.x, o1.y);
          widen4(v.w, o1.z, o1.w);
          uint8_t* line = b + row * 128;
          *reinterpret_cast<uint4*>(line + (((2 * c) ^ (row & 7)) << 4)) = o0;
          *reinterpret_cast<uint4*>(line + (((2 * c + 1) ^ (row & 7)) << 4)) = o1;
        }
        fence_proxy_async();  // generic-proxy writes above must be visible to the MMA's async-proxy reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bars->conv_full[cstage]));
          mbar_arrive(smem_u32(&bars->empty[stage]));  // the int8 tile of this stage has been read
        }
      }
    }
  } else {
    // ================= epilogue (warps 2..5) =================
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
    const int row_in_tile = quarter * 32 + lane;
    uint32_t acc_phase[ACC_BUFS] = {0, 0};
    int it = 0;
    for (int tile = blockIdx.x; cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT);
         tile += gridDim.x, ++it) {
      const int acc = it & 1;
      if (!mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase[acc], abort_flag)) {
        if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 400 + acc);
        *abort_flag = 1;
        break;
      }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int grow = tc.row0 + row_in_tile;
      const bool row_ok = grow < tc.row_end;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      __nv_bfloat16* orow = out + (size_t)grow * N;
      const float* sc0 = scale0 ? scale0[tc.group] : nullptr;
      const float* sc1 = (scale1 && MODE == kSwiGLU) ? scale1[tc.group] : nullptr;
      if (MODE == kSwiGLU) {
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
              float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
              float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
              if (sc0) {
                g0 *= sc0[n + 2 * j];
                g1 *= sc0[n + 2 * j + 1];
                u0 *= sc1[n + 2 * j];
                u1 *= sc1[n + 2 * j + 1];
              }
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
            for (int j = 0; j < 8; ++j) {
              float a0 = __uint_as_float(v[2 * j]), a1 = __uint_as_float(v[2 * j + 1]);
              if (sc0) {
                a0 *= sc0[n + 2 * j];
                a1 *= sc0[n + 2 * j + 1];
              }
              p[j] = pack_bf16x2(a0, a1);
            }
            uint4* dst = reinterpret_cast<uint4*>(orow + n);
            dst[0] = make_uint4(p[0], p[1], p[2], p[3]);
            dst[1] = make_uint4(p[4], p[5], p[6], p[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---- CUDA-core checking kernel ----------------------------------------------------------------
__global__ void grouped_gemm_check_kernel(GroupedGemmCheckArgs a) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int row = blockIdx.y;
  if (n >= a.N) return;
  const int total = a.group_offsets[a.num_groups];
  if (row >= total) return;
  int g = 0;
  while (g + 1 < a.num_groups && row >= a.group_offsets[g + 1]) ++g;
  const __nv_bfloat16* x = a.a + (size_t)row * a.K;
  float acc0 = 0.f, acc1 = 0.f;
  if (a.b_is_int8) {
    const int8_t* w0 = static_cast<const int8_t*>(a.b0[g]) + (size_t)n * a.K;
    const int8_t* w1 = a.mode == kSwiGLU ? static_cast<const int8_t*>(a.b1[g]) + (size_t)n * a.K : nullptr;
    for (int k = 0; k < a.K; ++k) {
      float xv = __bfloat162float(x[k]);
      acc0 = fmaf(xv, (float)w0[k], acc0);
      if (w1) acc1 = fmaf(xv, (float)w1[k], acc1);
    }
  } else {
    const __nv_bfloat16* w0 = static_cast<const __nv_bfloat16*>(a.b0[g]) + (size_t)n * a.K;
    const __nv_bfloat16* w1 =
        a.mode == kSwiGLU ? static_cast<const __nv_bfloat16*>(a.b1[g]) + (size_t)n * a.K : nullptr;
    for (int k = 0; k < a.K; ++k) {
      float xv = __bfloat162float(x[k]);
      acc0 = fmaf(xv, __bfloat162float(w0[k]), acc0);
      if (w1) acc1 = fmaf(xv, __bfloat162float(w1[k]), acc1);
    }
  }
  if (a.scale0) {
    acc0 *= a.scale0[g][n];
    if (a.mode == kSwiGLU) acc1 *= a.scale1[g][n];
  }
  float r = a.mode == kSwiGLU ? acc0 / (1.0f + expf(-acc0)) * acc1 : acc0;
  a.out[(size_t)row * a.N + n] = __float2bfloat16(r);
}

}  // namespace

template <int MODE, bool W8>
static int launch_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  constexpr int kSmem = W8 ? W8_SMEM_BYTES : SMEM_BYTES;
  constexpr int kThreads = W8 ? W8_NUM_THREADS : NUM_THREADS;
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_tcgen05_kernel<MODE, W8>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  }
  grouped_gemm_tcgen05_kernel<MODE, W8><<<dim3(num_sms), dim3(kThreads), kSmem, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.scale0, a.scale1, a.err);
  return (int)cudaGetLastError();
}

int launch_grouped_gemm_tcgen05(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (a.w8 && (!a.scale0 || (a.mode == kSwiGLU && !a.scale1))) return ATENIA_ERR_NULL;
  int rc;
  if (a.mode == kSwiGLU) rc = a.w8 ? launch_one<kSwiGLU, true>(a, num_sms, s) : launch_one<kSwiGLU, false>(a, num_sms, s);
  else rc = a.w8 ? launch_one<kPlain, true>(a, num_sms, s) : launch_one<kPlain, false>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

int launch_grouped_gemm_check(const GroupedGemmCheckArgs& a, cudaStream_t s) {
  if (a.num_groups <= 0 || a.max_rows <= 0) return ATENIA_OK;
  dim3 block(128), grid((a.N + 127) / 128, a.max_rows);
  grouped_gemm_check_kernel<<<grid, block, 0, s>>>(a);
  count_launch();
  return (int)cudaGetLastError();
}

// ---- tensor maps --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

int encode_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                      uint32_t box_cols, int swizzle64) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return ATENIA_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || cols % 16 != 0) return ATENIA_ERR_SHAPE;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle64 == 2 ? CU_TENSOR_MAP_SWIZZLE_128B
                                 : (swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ATENIA_OK : ATENIA_ERR_DRIVER;
}

int encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return ATENIA_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0) return ATENIA_ERR_SHAPE;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ATENIA_OK : ATENIA_ERR_DRIVER;
}

}  // namespace atenia
