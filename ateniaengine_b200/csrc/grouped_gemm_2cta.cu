// Grouped expert GEMM for bf16 weights with CTA pairs (tcgen05 cta_group::2).
//
// Two CTAs on the two SMs of a TPC form a cluster and work on one 256-row x 256-column MMA tile:
// each CTA stages its own 128 token rows (A) and only HALF of the weight tile (B: the gate rows in
// rank 0 and the up rows in rank 1 for kSwiGLU; the two 128-row halves of W_down for kPlain).  One
// thread of the leader CTA issues tcgen05.mma.cta_group::2 (M256 x N256 x K16), which reads A and B
// from both CTAs' shared memory and accumulates each CTA's 128 rows in that CTA's tensor memory.
// Per CTA a k-block costs 32 KiB of L2->shared traffic instead of 48 KiB, for the same math: the
// single-CTA kernel is limited by how many bytes it can keep in flight, this one by the tensor pipe.
//
// No TMA multicast is used: every CTA fetches its own tiles (cp.async.bulk.tensor ... cta_group::2
// only routes the completion to the leader's mbarrier).
//
// Barriers: full[s] lives in the leader and collects the bytes of both CTAs; empty[s] and
// acc_full[b] exist in both CTAs and are signalled by tcgen05.commit with a CTA mask; acc_empty[b]
// lives in the leader and is arrived on by the epilogue warps of both CTAs.
// Tiles are pairs of 128-row m-tiles of one expert; a pair whose second half lies past the expert's
// rows still runs (the MMA is one instruction for both) and masks its stores.
#include "tc_common.cuh"

namespace atenia {
namespace {
using namespace tc;

constexpr int BN2 = 256;
constexpr int PAIR_ROWS = 2 * BM;  // 256
constexpr int STAGES2 = 6;
constexpr int ACC_BUFS2 = 2;
constexpr int TMEM_COLS2 = 512;
constexpr int A_BYTES2 = BM * BK * 2;         // 16 KiB
constexpr int BH_BYTES2 = (BN2 / 2) * BK * 2; // 16 KiB: this CTA's half of the weight tile
constexpr int STAGE_BYTES2 = A_BYTES2 + BH_BYTES2;
constexpr int NUM_THREADS2 = 192;
constexpr int SMEM_BYTES2 = STAGES2 * STAGE_BYTES2 + 1024 + 256;

struct __align__(8) Barriers2 {
  uint64_t full[STAGES2];
  uint64_t empty[STAGES2];
  uint64_t acc_full[ACC_BUFS2];
  uint64_t acc_empty[ACC_BUFS2];
  uint32_t tmem_base;
  int abort_flag;
};

// D f32, A = B = bf16, K-major, M = 256 (per pair), N = 256.
constexpr uint32_t kInstrDesc2 = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(BN2 >> 3) << 17) |
                                 (uint32_t(PAIR_ROWS >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes go to an mbarrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS2, 1)
grouped_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const CUtensorMap* __restrict__ tmap_b0,
                         const CUtensorMap* __restrict__ tmap_b1, const int32_t* __restrict__ group_offsets_g,
                         int num_groups, int N, int K, __nv_bfloat16* __restrict__ out, DeviceError* err) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int32_t goff_s[kMaxGroupsShared + 1];
  const int32_t* group_offsets = stage_group_offsets(group_offsets_g, num_groups, goff_s);
  constexpr int BN_OUT = (MODE == kSwiGLU) ? BN2 / 2 : BN2;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  Barriers2* bars = reinterpret_cast<Barriers2*>(smem_aligned + STAGES2 * STAGE_BYTES2);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_kb = (K + BK - 1) / BK;
  const int n_tiles = (N + BN_OUT - 1) / BN_OUT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int b = 0; b < ACC_BUFS2; ++b) {
      mbar_init(smem_u32(&bars->acc_full[b]), 1);
      mbar_init(smem_u32(&bars->acc_empty[b]), 8);  // 4 epilogue warps of each CTA
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&bars->tmem_base)),
                 "r"(TMEM_COLS2)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  TileCursor cur;
  cur.group = 0;
  cur.base = 0;
  if (num_groups > 0) cursor_load(cur, group_offsets, PAIR_ROWS);
  TileCoord tc;

  if (warp == 0) {
    // ================= TMA producer (both CTAs) =================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int last_group = -1;
      uint32_t armed = 0;
      bool ok = true;
      for (int tile = pair; ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, PAIR_ROWS);
           tile += num_pairs) {
        // this CTA's half of the weight tile
        const CUtensorMap* mb;
        int nb;
        if (MODE == kSwiGLU) {
          mb = leader ? &tmap_b0[tc.group] : &tmap_b1[tc.group];
          nb = tc.n0;
        } else {
          mb = &tmap_b0[tc.group];
          nb = tc.n0 + (leader ? 0 : BN2 / 2);
        }
        if (tc.group != last_group) {
          tmap_acquire(mb);
          last_group = tc.group;
        }
        const int my_row0 = tc.row0 + (int)rank * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1100 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full_local = smem_u32(&bars->full[stage]);
          const uint32_t full_leader = mapa(full_local, 0);
          const uint32_t sa = smem_base + stage * STAGE_BYTES2;
          const uint32_t sb = sa + A_BYTES2;
          if (leader) mbar_expect_tx(full_local, 2 * STAGE_BYTES2);  // bytes of both CTAs
          tma_load_2d_pair(sa, &tmap_a, full_leader, kb * BK, my_row0);
          tma_load_2d_pair(sb, mb, full_leader, kb * BK, nb);
          armed |= 1u << stage;
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      (void)armed;
    }
  } else if (warp == 1) {
    // ================= MMA issuer (leader CTA only) =================
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[ACC_BUFS2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int tile = pair; ok && cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, PAIR_ROWS);
           tile += num_pairs, ++it) {
        const int acc = it & 1;
        if (!mbar_wait(smem_u32(&bars->acc_empty[acc]), acc_phase[acc] ^ 1u, abort_flag)) {
          report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1200 + acc);
          *abort_flag = 1;
          break;
        }
        acc_phase[acc] ^= 1u;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
            report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1300 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES2;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sa + A_BYTES2);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, kInstrDesc2, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit_pair(smem_u32(&bars->empty[stage]));
          if (++stage == STAGES2) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit_pair(smem_u32(&bars->acc_full[acc]));
      }
    }
  } else {
    // ================= epilogue (warps 2..5 of both CTAs) =================
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    uint32_t acc_phase[ACC_BUFS2] = {0, 0};
    int it = 0;
    for (int tile = pair; cursor_seek(cur, tile, n_tiles, num_groups, group_offsets, tc, BN_OUT, PAIR_ROWS);
         tile += num_pairs, ++it) {
      const int acc = it & 1;
      if (!mbar_wait(smem_u32(&bars->acc_full[acc]), acc_phase[acc], abort_flag)) {
        if (lane == 0) report_error(err, ATENIA_ERR_DEVICE_TIMEOUT, 1400 + acc);
        *abort_flag = 1;
        break;
      }
      acc_phase[acc] ^= 1u;
      tc_fence_after();
      const int grow = tc.row0 + (int)rank * BM + row_in_tile;
      const bool row_ok = grow < tc.row_end;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN2;
      __nv_bfloat16* orow = out + (size_t)grow * N;
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
            for (int j = 0; j < 8; ++j)
              p[j] = pack_bf16x2(silu_mul(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j])),
                                 silu_mul(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1])));
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
            for (int j = 0; j < 8; ++j) p[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            uint4* dst = reinterpret_cast<uint4*>(orow + n);
            dst[0] = make_uint4(p[0], p[1], p[2], p[3]);
            dst[1] = make_uint4(p[4], p[5], p[6], p[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(mapa(smem_u32(&bars->acc_empty[acc]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while its peer may still signal or read it
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS2)
                 : "memory");
  }
}

template <int MODE>
int launch_2cta_one(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  static bool attr_set[kMaxDevices] = {};
  if (first_use_on_current_device(attr_set)) {
    ATENIA_CUDA_TRY(cudaFuncSetAttribute(grouped_gemm_2cta_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES2));
  }
  const int grid = num_sms & ~1;  // whole pairs
  grouped_gemm_2cta_kernel<MODE><<<dim3(grid), dim3(NUM_THREADS2), SMEM_BYTES2, s>>>(
      a.tmap_a, a.tmap_b0, MODE == kSwiGLU ? a.tmap_b1 : a.tmap_b0, a.group_offsets, a.num_groups, a.N, a.K, a.out,
      a.err);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_grouped_gemm_2cta(const GroupedGemmArgs& a, int num_sms, cudaStream_t s) {
  if (a.num_groups <= 0) return ATENIA_OK;
  if (a.N % 16 != 0 || a.K % 16 != 0) return ATENIA_ERR_SHAPE;
  if (a.w8) return ATENIA_ERR_UNSUPPORTED;  // INT8 weights: w8_gemm.cu / w8_gemm_m256.cu
  int rc = a.mode == kSwiGLU ? launch_2cta_one<kSwiGLU>(a, num_sms, s) : launch_2cta_one<kPlain>(a, num_sms, s);
  count_launch();
  count_tcgen05_launch();
  return rc;
}

}  // namespace atenia
