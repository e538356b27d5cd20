// Device-side building blocks shared by the tensor-core kernels: PTX wrappers (mbarrier, TMA,
// tcgen05), the shared-memory matrix descriptor, and the walk over the grouped tile list.
#pragma once
#include "common.cuh"

namespace atenia {
namespace tc {

constexpr int BM = 128;  // rows (tokens) per tile
constexpr int BK = 64;   // k elements per stage: 128 bytes of bf16 = one 128B-swizzle row
constexpr int UMMA_K = 16;
constexpr uint32_t kSpinLimit = 1u << 26;  // iterations of a try_wait loop before giving up

// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tmap_acquire(const CUtensorMap* m) {
  // A tensor map that lives in global memory and was written by the host is made visible to the
  // tensor-map proxy of this CTA before its first use.
  asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(m))
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, eight-row
// groups 1024 bytes apart.  Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused with a
// swizzled K-major tile, set to 1), [32,46) stride offset>>4, [46,48) version = 1, [61,64) swizzle
// mode (2 = 128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
__device__ __forceinline__ void tc_mma_bf16_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Four int8 codes (one 32-bit word) -> two packed bf16 pairs, exact.  With v = q & 0x7f and b7 the
// sign bit, q = (128 + v) - (128 + 128*b7).  Both terms are bf16 numbers that can be assembled by
// byte permutes: 0x43:v is 128 + v (bf16 has unit spacing in [128, 256)) and 0x43:(b7 << 7) is 128
// or 256.  One packed subtraction gives q.  (A and B of one tcgen05 kind::f16 MMA must have the
// same element type: bf16 activations with f16 weights is an illegal instruction on sm_100a.)
__device__ __forceinline__ void widen4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t v = w & 0x7f7f7f7fu;
  const uint32_t sg = w & 0x80808080u;
  const uint32_t a = __byte_perm(v, 0x43434343u, 0x5140);   // {0x43:v1, 0x43:v0}
  const uint32_t c = __byte_perm(sg, 0x43434343u, 0x5140);
  const uint32_t b = __byte_perm(v, 0x43434343u, 0x5342);   // {0x43:v3, 0x43:v2}
  const uint32_t d = __byte_perm(sg, 0x43434343u, 0x5342);
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(lo) : "r"(a), "r"(c));
  asm("sub.bf16x2 %0, %1, %2;" : "=r"(hi) : "r"(b), "r"(d));
}

__device__ __forceinline__ float silu_mul(float g, float u) {
  // silu(g) * u = g * u / (1 + exp(-g))
  return __fdividef(g * u, 1.0f + __expf(-g));
}

// ---- tile walk ---------------------------------------------------------------------------------
// The producer, the MMA issuer and the epilogue warps of a CTA each walk the group offsets at every tile
// change (a persistent CTA's next tile is a grid width further on: with 60 experts of 20 tiles that is
// seven groups, two dependent loads each).  From global memory that walk costs microseconds per tile and
// the ring runs dry meanwhile, so kernels with many groups copy the offsets into shared memory first.
constexpr int kMaxGroupsShared = 256;
__device__ __forceinline__ const int32_t* stage_group_offsets(const int32_t* __restrict__ off_global, int num_groups,
                                                              int32_t* off_shared) {
  if (num_groups > kMaxGroupsShared) return off_global;
  for (int i = threadIdx.x; i <= num_groups; i += blockDim.x) off_shared[i] = off_global[i];
  return off_shared;  // (valid after the caller's next block-wide barrier)
}

struct TileCursor {
  int group;      // current group
  int base;       // first tile index of the current group
  int m_tiles;    // m tiles of the current group
  int row_begin;  // first row of the group
  int row_end;
};
struct TileCoord {
  int group, row0, row_end, n0;
};

__device__ __forceinline__ void cursor_load(TileCursor& c, const int32_t* __restrict__ off, int tile_rows = BM) {
  c.row_begin = off[c.group];
  c.row_end = off[c.group + 1];
  c.m_tiles = (c.row_end - c.row_begin + tile_rows - 1) / tile_rows;
}
// Advance the cursor to the group holding `tile`; false when the tile list is exhausted.
__device__ __forceinline__ bool cursor_seek(TileCursor& c, int tile, int n_tiles, int num_groups,
                                            const int32_t* __restrict__ off, TileCoord& out, int bn_out,
                                            int tile_rows = BM) {
  while (c.group < num_groups) {
    int tiles_here = c.m_tiles * n_tiles;
    if (tile < c.base + tiles_here) {
      int local = tile - c.base;
      int nt = local / c.m_tiles;  // n-major, m-minor: neighbouring CTAs share a weight tile
      int mt = local - nt * c.m_tiles;
      out.group = c.group;
      out.row0 = c.row_begin + mt * tile_rows;
      out.row_end = c.row_end;
      out.n0 = nt * bn_out;
      return true;
    }
    c.base += tiles_here;
    c.group += 1;
    if (c.group < num_groups) cursor_load(c, off, tile_rows);
  }
  return false;
}

}  // namespace tc
}  // namespace atenia
