// Row placement of the direct (peer-store) expert-parallel exchange, written once for host and device.
//
// counts_all[p * E + e] = rows rank p holds for expert e, in p's dispatch order (sorted by expert, so
// the rows for one owner rank are contiguous).  Expert e lives on rank e / (E / world).  The receive
// buffer of a rank is laid out [local expert j][source rank p][rows]: all rows of one expert are
// contiguous, so the grouped GEMM runs one group per local expert whatever the number of ranks.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ATENIA_HD __host__ __device__
#else
#define ATENIA_HD
#endif

namespace atenia {

// For the calling rank (El = E / world):
//   dst_base[e]               first row, in the receive buffer of e's owner, of the rows this rank holds for e
//   gemm_offsets[j]           first row of local expert j in this rank's own receive buffer (El + 1 entries)
//   sub_offsets[j*world + p]  first row of the rows rank p sent for local expert j (El * world + 1 entries)
//   src_base[j*world + p]     first row of those rows in rank p's dispatch-ordered buffers, where the
//                             results go back to
// Entry i in [0, E) of the plan: dst_base[i], and the slice (j, p) = (i / world, i % world) of this
// rank's receive buffer (E = El * world, so one index covers both).  Entries are independent: the
// device computes them with one thread each, the host in a loop.
ATENIA_HD inline void ep_direct_plan_entry(const int32_t* counts_all, int world, int E, int rank, int i,
                                           int32_t* dst_base, int32_t* src_base, int32_t* sub_offsets,
                                           int32_t* gemm_offsets) {
  const int El = E / world;
  {
    const int owner = i / El;
    int run = 0;
    for (int e = owner * El; e < i; ++e)
      for (int p = 0; p < world; ++p) run += counts_all[p * E + e];
    int before = 0;
    for (int p = 0; p < rank; ++p) before += counts_all[p * E + i];
    dst_base[i] = run + before;
  }
  {
    const int j = i / world, p = i - j * world;
    const int e = rank * El + j;
    int run = 0;
    for (int jj = 0; jj < j; ++jj)
      for (int pp = 0; pp < world; ++pp) run += counts_all[pp * E + rank * El + jj];
    int within = 0;
    for (int pp = 0; pp < p; ++pp) within += counts_all[pp * E + e];
    int src = 0;
    for (int e2 = 0; e2 < e; ++e2) src += counts_all[p * E + e2];
    sub_offsets[i] = run + within;
    src_base[i] = src;
    if (p == 0) gemm_offsets[j] = run;
    if (i == E - 1) {
      const int total = run + within + counts_all[p * E + e];
      gemm_offsets[El] = total;
      sub_offsets[E] = total;
    }
  }
}

ATENIA_HD inline void ep_direct_plan(const int32_t* counts_all, int world, int E, int rank, int32_t* dst_base,
                                     int32_t* src_base, int32_t* sub_offsets, int32_t* gemm_offsets) {
  for (int i = 0; i < E; ++i)
    ep_direct_plan_entry(counts_all, world, E, rank, i, dst_base, src_base, sub_offsets, gemm_offsets);
}

}  // namespace atenia
