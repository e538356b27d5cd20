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
ATENIA_HD inline void ep_direct_plan(const int32_t* counts_all, int world, int E, int rank, int32_t* dst_base,
                                     int32_t* src_base, int32_t* sub_offsets, int32_t* gemm_offsets) {
  const int El = E / world;
  for (int r = 0; r < world; ++r) {
    int run = 0;
    for (int j = 0; j < El; ++j) {
      const int e = r * El + j;
      int before = 0;
      for (int p = 0; p < rank; ++p) before += counts_all[p * E + e];
      dst_base[e] = run + before;
      for (int p = 0; p < world; ++p) run += counts_all[p * E + e];
    }
  }
  int run = 0;
  for (int j = 0; j < El; ++j) {
    const int e = rank * El + j;
    gemm_offsets[j] = run;
    for (int p = 0; p < world; ++p) {
      int src = 0;
      for (int e2 = 0; e2 < e; ++e2) src += counts_all[p * E + e2];
      sub_offsets[j * world + p] = run;
      src_base[j * world + p] = src;
      run += counts_all[p * E + e];
    }
  }
  gemm_offsets[El] = run;
  sub_offsets[El * world] = run;
}

}  // namespace atenia
