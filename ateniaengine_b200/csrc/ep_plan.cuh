// Row placement of the direct (peer-store) expert-parallel exchange, written once for host and device.
//
// counts_all[p * E + e] = rows rank p holds for expert e, in p's dispatch order (sorted by expert, so
// the rows for one owner rank are contiguous).  Expert e lives on rank e / (E / world).  The receive
// buffer of a rank is laid out [source rank p][local expert j][rows], which is the group order of its
// grouped GEMM.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ATENIA_HD __host__ __device__
#else
#define ATENIA_HD
#endif

namespace atenia {

// For the calling rank:
//   dst_base[e]            first row, in the receive buffer of e's owner, of the rows this rank holds for e
//   group_offsets[p*El+j]  first row of group (p, j) in this rank's own receive buffer (+ total at the end)
//   src_base[p*El+j]       first row of that group's rows in rank p's dispatch-ordered buffers, where
//                          the results go back to
ATENIA_HD inline void ep_direct_plan(const int32_t* counts_all, int world, int E, int rank, int32_t* dst_base,
                                     int32_t* src_base, int32_t* group_offsets) {
  const int El = E / world;
  for (int r = 0; r < world; ++r) {
    int run = 0;
    for (int p = 0; p < rank; ++p)
      for (int j = 0; j < El; ++j) run += counts_all[p * E + r * El + j];
    for (int j = 0; j < El; ++j) {
      dst_base[r * El + j] = run;
      run += counts_all[rank * E + r * El + j];
    }
  }
  int run = 0;
  for (int p = 0; p < world; ++p) {
    int src = 0;
    for (int e = 0; e < rank * El; ++e) src += counts_all[p * E + e];
    for (int j = 0; j < El; ++j) {
      const int c = counts_all[p * E + rank * El + j];
      group_offsets[p * El + j] = run;
      src_base[p * El + j] = src;
      run += c;
      src += c;
    }
  }
  group_offsets[world * El] = run;
}

}  // namespace atenia
