// Test-only: compiles the device routing function of the library with a host compiler so that the
// CPU test-suite can run the very same code against the oracle.  Not part of the product library.
#include "../ateniaengine_b200/csrc/v3_route.cuh"

extern "C" int v3_probe_route(const float* logits, const float* bias, int n, int top_k, int n_group, int topk_group,
                              int norm, double scaling, int32_t* idx, float* w) {
  atenia::V3RouteParams p{n, top_k, n_group, topk_group, norm, scaling};
  int rc = atenia::v3_validate(p);
  if (rc) return rc;
  double scores[atenia::kV3MaxExperts], choice[atenia::kV3MaxExperts];
  return atenia::v3_route_one(logits, bias, p, idx, w, scores, choice);
}
