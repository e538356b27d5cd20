// DeepSeek-V3 routing of one token (src/moe/v3_router.rs:206-309), written once for device and host:
// the CUDA kernel in router.cu calls it per thread, and the CPU test-suite compiles this header with
// a host compiler to check the very same code against the oracle.
//
//   scores  = sigmoid(logits) in f64;  choice = scores + bias  (the bias steers selection only)
//   group score = sum of the two largest choices of a group; the topk_group best groups stay eligible
//   top_k experts by choice among the eligible ones; ties go to the lower index everywhere
//   weights = ORIGINAL scores, / (their sum + 1e-20) when norm_topk_prob, * routed_scaling_factor
#pragma once
#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define ATENIA_HD __host__ __device__
#else
#define ATENIA_HD
#endif

namespace atenia {

struct V3RouteParams {
  int n;           // routed experts
  int top_k;
  int n_group;
  int topk_group;
  int norm_topk_prob;
  double scaling;  // routed_scaling_factor
};

constexpr int kV3MaxExperts = 128;
constexpr int kV3MaxTopK = 8;

// V3RouterConfig::validate (src/moe/v3_router.rs:150-183).  0 = valid.
ATENIA_HD inline int v3_validate(const V3RouteParams& p) {
  if (p.top_k <= 0 || p.n_group <= 0 || p.topk_group <= 0 || p.n <= 0) return -1;
  if (p.n % p.n_group) return -2;
  const int epg = p.n / p.n_group;
  if (epg < 2) return -3;
  if (p.topk_group > p.n_group) return -4;
  if (p.top_k > p.topk_group * epg) return -5;
  if (p.n > kV3MaxExperts || p.top_k > kV3MaxTopK) return -7;
  return 0;
}

// Routes one token.  `scores` and `choice` are caller-provided scratch of n doubles each.
// Writes top_k ascending indices and their f32 weights.  Returns 0, or -6 for a non-finite input.
ATENIA_HD inline int v3_route_one(const float* logits, const float* bias, const V3RouteParams& p, int32_t* idx_out,
                                  float* w_out, double* scores, double* choice) {
  const int n = p.n, epg = p.n / p.n_group;
  for (int i = 0; i < n; ++i) {
    const float l = logits[i], b = bias[i];
    if (!(l - l == 0.0f) || !(b - b == 0.0f)) return -6;  // NaN or infinity
    scores[i] = 1.0 / (1.0 + exp(-(double)l));
    choice[i] = scores[i] + (double)b;
  }
  // eligible groups: topk_group rounds of "largest group score, lowest index"
  unsigned long long group_taken = 0ull;  // n_group <= 64 (n <= 128, >= 2 experts per group)
  for (int s = 0; s < p.topk_group; ++s) {
    int best = -1;
    double best_v = 0.0;
    for (int g = 0; g < p.n_group; ++g) {
      if ((group_taken >> g) & 1ull) continue;
      double a = -INFINITY, b2 = -INFINITY;  // the two largest choices of the group
      for (int j = 0; j < epg; ++j) {
        const double v = choice[g * epg + j];
        if (v > a) {
          b2 = a;
          a = v;
        } else if (v > b2) {
          b2 = v;
        }
      }
      const double gs = a + b2;
      if (best < 0 || gs > best_v) {
        best = g;
        best_v = gs;
      }
    }
    group_taken |= 1ull << best;
  }
  // top_k rounds of "largest choice among eligible, lowest index"; ineligible experts count as -inf
  // and are only reached when nothing else is left (validate() rules that out)
  unsigned long long taken[2] = {0ull, 0ull};
  for (int s = 0; s < p.top_k; ++s) {
    int best = -1;
    double best_v = 0.0;
    for (int i = 0; i < n; ++i) {
      if ((taken[i >> 6] >> (i & 63)) & 1ull) continue;
      const double v = ((group_taken >> (i / epg)) & 1ull) ? choice[i] : -INFINITY;
      if (best < 0 || v > best_v) {
        best = i;
        best_v = v;
      }
    }
    taken[best >> 6] |= 1ull << (best & 63);
  }
  double denom = 0.0;
  int m = 0;
  for (int i = 0; i < n; ++i)
    if ((taken[i >> 6] >> (i & 63)) & 1ull) {
      idx_out[m++] = i;  // ascending
      denom += scores[i];
    }
  denom += 1e-20;
  for (int s = 0; s < p.top_k; ++s) {
    double w = scores[idx_out[s]];
    if (p.norm_topk_prob) w /= denom;
    w *= p.scaling;
    w_out[s] = (float)w;
  }
  return 0;
}

}  // namespace atenia
