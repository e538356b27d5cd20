/*
 * CPU oracle for the Atenia MoE block.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a from-scratch C restatement of the reference's CPU algorithm
 * for one MoE block (router -> softmax -> top-k -> SwiGLU experts -> weighted
 * combine -> shared expert).  It exists so that the CUDA path can be checked
 * against the reference's arithmetic on a machine that has no Rust toolchain.
 * Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
 * load it; the product library never links, loads or calls it.
 *
 * Parity status: PINNED.  The restatement reproduces the reference's committed
 * golden vectors (fixtures/moe/{mixtral,qwen15_moe,qwen2_moe,qwen3_moe}_layer0,
 * deepseek_block) and the known-answer unit tests of src/moe/sparse.rs and
 * src/moe/dense.rs; tests/test_oracle_golden.py asserts that.  The INT8 block
 * output has no golden vector in the reference, so for INT8 the oracle is pinned
 * only through the quantiser's round-trip properties (src/tensor/disk_tier.rs:1310-1334).
 *
 * Each function cites the reference file:line it follows (paths relative to the
 * reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { ORACLE_W_F32 = 0, ORACLE_W_BF16 = 1, ORACLE_W_INT8_ROW = 2 };
enum { ORACLE_ACC_F64 = 0, ORACLE_ACC_F32 = 1 };

/* One weight matrix, row-major [rows, cols].  For INT8 `scales` has one f32 per row. */
typedef struct {
  const void* data;
  const float* scales;
} OracleMat;

typedef struct {
  int32_t num_experts;
  int32_t top_k;
  int32_t d_model;
  int32_t d_ff;
  int32_t shared_d_ff;  /* 0 = no shared expert */
  int32_t renormalize;  /* 1 = selected weights divided by their sum */
  int32_t shared_gated; /* 1 = shared output scaled by sigmoid(g.x) */
  int32_t weight_kind;  /* ORACLE_W_* for expert matrices (router is always f32) */
  int32_t accum;        /* ORACLE_ACC_* for the expert matvecs (router is always f64) */
  int32_t router_mode;  /* 0 softmax + top-k, 1 DeepSeek-V3 routing (renormalize = norm_topk_prob) */
  int32_t n_group;
  int32_t topk_group;
  double scaling;       /* routed_scaling_factor */
} OracleConfig;

typedef struct {
  const float* w_router;    /* [E, d] */
  const float* router_bias; /* [E] or NULL; synthetic skew, added in f64 before the f32 rounding */
  const OracleMat* gate;    /* [E] each [F, d] */
  const OracleMat* up;      /* [E] each [F, d] */
  const OracleMat* down;    /* [E] each [d, F] */
  OracleMat shared_gate_proj; /* [Fs, d] */
  OracleMat shared_up_proj;   /* [Fs, d] */
  OracleMat shared_down_proj; /* [d, Fs] */
  const float* shared_gate;   /* [d] or NULL */
  const float* e_score_bias;  /* [E] or NULL (zeros): V3 e_score_correction_bias */
} OracleWeights;

/* bf16 is the high half of an f32: decode is bits << 16 (src/tensor/tensor.rs:294-308). */
static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = ((uint32_t)b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Element (r, c) of a matrix as the f32 value the reference would hold in RAM:
 * f32 as is; bf16 upcast (exact); int8 dequantised as (f32)q * scale[r]
 * (src/tensor/disk_tier.rs:249-259, materialised by src/moe/residency.rs:452-458). */
static inline float mat_at(const OracleMat* m, int kind, size_t r, size_t cols, size_t c) {
  size_t i = r * cols + c;
  switch (kind) {
    case ORACLE_W_BF16: return bf16_to_f32(((const uint16_t*)m->data)[i]);
    case ORACLE_W_INT8_ROW: return (float)((const int8_t*)m->data)[i] * m->scales[r];
    default: return ((const float*)m->data)[i];
  }
}

/* Fetch a row as f32 into `dst` (so the inner loops run on plain floats). */
static void mat_row(const OracleMat* m, int kind, size_t r, size_t cols, float* dst) {
  switch (kind) {
    case ORACLE_W_BF16: {
      const uint16_t* p = (const uint16_t*)m->data + r * cols;
      for (size_t c = 0; c < cols; ++c) dst[c] = bf16_to_f32(p[c]);
      break;
    }
    case ORACLE_W_INT8_ROW: {
      const int8_t* p = (const int8_t*)m->data + r * cols;
      float s = m->scales[r];
      for (size_t c = 0; c < cols; ++c) dst[c] = (float)p[c] * s;
      break;
    }
    default:
      memcpy(dst, (const float*)m->data + r * cols, cols * sizeof(float));
  }
}

/* y = W.x, sequential accumulation over c ascending per output row.
 * accum f64: src/moe/dense.rs:97-115 (acc += (f64)w * (f64)x; y = (f32)acc).
 * accum f32: src/moe/dense.rs:120-138 (acc += w * x in f32, unfused).
 * Rows are processed four at a time; each row keeps its own accumulator and its
 * own ascending-c order, so every y[r] is the value the serial loop gives.
 * The f64 product of two f32 values is exact, so fma() equals multiply-then-add. */
#define RB 4
static void matvec_mat(const OracleMat* m, int kind, int accum, size_t rows, size_t cols,
                       const float* x, float* y, float* scratch /* RB*cols */) {
  size_t r = 0;
  for (; r < rows; r += RB) {
    size_t nb = rows - r < RB ? rows - r : RB;
    const float* rowp[RB];
    for (size_t j = 0; j < RB; ++j) {
      size_t rr = j < nb ? r + j : r;
      if (kind == ORACLE_W_F32) {
        rowp[j] = (const float*)m->data + rr * cols;
      } else {
        if (j < nb) mat_row(m, kind, rr, cols, scratch + j * cols);
        rowp[j] = scratch + (j < nb ? j : 0) * cols;
      }
    }
    if (accum == ORACLE_ACC_F64) {
      double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
      const float *p0 = rowp[0], *p1 = rowp[1], *p2 = rowp[2], *p3 = rowp[3];
      for (size_t c = 0; c < cols; ++c) {
        double xc = (double)x[c];
        a0 = fma((double)p0[c], xc, a0);
        a1 = fma((double)p1[c], xc, a1);
        a2 = fma((double)p2[c], xc, a2);
        a3 = fma((double)p3[c], xc, a3);
      }
      double a[RB] = {a0, a1, a2, a3};
      for (size_t j = 0; j < nb; ++j) y[r + j] = (float)a[j];
    } else {
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float *p0 = rowp[0], *p1 = rowp[1], *p2 = rowp[2], *p3 = rowp[3];
      for (size_t c = 0; c < cols; ++c) {
        float xc = x[c];
        float t0 = p0[c] * xc, t1 = p1[c] * xc, t2 = p2[c] * xc, t3 = p3[c] * xc;
        a0 = a0 + t0;
        a1 = a1 + t1;
        a2 = a2 + t2;
        a3 = a3 + t3;
      }
      float a[RB] = {a0, a1, a2, a3};
      for (size_t j = 0; j < nb; ++j) y[r + j] = a[j];
    }
  }
}

/* src/moe/dense.rs:74-77 */
static inline float silu_ref(float x) {
  double xd = (double)x;
  return (float)(xd / (1.0 + exp(-xd)));
}

/* Router logits: src/moe/dense.rs:333 (matvec, always f64) with the optional
 * synthetic bias folded in as one more f64 term before the f32 rounding. */
ORACLE_API void oracle_router_logits(const float* w_router, const float* bias, int E, int d,
                                     const float* x, float* logits) {
  for (int e = 0; e < E; ++e) {
    double acc = 0.0;
    const float* w = w_router + (size_t)e * d;
    for (int c = 0; c < d; ++c) acc += (double)w[c] * (double)x[c];
    if (bias) acc += (double)bias[e];
    logits[e] = (float)acc;
  }
}

/* src/moe/dense.rs:172-187.  The subtraction v - max is done in f32. */
ORACLE_API void oracle_softmax(const float* logits, int n, float* out) {
  if (n <= 0) return;
  float mx = -INFINITY;
  for (int i = 0; i < n; ++i) mx = fmaxf(mx, logits[i]);
  double* e = (double*)malloc(sizeof(double) * (size_t)n);
  double sum = 0.0;
  for (int i = 0; i < n; ++i) {
    float dlt = logits[i] - mx;
    e[i] = exp((double)dlt);
  }
  for (int i = 0; i < n; ++i) sum += e[i];
  double inv = sum > 0.0 ? 1.0 / sum : 0.0;
  for (int i = 0; i < n; ++i) out[i] = (float)(e[i] * inv);
  free(e);
}

/* src/moe/sparse.rs:142-191.  Returns 0, or a negative code:
 * -1 k == 0, -2 k > n, -3 non-finite weight, -4 negative weight, -5 selected sum <= 0. */
ORACLE_API int oracle_top_k(const float* weights, int n, int k, int renormalize,
                            int32_t* idx_out, float* w_out) {
  if (k <= 0 || n <= 0) return -1;
  if (k > n) return -2;
  for (int i = 0; i < n; ++i) {
    if (!isfinite(weights[i])) return -3;
    if (weights[i] < 0.0f) return -4;
  }
  /* order by (weight desc, index asc): repeated selection of the best unused entry */
  uint8_t* used = (uint8_t*)calloc((size_t)n, 1);
  for (int s = 0; s < k; ++s) {
    int best = -1;
    for (int i = 0; i < n; ++i) {
      if (used[i]) continue;
      if (best < 0 || weights[i] > weights[best]) best = i; /* strict >: ties keep the lower index */
    }
    used[best] = 1;
  }
  int m = 0;
  for (int i = 0; i < n; ++i)
    if (used[i]) idx_out[m++] = i; /* ascending */
  free(used);
  double sum = 0.0;
  for (int s = 0; s < k; ++s) sum += (double)weights[idx_out[s]];
  if (sum <= 0.0) return -5;
  double scale = renormalize ? 1.0 / sum : 1.0;
  for (int s = 0; s < k; ++s) w_out[s] = (float)((double)weights[idx_out[s]] * scale);
  return 0;
}

/* src/moe/dense.rs:253-270 */
static void expert_forward(const OracleMat* g, const OracleMat* u, const OracleMat* dn, int kind,
                           int accum, int d, int F, const float* x, float* y, float* gate,
                           float* up, float* h, float* scratch) {
  matvec_mat(g, kind, accum, (size_t)F, (size_t)d, x, gate, scratch);
  matvec_mat(u, kind, accum, (size_t)F, (size_t)d, x, up, scratch);
  for (int i = 0; i < F; ++i) h[i] = silu_ref(gate[i]) * up[i];
  matvec_mat(dn, kind, accum, (size_t)d, (size_t)F, h, y, scratch);
}

/* src/moe/layer.rs:436-443 */
static float sigmoid_dot(const float* g, const float* x, int n) {
  double acc = 0.0;
  for (int i = 0; i < n; ++i) acc += (double)g[i] * (double)x[i];
  return (float)(1.0 / (1.0 + exp(-acc)));
}

ORACLE_API int oracle_v3_route(const float* logits, const float* bias, int n, int top_k, int n_group,
                               int topk_group, double scaling, int norm_topk_prob, int32_t* idx_out,
                               float* w_out, float* dense_out);

/* One token: src/moe/layer.rs:405-431 over src/moe/sparse.rs:218-238. */
static int token_forward(const OracleConfig* c, const OracleWeights* w, const float* x, float* out,
                         int32_t* idx, float* tw, float* logits, float* buf) {
  const int E = c->num_experts, k = c->top_k, d = c->d_model, F = c->d_ff, Fs = c->shared_d_ff;
  int Fmax = F > Fs ? F : Fs;
  int cmax = d > Fmax ? d : Fmax;
  float* probs = buf;               /* E */
  float* y = probs + E;             /* d */
  float* gate = y + d;              /* Fmax */
  float* up = gate + Fmax;          /* Fmax */
  float* h = up + Fmax;             /* Fmax */
  float* scratch = h + Fmax;        /* RB * cmax */
  (void)cmax;
  oracle_router_logits(w->w_router, w->router_bias, E, d, x, logits);
  int rc;
  if (c->router_mode == 1) {
    /* V3: logits exclude the synthetic bias; selection bias is e_score_bias (zeros when absent) */
    for (int e = 0; e < E; ++e) probs[e] = w->e_score_bias ? w->e_score_bias[e] : 0.0f;
    rc = oracle_v3_route(logits, probs, E, k, c->n_group, c->topk_group, c->scaling, c->renormalize, idx, tw, NULL);
  } else {
    oracle_softmax(logits, E, probs);
    rc = oracle_top_k(probs, E, k, c->renormalize, idx, tw);
  }
  if (rc) return rc;
  for (int i = 0; i < d; ++i) out[i] = 0.0f;
  for (int s = 0; s < k; ++s) {
    int e = idx[s];
    expert_forward(&w->gate[e], &w->up[e], &w->down[e], c->weight_kind, c->accum, d, F, x, y, gate,
                   up, h, scratch);
    float ws = tw[s];
    for (int i = 0; i < d; ++i) {
      float t = ws * y[i];
      out[i] = out[i] + t;
    }
  }
  if (Fs > 0) {
    expert_forward(&w->shared_gate_proj, &w->shared_up_proj, &w->shared_down_proj, c->weight_kind,
                   c->accum, d, Fs, x, y, gate, up, h, scratch);
    float scale = 1.0f;
    if (c->shared_gated && w->shared_gate) scale = sigmoid_dot(w->shared_gate, x, d);
    for (int i = 0; i < d; ++i) {
      float t = scale * y[i];
      out[i] = out[i] + t;
    }
  }
  return 0;
}

/* The operator: a flat [T*d] batch applied row by row (src/moe/graph_op.rs:327-350).
 * Rows are independent, so they run on `nthreads` host threads (the reference
 * parallelises inside a matvec with rayon, src/moe/dense.rs:106-108; the result
 * of either split is the same).  Optional outputs may be NULL.
 * Returns 0, or the first token's negative top-k error code. */
ORACLE_API int oracle_moe_forward(const OracleConfig* c, const OracleWeights* w, const float* x,
                                  int T, float* out, int32_t* topk_idx, float* topk_w,
                                  float* logits, int nthreads) {
  const int E = c->num_experts, k = c->top_k, d = c->d_model;
  int Fmax = c->d_ff > c->shared_d_ff ? c->d_ff : c->shared_d_ff;
  int cmax = d > Fmax ? d : Fmax;
  size_t per = (size_t)E + d + 3 * (size_t)Fmax + (size_t)RB * cmax + (size_t)E + 2 * (size_t)k + 64;
  int status = 0;
#ifdef _OPENMP
  if (nthreads <= 0) nthreads = omp_get_max_threads();
#else
  nthreads = 1;
#endif
#pragma omp parallel num_threads(nthreads)
  {
    float* buf = (float*)malloc(per * sizeof(float));
    float* lg = buf + (E + d + 3 * (size_t)Fmax + (size_t)RB * cmax);
    float* twl = lg + E;
    int32_t* idl = (int32_t*)(twl + k);
#pragma omp for schedule(dynamic, 1)
    for (int t = 0; t < T; ++t) {
      int rc = token_forward(c, w, x + (size_t)t * d, out + (size_t)t * d, idl, twl, lg, buf);
      if (rc) {
#pragma omp critical
        if (!status) status = rc;
        continue;
      }
      if (topk_idx) memcpy(topk_idx + (size_t)t * k, idl, sizeof(int32_t) * (size_t)k);
      if (topk_w) memcpy(topk_w + (size_t)t * k, twl, sizeof(float) * (size_t)k);
      if (logits) memcpy(logits + (size_t)t * E, lg, sizeof(float) * (size_t)E);
    }
    free(buf);
  }
  return status;
}

/* Routing only, from given logits (softmax + top-k per token). */
ORACLE_API int oracle_route_from_logits(const float* logits, int T, int E, int k, int renormalize,
                                        int32_t* topk_idx, float* topk_w) {
  float* probs = (float*)malloc(sizeof(float) * (size_t)E);
  int status = 0;
  for (int t = 0; t < T && !status; ++t) {
    oracle_softmax(logits + (size_t)t * E, E, probs);
    status = oracle_top_k(probs, E, k, renormalize, topk_idx + (size_t)t * k, topk_w + (size_t)t * k);
  }
  free(probs);
  return status;
}

/* Canonical dispatch permutation.  The reference never builds one (it loops
 * token by token, src/moe/graph_op.rs:346-348, experts ascending per token,
 * src/moe/sparse.rs:173-175); the only order it defines is tokens ascending and
 * selected experts ascending inside a token.  The permutation is therefore the
 * stable counting sort of the flat (token, slot) list by expert id:
 * expert_offsets[e] = rows of experts < e; perm[row] = t*k + s. */
ORACLE_API void oracle_dispatch_permutation(const int32_t* topk_idx, int T, int k, int E,
                                            int32_t* expert_offsets /* E+1 */,
                                            int32_t* perm /* T*k */, int32_t* inv_perm /* T*k */) {
  size_t n = (size_t)T * k;
  int32_t* cursor = (int32_t*)calloc((size_t)E + 1, sizeof(int32_t));
  for (int e = 0; e <= E; ++e) expert_offsets[e] = 0;
  for (size_t i = 0; i < n; ++i) expert_offsets[topk_idx[i] + 1]++;
  for (int e = 0; e < E; ++e) expert_offsets[e + 1] += expert_offsets[e];
  for (int e = 0; e < E; ++e) cursor[e] = expert_offsets[e];
  for (size_t i = 0; i < n; ++i) {
    int32_t pos = cursor[topk_idx[i]]++;
    perm[pos] = (int32_t)i;
    if (inv_perm) inv_perm[i] = pos;
  }
  free(cursor);
}

/* Rust f32::round: half away from zero. */
static inline float round_half_away(float v) { return roundf(v); }

/* src/tensor/disk_tier.rs:231-245 */
ORACLE_API void oracle_quantize_per_row_i8(const float* data, size_t rows, size_t cols, int8_t* q,
                                           float* scales) {
  for (size_t r = 0; r < rows; ++r) {
    const float* row = data + r * cols;
    float amax = 0.0f;
    for (size_t c = 0; c < cols; ++c) amax = fmaxf(amax, fabsf(row[c]));
    float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
    scales[r] = scale;
    float inv = 1.0f / scale;
    for (size_t c = 0; c < cols; ++c) {
      float v = round_half_away(row[c] * inv);
      if (v < -127.0f) v = -127.0f;
      if (v > 127.0f) v = 127.0f;
      q[r * cols + c] = (int8_t)v;
    }
  }
}

/* src/tensor/disk_tier.rs:249-259 */
ORACLE_API void oracle_dequantize_per_row_i8(const int8_t* q, const float* scales, size_t rows,
                                             size_t cols, float* out) {
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) out[r * cols + c] = (float)q[r * cols + c] * scales[r];
}

/* Dense W8A16 quantiser: weight [K, N] row-major, one scale per (group of `group_size` consecutive
 * rows, column).  src/tensor/quantizer.rs:67-118 (per channel = one group of K rows) and :176-246
 * (per group).  scale = max(amax/127, 1e-12); q = clamp(round_half_away(w / scale), -127, 127) with
 * a true division; a NaN quotient becomes 0 (Rust's saturating `as i32`).  `v > max` skips NaNs. */
ORACLE_API void oracle_absmax_per_group_symmetric(const float* w, size_t K, size_t N, size_t group_size,
                                                  int8_t* q, float* scales) {
  if (K == 0 || N == 0 || group_size == 0) return;
  const size_t groups = (K + group_size - 1) / group_size;
  for (size_t g = 0; g < groups; ++g) {
    const size_t lo = g * group_size, hi = (g + 1) * group_size < K ? (g + 1) * group_size : K;
    for (size_t c = 0; c < N; ++c) {
      float amax = 0.0f;
      for (size_t r = lo; r < hi; ++r) {
        const float v = fabsf(w[r * N + c]);
        if (v > amax) amax = v;
      }
      float sc = amax / 127.0f;
      if (!(sc >= 1e-12f)) sc = 1e-12f; /* f32::max(1e-12); amax is never NaN here */
      scales[g * N + c] = sc;
    }
  }
  for (size_t r = 0; r < K; ++r) {
    const float* srow = scales + (r / group_size) * N;
    for (size_t c = 0; c < N; ++c) {
      float v = round_half_away(w[r * N + c] / srow[c]);
      if (v != v) {
        q[r * N + c] = 0;
        continue;
      }
      if (v < -127.0f) v = -127.0f;
      if (v > 127.0f) v = 127.0f;
      q[r * N + c] = (int8_t)(int32_t)v;
    }
  }
}

/* The reference's materialising dequant: bf16 = high 16 bits of (float)q * scale[group, col]
 * (truncation).  src/cuda/int8_to_bf16.cu:24-40 (per channel) and :99-117 (per group). */
ORACLE_API void oracle_int8_to_bf16_per_group(const int8_t* q, const float* scales, size_t K, size_t N,
                                              size_t group_size, uint16_t* out) {
  if (group_size == 0) return;
  for (size_t r = 0; r < K; ++r)
    for (size_t c = 0; c < N; ++c) {
      const float f = (float)q[r * N + c] * scales[(r / group_size) * N + c];
      uint32_t bits;
      memcpy(&bits, &f, 4);
      out[r * N + c] = (uint16_t)(bits >> 16);
    }
}

/* src/moe/sparse.rs:87-116 */
ORACLE_API int oracle_combine_selected(const int32_t* indices, const float* weights, int k,
                                       const float* expert_outputs, size_t n_outputs, int d,
                                       float* out) {
  for (int i = 0; i < d; ++i) out[i] = 0.0f;
  for (int s = 0; s < k; ++s) {
    size_t base = (size_t)indices[s] * d;
    if (base + d > n_outputs) return -1;
    float w = weights[s];
    for (int i = 0; i < d; ++i) {
      float t = w * expert_outputs[base + i];
      out[i] = out[i] + t;
    }
  }
  return 0;
}

/* DeepSeek-V3 routing for one token: src/moe/v3_router.rs:206-309.
 * scores = sigmoid(logits) in f64; choice = scores + bias; group score = sum of the two largest
 * choices of a group; the topk_group best groups stay eligible (ties: lower group); top_k experts by
 * choice among them (ties: lower index; -inf only if nothing else is left); combine weights are the
 * ORIGINAL scores, divided by (their sum + 1e-20) when norm_topk_prob, times routed_scaling_factor.
 * Outputs: idx_out ascending, w_out f32, dense_out[n] (may be NULL).  Returns 0 or a negative code:
 * -1 zero parameter, -2 n % n_group, -3 group < 2 experts, -4 topk_group > n_group,
 * -5 top_k > selectable, -6 non-finite input. */
static void v3_top_k(const double* score, int n, int k, int* out) {
  uint8_t* used = (uint8_t*)calloc((size_t)n, 1);
  for (int s = 0; s < k; ++s) {
    int best = -1;
    for (int i = 0; i < n; ++i) {
      if (used[i]) continue;
      if (best < 0 || score[i] > score[best]) best = i; /* strict >: ties keep the lower index */
    }
    used[best] = 1;
    out[s] = best;
  }
  free(used);
}

ORACLE_API int oracle_v3_route(const float* logits, const float* bias, int n, int top_k, int n_group,
                               int topk_group, double scaling, int norm_topk_prob, int32_t* idx_out,
                               float* w_out, float* dense_out) {
  if (top_k <= 0 || n_group <= 0 || topk_group <= 0) return -1;
  if (n % n_group) return -2;
  const int epg = n / n_group;
  if (epg < 2) return -3;
  if (topk_group > n_group) return -4;
  if (top_k > topk_group * epg) return -5;
  for (int i = 0; i < n; ++i)
    if (!isfinite(logits[i]) || !isfinite(bias[i])) return -6;
  double* scores = (double*)malloc(sizeof(double) * (size_t)n * 3);
  double* choice = scores + n;
  double* masked = choice + n;
  for (int i = 0; i < n; ++i) {
    scores[i] = 1.0 / (1.0 + exp(-(double)logits[i]));
    choice[i] = scores[i] + (double)bias[i];
  }
  double* gscore = (double*)malloc(sizeof(double) * (size_t)n_group);
  int* gsel = (int*)malloc(sizeof(int) * (size_t)(topk_group + top_k));
  int* esel = gsel + topk_group;
  for (int g = 0; g < n_group; ++g) {
    double a = -INFINITY, b = -INFINITY; /* two largest, a >= b */
    for (int j = 0; j < epg; ++j) {
      double v = choice[g * epg + j];
      if (v > a) {
        b = a;
        a = v;
      } else if (v > b) {
        b = v;
      }
    }
    gscore[g] = a + b;
  }
  v3_top_k(gscore, n_group, topk_group, gsel);
  for (int i = 0; i < n; ++i) masked[i] = -INFINITY;
  for (int s = 0; s < topk_group; ++s)
    for (int j = 0; j < epg; ++j) masked[gsel[s] * epg + j] = choice[gsel[s] * epg + j];
  v3_top_k(masked, n, top_k, esel);
  /* ascending indices */
  for (int a = 1; a < top_k; ++a) {
    int v = esel[a], b = a - 1;
    while (b >= 0 && esel[b] > v) {
      esel[b + 1] = esel[b];
      --b;
    }
    esel[b + 1] = v;
  }
  double denom = 0.0;
  for (int s = 0; s < top_k; ++s) denom += scores[esel[s]];
  denom += 1e-20;
  if (dense_out)
    for (int i = 0; i < n; ++i) dense_out[i] = 0.0f;
  for (int s = 0; s < top_k; ++s) {
    double w = scores[esel[s]];
    if (norm_topk_prob) w /= denom;
    w *= scaling;
    idx_out[s] = esel[s];
    w_out[s] = (float)w;
    if (dense_out) dense_out[esel[s]] = (float)w;
  }
  free(gsel);
  free(gscore);
  free(scores);
  return 0;
}

/* One expert's forward for one token (src/moe/dense.rs:253-270), f32 weights, exported for tests
 * that compose a block from routing weights themselves. */
ORACLE_API void oracle_expert_forward_f32(const float* w_gate, const float* w_up, const float* w_down, int d,
                                          int F, int accum, const float* x, float* y) {
  OracleMat g = {w_gate, NULL}, u = {w_up, NULL}, dn = {w_down, NULL};
  int cmax = d > F ? d : F;
  float* buf = (float*)malloc(sizeof(float) * ((size_t)3 * F + (size_t)RB * cmax));
  expert_forward(&g, &u, &dn, ORACLE_W_F32, accum, d, F, x, y, buf, buf + F, buf + 2 * F, buf + 3 * F);
  free(buf);
}

ORACLE_API float oracle_mat_at(const OracleMat* m, int kind, size_t r, size_t cols, size_t c) {
  return mat_at(m, kind, r, cols, c);
}

ORACLE_API int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Post-attention RMSNorm and its gain, as applied before the MoE block: rms_norm
 * (src/nn/normalization.rs:8-37: f32 sum of squares in index order, mean over the row, 1 / sqrt(mean +
 * eps), x * inv_rms) followed by broadcast_mul with gamma (src/moe/full_forward.rs:239-242).
 * gamma may be NULL (unit gain). */
ORACLE_API void oracle_rms_norm_gamma(const float* x, int T, int d, const float* gamma, float eps, float* out) {
  for (int t = 0; t < T; ++t) {
    const float* row = x + (size_t)t * d;
    float sum_sq = 0.0f;
    for (int i = 0; i < d; ++i) sum_sq += row[i] * row[i];
    const float cols = d > 1 ? (float)d : 1.0f;
    const float mean_sq = sum_sq / cols;
    const float inv_rms = 1.0f / sqrtf(mean_sq + eps);
    for (int i = 0; i < d; ++i) {
      const float n = row[i] * inv_rms;
      out[(size_t)t * d + i] = gamma ? n * gamma[i] : n;
    }
  }
}

