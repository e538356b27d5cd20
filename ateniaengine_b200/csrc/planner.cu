// Host-only parts of the C ABI: the expert-residency planner and the numeric-policy switch.
//
// Residency.  The reference keeps experts in a RAM/NVMe tier and sizes a per-layer LRU cache as
// clamp(budget / (layers * bytes_per_expert), 1, E) (auto_expert_cache_capacity,
// src/moe/residency.rs:201-211; resolved per model in src/moe/runtime.rs:559-584).  On a B200 the
// tier is HBM itself and the question becomes: do all experts of all layers fit one GPU, and if
// not, over how many expert-parallel ranks must they be sharded?  atenia_moe_plan_residency applies
// the reference's formula to what is left of the budget once the per-rank fixed costs (router,
// shared expert, workspace) are paid, for ep_world = 1, 2, 4, 8, and returns the smallest world in
// which every rank's share of the experts is resident.  It refuses a model that does not fit 8 ranks.
//
// Numeric policy.  The reference reads ATENIA_NUMERIC_POLICY = {certified, strict, fast}
// (src/moe/numeric_policy.rs:37-127) inside its expert matvec (src/moe/dense.rs:159-168): only Fast
// sends the contraction to the GPU, Certified (f64) and Strict (f32) stay on its own CPU arms, and
// the router is f64 under every policy.  This library IS the Fast arm.  The functions below restate
// the switch (same strings, same precedence: in-process override, then the environment read once,
// then Certified) so that a host can ask whether the library serves the active policy.
#include <algorithm>
#include <vector>
#include <atomic>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"

namespace atenia {
namespace {

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// cudaMalloc hands out 256-byte aligned blocks at least; count every buffer rounded up to that.
struct Tally {
  uint64_t total = 0;
  void add(uint64_t bytes) {
    if (bytes) total += align_up(bytes, 256);
  }
};

int valid_for_plan(const AteniaMoeConfig& c) {
  if (c.num_experts < 1 || c.num_experts > 128) return ATENIA_ERR_SHAPE;
  if (c.experts_per_token < 1 || c.experts_per_token > 8 || c.experts_per_token > c.num_experts)
    return ATENIA_ERR_SHAPE;
  if (c.d_model < 16 || c.d_model % 16 || c.d_ff < 16 || c.d_ff % 16) return ATENIA_ERR_SHAPE;
  if (c.shared_d_ff < 0 || c.shared_d_ff % 16) return ATENIA_ERR_SHAPE;
  if (c.weight_dtype != ATENIA_W_BF16 && c.weight_dtype != ATENIA_W_INT8_ROW) return ATENIA_ERR_SHAPE;
  if (c.max_tokens < 1) return ATENIA_ERR_SHAPE;
  return ATENIA_OK;
}

uint64_t matrix_bytes(uint64_t rows, uint64_t cols, bool int8) {
  // int8: one byte per weight plus one f32 scale per output row (src/tensor/disk_tier.rs:168-224)
  return int8 ? align_up(rows * cols, 256) + align_up(rows * 4, 256) : align_up(rows * cols * 2, 256);
}

}  // namespace

// Bytes atenia_moe_create allocates for a layer of this configuration (the list mirrors the
// allocations of moe_layer.cu; tests/test_residency_planner.py compares it with the free-memory
// delta of a real create).  `world` replaces cfg.ep_world.
uint64_t layer_workspace_bytes(const AteniaMoeConfig& c, int world) {
  const uint64_t Tm = (uint64_t)c.max_tokens, k = (uint64_t)c.experts_per_token, E = (uint64_t)c.num_experts;
  const uint64_t d = (uint64_t)c.d_model, F = (uint64_t)c.d_ff, Fs = (uint64_t)c.shared_d_ff;
  const uint64_t R = Tm * k;
  const uint64_t nblk = (R + kDispatchChunk - 1) / kDispatchChunk;
  const uint64_t groups = E;  // GEMM groups: E on one GPU, e_local * world = E under expert parallelism
  const bool q = c.weight_dtype == ATENIA_W_INT8_ROW;
  Tally t;
  t.add(E * d * 4);           // router copy
  t.add(E * 4);               // bias
  t.add(d * 4);               // gate vector
  if (c.router_mode == ATENIA_ROUTER_V3) {
    t.add(E * 4);
    t.add(Tm * E * 4);
  }
  t.add(R * 4);               // topk_idx
  t.add(R * 4);               // topk_w
  t.add(Tm * 4);              // gate_scale
  t.add(R * 4);               // perm
  t.add(R * 4);               // inv_perm
  t.add((E + 1) * 4);
  t.add(2 * 4);
  t.add(nblk * E * 4);
  t.add(nblk * E * 4);
  t.add(R * d * 2);           // x_perm
  t.add(R * d * 2);           // y_perm
  if (world == 1) t.add(R * F * 2);  // h
  t.add(Tm * d * 2);          // x_bf16
  if (Fs) {
    t.add(Tm * Fs * 2);
    t.add(Tm * d * 2);
  }
  t.add(8);                   // error word
  const uint64_t tm = 128;    // one CUtensorMap
  t.add(groups * tm);
  t.add(groups * tm);
  t.add(groups * tm);
  t.add(3 * tm);
  t.add((uint64_t)148 * 2 * kW8SplitKSlotFloats * 4);  // stream-K partial sums, one pair of slots per SM
  t.add((uint64_t)kSplitKMaxTiles * 8 * 4);            // arrival counters of split tiles
  if (q) {
    if (Fs) t.add((uint64_t)148 * 2 * kW8SplitKSlotFloats * 4);  // the same for the shared expert's launches
    for (int i = 0; i < 3; ++i) t.add(groups * tm);               // weight maps of the integer-MMA decode kernel
    const uint64_t pr = std::min<uint64_t>(kI8DecodeDefaultRows, (R + 15) / 16 * 16);
    t.add(4 * pr * d);                                            // digit planes of the token rows
    t.add(4 * pr * F);                                            // and of the intermediate rows
    t.add(pr * 4);
    t.add(pr * 4);
    t.add(groups * tm);
    t.add(groups * tm);
    t.add(groups * tm);
    t.add(3 * tm);
  }
  for (int i = 0; i < 3; ++i) t.add(groups * 8);  // scale pointer arrays
  t.add(3 * 8);
  for (int i = 0; i < 3; ++i) t.add(groups * 8);  // matrix pointer arrays
  t.add(3 * 8);
  if (world > 1) {
    const uint64_t RC = R * (uint64_t)world;  // worst case: every row of every rank lands here
    t.add(RC * d * 2);
    t.add(RC * F * 2);
    t.add(RC * d * 2);
    t.add((uint64_t)world * E * 4);
    t.add((groups + 1) * 4);
  }
  return t.total;
}


// ---- sub-batch schedule of the host-buffer operator -------------------------------------------------
// execute_real_moe_layer copies a batch in, runs it and copies the result out.  Cut into pieces, the copy
// in of piece i+1 and the copy out of piece i-1 overlap the forward of piece i (two staging buffers each
// way); what stays exposed is the first copy in and the last copy out, and every piece streams the expert
// weights again.  Which cut is best depends on whether the layer is slower than the PCIe link or faster,
// so it is chosen with a model: a forward of T tokens costs the touched expert weights at the HBM rate
// plus T times the flops of a token at the rate the grouped GEMMs sustain, a copy costs its bytes at the
// rate of a pinned host buffer.  Measured on B200 (Mixtral shape, 4096 tokens, host f32 buffers): one pass
// 4.68 ms, two halves 3.99 - 4.05 ms, quarters 4.32 ms, pieces of 768 / 2560 / 768 tokens 3.51 ms; a
// DeepSeek-V2-Lite-shaped layer at 8192 tokens is slower over PCIe than on the GPU and wants equal pieces
// (halves 2.55 ms, the three-piece cut above 2.82 ms).
constexpr double kModelHbmBytesPerMs = 6.5e9;     // streamed weights
constexpr double kModelFlopsPerMsBf16 = 1.5e12;   // grouped bf16 GEMMs beside the weight stream (1.7e12 fits a Mixtral-shaped layer, 1.3e12 a DeepSeek-shaped one)
constexpr double kModelFlopsPerMsInt8 = 1.2e12;   // W8A16: the widening kernels
constexpr double kModelPcieBytesPerMs = 53.0e6;   // pinned host memory, either direction
constexpr double kModelPieceOverheadMs = 0.06;    // routing, dispatch, combine, launch gaps of one forward
constexpr uint64_t kModelMinPiece = 256;          // smaller pieces: the line forward(T) = a + b T no longer holds

struct ExecModel {
  double expert_ms, shared_ms, token_ms, copy_token_ms;
  uint64_t E, k;
  bool fitted;         // forward(T) = fit_a + fit_b T from the operator's own timings
  double fit_a, fit_b;
};

ExecModel exec_model(const AteniaMoeConfig& c) {
  const double d = c.d_model, F = c.d_ff, Fs = c.shared_d_ff;
  const bool q = c.weight_dtype == ATENIA_W_INT8_ROW;
  const double wb = q ? 1.0 : 2.0;
  ExecModel m;
  m.expert_ms = 3.0 * F * d * wb / kModelHbmBytesPerMs;
  m.shared_ms = 3.0 * Fs * d * wb / kModelHbmBytesPerMs;
  m.token_ms = (c.experts_per_token * 6.0 * d * F + 6.0 * d * Fs) / (q ? kModelFlopsPerMsInt8 : kModelFlopsPerMsBf16);
  m.copy_token_ms = d * 4.0 / kModelPcieBytesPerMs;
  m.E = (uint64_t)c.num_experts;
  m.k = (uint64_t)c.experts_per_token;
  m.fitted = false;
  m.fit_a = m.fit_b = 0.0;
  return m;
}

double model_forward_ms(const ExecModel& m, uint64_t T) {
  if (m.fitted) return m.fit_a + m.fit_b * (double)T;
  const uint64_t touched = std::min<uint64_t>(m.E, T * m.k);
  return kModelPieceOverheadMs + (double)touched * m.expert_ms + m.shared_ms + (double)T * m.token_ms;
}

// End of the last copy out when `pieces` run through the two-buffer pipeline of execute_pipelined.
double model_pipeline_ms(const ExecModel& m, const std::vector<uint64_t>& pieces) {
  double h = 0.0, c = 0.0, o = 0.0;
  std::vector<double> fwd_done, out_done;
  for (size_t i = 0; i < pieces.size(); ++i) {
    const double copy = (double)pieces[i] * m.copy_token_ms;
    double hs = h;
    if (i >= 2) hs = std::max(hs, fwd_done[i - 2]);  // the input buffer is free again
    h = hs + copy;
    double cs = std::max(c, h);
    if (i >= 2) cs = std::max(cs, out_done[i - 2]);  // the output buffer is free again
    c = cs + model_forward_ms(m, pieces[i]);
    fwd_done.push_back(c);
    o = std::max(o, c) + copy;
    out_done.push_back(o);
  }
  return o;
}

// Pieces of a batch of n tokens, none above cap: p pieces, the two end ones of `end` tokens and the rest
// equal, over p = 1 .. 8 and end in steps of n / 32 (multiples of 64 tokens).  One piece means no overlap.
std::vector<uint64_t> plan_exec_pieces(const AteniaMoeConfig& c, uint64_t n, uint64_t cap, const ExecFit* fit) {
  std::vector<uint64_t> best;
  if (n == 0 || cap == 0) return best;
  ExecModel m = exec_model(c);
  if (fit && fit->valid) {
    m.fitted = true;
    m.fit_a = fit->a_ms;
    m.fit_b = fit->b_ms;
    m.copy_token_ms = fit->copy_token_ms;
  }
  double best_ms = 0.0;
  auto consider = [&](const std::vector<uint64_t>& pieces) {
    uint64_t sum = 0;
    for (uint64_t v : pieces) {
      if (v == 0 || v > cap) return;
      if (pieces.size() > 1 && v < kModelMinPiece) return;
      sum += v;
    }
    if (sum != n) return;
    const double ms = model_pipeline_ms(m, pieces);
    if (best.empty() || ms < best_ms * 0.99) {  // (more pieces must earn at least a percent)
      best = pieces;
      best_ms = ms;
    }
  };
  const uint64_t p_min = (n + cap - 1) / cap;
  for (uint64_t p = p_min; p <= p_min + 7; ++p) {
    if (p == 1) {
      consider({n});
      continue;
    }
    if (n < kModelMinPiece * p) break;
    const uint64_t step = std::max<uint64_t>(64, n / 32 / 64 * 64);
    if (p == 2) {
      consider({(n + 1) / 2, n / 2});
      continue;
    }
    for (uint64_t end = step; 2 * end < n; end += step) {
      const uint64_t mid_total = n - 2 * end, mids = p - 2;
      if (mid_total < mids) break;
      std::vector<uint64_t> pieces;
      pieces.push_back(end);
      for (uint64_t j = 0; j < mids; ++j) pieces.push_back(mid_total / mids + (j < mid_total % mids ? 1 : 0));
      pieces.push_back(end);
      consider(pieces);
    }
  }
  return best;
}

// Modelled duration of a call cut into `pieces` (the operator compares its current cut with a new one).
double model_exec_ms(const AteniaMoeConfig& c, const std::vector<uint64_t>& pieces, const ExecFit* fit) {
  ExecModel m = exec_model(c);
  if (fit && fit->valid) {
    m.fitted = true;
    m.fit_a = fit->a_ms;
    m.fit_b = fit->b_ms;
    m.copy_token_ms = fit->copy_token_ms;
  }
  return model_pipeline_ms(m, pieces);
}

// The operator's own timings of one pipelined call refine the model: piece i of tokens[i] tokens took
// forward_ms[i] on the device, and copying copy_tokens tokens took copy_ms.  Two piece sizes give the line
// forward(T) = a + b T; one size scales the analytical model to it.  Half of each new value is taken.
void update_exec_fit(const AteniaMoeConfig& c, const uint64_t* tokens, const float* forward_ms, int n_pieces,
                     uint64_t copy_tokens, float copy_ms, ExecFit* fit) {
  if (!fit || n_pieces <= 0) return;
  double st = 0, sm = 0, stt = 0, stm = 0;
  int used = 0;
  for (int i = 0; i < n_pieces; ++i) {
    if (!(forward_ms[i] > 0.f) || tokens[i] == 0) continue;
    const double t = (double)tokens[i], ms = forward_ms[i];
    st += t;
    sm += ms;
    stt += t * t;
    stm += t * ms;
    ++used;
  }
  if (used == 0) return;
  const ExecModel m = exec_model(c);
  double a, b;
  const double den = used * stt - st * st;
  if (used >= 2 && den > 1e-6 * stt) {
    b = (used * stm - st * sm) / den;
    a = (sm - b * st) / used;
  } else {
    a = b = -1.0;
  }
  if (!(a > 0.0) || !(b > 0.0)) {
    // one size (or a degenerate line): keep the model's shape, match its level
    const double mean_t = st / used;
    const double pred = model_forward_ms(m, (uint64_t)mean_t);
    const double scale = (sm / used) / pred;
    b = m.token_ms * scale;
    a = (pred - m.token_ms * mean_t) * scale;
  }
  double cp = fit->valid ? fit->copy_token_ms : m.copy_token_ms;
  if (copy_tokens > 0 && copy_ms > 0.f) cp = (double)copy_ms / (double)copy_tokens;
  if (fit->valid) {
    fit->a_ms = 0.5 * (fit->a_ms + a);
    fit->b_ms = 0.5 * (fit->b_ms + b);
    fit->copy_token_ms = 0.5 * (fit->copy_token_ms + cp);
  } else {
    fit->a_ms = a;
    fit->b_ms = b;
    fit->copy_token_ms = cp;
    fit->valid = true;
  }
}

}  // namespace atenia

using namespace atenia;

extern "C" {

uint64_t atenia_auto_expert_cache_capacity(uint64_t budget_bytes, uint64_t n_layers, uint64_t per_expert_bytes,
                                           uint64_t num_experts) {
  // src/moe/residency.rs:201-211, term for term (saturating product, clamp to [1, max(E, 1)])
  const uint64_t per_layer = per_expert_bytes > 1 ? per_expert_bytes : 1;
  const uint64_t layers = n_layers > 1 ? n_layers : 1;
  uint64_t denom = layers * per_layer;
  if (per_layer != 0 && denom / per_layer != layers) denom = UINT64_MAX;  // saturating_mul
  if (denom == 0) denom = 1;
  uint64_t cap = budget_bytes / denom;
  const uint64_t hi = num_experts > 1 ? num_experts : 1;
  if (cap < 1) cap = 1;
  if (cap > hi) cap = hi;
  return cap;
}

uint64_t atenia_moe_workspace_bytes(const AteniaMoeConfig* cfg) {
  if (!cfg || valid_for_plan(*cfg) != ATENIA_OK) return 0;
  const int world = cfg->ep_world >= 1 ? cfg->ep_world : 1;
  return layer_workspace_bytes(*cfg, world);
}

int atenia_moe_plan_residency(const AteniaMoeConfig* cfg, int n_layers, uint64_t hbm_budget_bytes,
                              AteniaResidencyPlan* plan) {
  if (!cfg || !plan) return ATENIA_ERR_NULL;
  memset(plan, 0, sizeof(*plan));
  int rc = valid_for_plan(*cfg);
  if (rc) return rc;
  if (n_layers < 1) return ATENIA_ERR_SHAPE;
  const AteniaMoeConfig& c = *cfg;
  const bool q = c.weight_dtype == ATENIA_W_INT8_ROW;
  const uint64_t d = (uint64_t)c.d_model, F = (uint64_t)c.d_ff, Fs = (uint64_t)c.shared_d_ff, E = (uint64_t)c.num_experts;
  const uint64_t per_expert = 2 * matrix_bytes(F, d, q) + matrix_bytes(d, F, q);
  const uint64_t shared = Fs ? 2 * matrix_bytes(Fs, d, q) + matrix_bytes(d, Fs, q) : 0;
  plan->bytes_per_expert = per_expert;
  static const int worlds[4] = {1, 2, 4, 8};
  int last_rc = ATENIA_ERR_CAPACITY;
  for (int wi = 0; wi < 4; ++wi) {
    const int G = worlds[wi];
    if (E % (uint64_t)G) continue;
    const uint64_t e_local = E / (uint64_t)G;
    // per rank and layer: the shared expert (replicated) and the layer's workspace; the router, bias and
    // gate vector are part of the workspace tally
    const uint64_t fixed_per_layer = shared + layer_workspace_bytes(c, G);
    const uint64_t fixed = fixed_per_layer * (uint64_t)n_layers;
    plan->min_ep_world = G;
    plan->experts_per_rank = (int32_t)e_local;
    plan->fixed_bytes_per_rank = fixed;
    plan->bytes_per_rank = fixed + per_expert * e_local * (uint64_t)n_layers;
    if (fixed >= hbm_budget_bytes) {
      plan->resident_experts_per_layer = 0;
      continue;
    }
    // the reference's capacity rule on what is left for experts
    const uint64_t cap = atenia_auto_expert_cache_capacity(hbm_budget_bytes - fixed, (uint64_t)n_layers, per_expert, e_local);
    const bool fits = plan->bytes_per_rank <= hbm_budget_bytes;
    plan->resident_experts_per_layer = (int32_t)(fits ? e_local : (cap < e_local ? cap : e_local - 1));
    if (fits) return ATENIA_OK;
  }
  // no world of at most 8 ranks holds its share: the plan describes the largest world tried
  return last_rc;
}

/* ---- numeric policy ---------------------------------------------------------------------------- */

namespace {
constexpr int kPolicyUnset = -1;
std::atomic<int> g_policy_override{kPolicyUnset};
std::once_flag g_env_once;
int g_env_policy = kPolicyUnset;  // kPolicyUnset: variable absent or not a policy name

std::string lower_trim(const char* s) {
  std::string t(s ? s : "");
  size_t a = 0, b = t.size();
  while (a < b && std::isspace((unsigned char)t[a])) ++a;
  while (b > a && std::isspace((unsigned char)t[b - 1])) --b;
  t = t.substr(a, b - a);
  for (char& ch : t) ch = (char)std::tolower((unsigned char)ch);
  return t;
}

void read_env_policy() {
  const char* e = std::getenv("ATENIA_NUMERIC_POLICY");
  g_env_policy = e ? atenia_numeric_policy_from_str(e) : kPolicyUnset;
  if (g_env_policy < 0) g_env_policy = kPolicyUnset;
}
}  // namespace

int atenia_numeric_policy_from_str(const char* name) {
  const std::string t = lower_trim(name);
  if (t == "certified" || t == "f64") return ATENIA_POLICY_CERTIFIED;
  if (t == "strict" || t == "f32") return ATENIA_POLICY_STRICT;
  if (t == "fast") return ATENIA_POLICY_FAST;
  return ATENIA_ERR_SHAPE;
}

const char* atenia_numeric_policy_str(int policy) {
  switch (policy) {
    case ATENIA_POLICY_CERTIFIED: return "certified";
    case ATENIA_POLICY_STRICT: return "strict";
    case ATENIA_POLICY_FAST: return "fast";
    default: return "unknown";
  }
}

int atenia_numeric_policy(void) {
  const int o = g_policy_override.load(std::memory_order_relaxed);
  if (o != kPolicyUnset) return o;
  std::call_once(g_env_once, read_env_policy);
  return g_env_policy == kPolicyUnset ? ATENIA_POLICY_CERTIFIED : g_env_policy;
}

int atenia_numeric_policy_is_explicit(void) {
  if (g_policy_override.load(std::memory_order_relaxed) != kPolicyUnset) return 1;
  std::call_once(g_env_once, read_env_policy);
  return g_env_policy != kPolicyUnset ? 1 : 0;
}

int atenia_set_numeric_policy(int policy) {
  if (policy != ATENIA_POLICY_CERTIFIED && policy != ATENIA_POLICY_STRICT && policy != ATENIA_POLICY_FAST)
    return ATENIA_ERR_SHAPE;
  g_policy_override.store(policy, std::memory_order_relaxed);
  return ATENIA_OK;
}

void atenia_clear_numeric_policy_override(void) { g_policy_override.store(kPolicyUnset, std::memory_order_relaxed); }

int atenia_numeric_policy_ffn_uses_f32(int policy) { return policy != ATENIA_POLICY_CERTIFIED ? 1 : 0; }

int atenia_numeric_policy_ffn_uses_cuda(int policy) { return policy == ATENIA_POLICY_FAST ? 1 : 0; }

int atenia_numeric_policy_gate(void) {
  // A host that has SAID which arm it wants and did not say Fast must not be served by the GPU arm
  // silently; a host that said nothing chose this library by calling it.
  if (!atenia_numeric_policy_is_explicit()) return ATENIA_OK;
  return atenia_numeric_policy_ffn_uses_cuda(atenia_numeric_policy()) ? ATENIA_OK : ATENIA_ERR_POLICY;
}

int atenia_moe_plan_exec_pieces(const AteniaMoeConfig* cfg, uint64_t n_tokens, uint64_t* pieces_out, int max_pieces) {
  return atenia_moe_plan_exec_pieces_measured(cfg, n_tokens, 0.0, 0.0, 0.0, pieces_out, max_pieces);
}

int atenia_moe_plan_exec_pieces_measured(const AteniaMoeConfig* cfg, uint64_t n_tokens, double forward_base_ms,
                                         double forward_token_ms, double copy_token_ms, uint64_t* pieces_out,
                                         int max_pieces) {
  if (!cfg || !pieces_out) return ATENIA_ERR_NULL;
  if (max_pieces <= 0 || cfg->max_tokens <= 0 || cfg->d_model <= 0 || cfg->num_experts <= 0) return ATENIA_ERR_SHAPE;
  if (forward_base_ms < 0.0 || forward_token_ms < 0.0 || copy_token_ms < 0.0) return ATENIA_ERR_SHAPE;
  ExecFit fit;
  fit.a_ms = forward_base_ms;
  fit.b_ms = forward_token_ms;
  fit.copy_token_ms = copy_token_ms;
  fit.valid = forward_token_ms > 0.0 && copy_token_ms > 0.0;  // all zero: the analytical model
  const std::vector<uint64_t> pieces = plan_exec_pieces(*cfg, n_tokens, (uint64_t)cfg->max_tokens, &fit);
  if ((int)pieces.size() > max_pieces) return ATENIA_ERR_CAPACITY;
  for (size_t i = 0; i < pieces.size(); ++i) pieces_out[i] = pieces[i];
  return (int)pieces.size();
}

}  // extern "C"
