// C ABI of the MoE block: layer life cycle, weight binding, the forward pass.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "layer.cuh"
#include "v3_route.cuh"

namespace atenia {

static std::atomic<uint64_t> g_counters[8];

void count_launch(int n) { g_counters[ATENIA_COUNTER_KERNEL_LAUNCHES] += (uint64_t)n; }
void count_tcgen05_launch() { g_counters[ATENIA_COUNTER_TCGEN05_LAUNCHES] += 1; }
void count_bytes(int which, uint64_t n) { g_counters[which] += n; }

namespace {

template <typename T>
int dev_alloc(T** p, size_t count) {
  *p = nullptr;
  if (count == 0) return ATENIA_OK;
  return (int)cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T));
}

int validate_config(const AteniaMoeConfig& c) {
  if (c.num_experts < 1 || c.num_experts > 128) return ATENIA_ERR_SHAPE;
  if (c.experts_per_token < 1 || c.experts_per_token > 8 || c.experts_per_token > c.num_experts)
    return ATENIA_ERR_SHAPE;
  if (c.d_model < 16 || c.d_model % 16 || c.d_ff < 16 || c.d_ff % 16) return ATENIA_ERR_SHAPE;
  if (c.shared_d_ff < 0 || c.shared_d_ff % 16) return ATENIA_ERR_SHAPE;
  if (c.weight_dtype != ATENIA_W_BF16 && c.weight_dtype != ATENIA_W_INT8_ROW) return ATENIA_ERR_SHAPE;
  if (c.max_tokens < 1) return ATENIA_ERR_SHAPE;
  if (c.ep_world != 1 && c.ep_world != 2 && c.ep_world != 4 && c.ep_world != 8) return ATENIA_ERR_SHAPE;
  if (c.ep_rank < 0 || c.ep_rank >= c.ep_world || c.num_experts % c.ep_world) return ATENIA_ERR_SHAPE;
  if ((int64_t)c.max_tokens * c.experts_per_token * c.ep_world > (int64_t)1 << 30) return ATENIA_ERR_SHAPE;
  if (c.router_mode != ATENIA_ROUTER_SOFTMAX && c.router_mode != ATENIA_ROUTER_V3) return ATENIA_ERR_SHAPE;
  if (c.router_mode == ATENIA_ROUTER_V3) {
    V3RouteParams p{c.num_experts, c.experts_per_token, c.n_group, c.topk_group, c.renormalize,
                    (double)c.routed_scaling_factor};
    if (v3_validate(p) != 0) return ATENIA_ERR_SHAPE;
  }
  return ATENIA_OK;
}

}  // namespace

int run_expert_gemms(AteniaMoeLayer* L, const CUtensorMap& tm_a, const CUtensorMap& tm_mid,
                     const __nv_bfloat16* a_ptr, __nv_bfloat16* mid, __nv_bfloat16* out,
                     const int32_t* group_offsets, int num_groups, int max_rows, cudaStream_t s) {
  const AteniaMoeConfig& c = L->cfg;
  const bool q = c.weight_dtype == ATENIA_W_INT8_ROW;
  const bool large = max_rows >= 256 * num_groups;
  // INT8: the tensor-memory kernel of w8_gemm.cu while groups are small (its MMA width follows the row
  // count), the 256-row-tile kernel of w8_gemm_m256.cu once every group fills a tile (measured on B200,
  // Mixtral shape: 1.07 / 1.61 / 2.51 ms at 1024 / 2048 / 4096 tokens against 1.27 / - / 3.56 ms of the
  // 128-row shared-memory widening kernel).  w8_mode 1 / 2 pin the small-group kernel / the 128-row
  // shared-memory widening kernel of grouped_gemm.cu (tests, A/B runs).
  const bool m256 = q && large && L->w8_mode != 1 && L->w8_mode != 2 && !L->use_check_gemm;
  const bool tmem = q && !m256 && (L->w8_mode == 1 || (L->w8_mode != 2 && !large));
  // bf16: 256-row CTA-pair tiles pay off once an average group fills a few of them; a call of at most
  // 16 rows (decode) takes the stream-K kernel of bf16_decode_gemm.cu, which spreads the few tiles
  // there are over all SMs (bf16_decode 1 / 0 pins it on for every call of at most 128 rows / off).
  const bool dec = !q && !L->use_check_gemm && L->splitk_ws &&
                   (L->bf16_decode == 1 ? max_rows <= 128 : (L->bf16_decode < 0 && max_rows <= 16));
  const bool pairs = !q && !dec && (L->pair_mode == 1 || (L->pair_mode == 0 && max_rows >= 512 * num_groups));
  // a call of at most two rows in all (decode at batch 1) is a stream over the touched experts' weights:
  // the CUDA-core matrix-vector kernel (ATENIA_MOE_GEMV=0 keeps the tensor-core kernels: A/B runs)
  // INT8, calls of at most i8_rows rows (decode): the codes multiplied as integers against digit planes of
  // the token rows (bf16_decode_gemm.cu, I8 form) -- nothing is widened and the kernel streams weights like
  // the bf16 one.  Measured on B200, Mixtral shape, 1 / 8 / 64 tokens: 0.145 / 0.221 / 0.390 ms against
  // 0.160 (matrix-vector kernel) / 0.300 / 0.525 ms (tensor-memory kernel).  ATENIA_MOE_W8_I8=0 or a pinned
  // w8_mode keep the widening kernels (tests, A/B runs).
  const bool i8dec = q && L->w8_i8 && L->dq_x && max_rows <= L->i8_rows && !L->use_check_gemm && L->w8_mode == 0;
  const bool gemv = L->use_gemv && max_rows <= L->gemv_rows && !L->use_check_gemm && !i8dec;
  if (L->timing) cudaEventRecord(L->ev[0], s);
  // (set by the forward when it left the row gather to the digit kernel; consumed here)
  const bool gather_here = L->i8_src_set && a_ptr == L->x_perm;
  L->i8_src_set = false;
  if (i8dec) {
    const DigitSource own{a_ptr, 0, nullptr, 1, max_rows};
    int rc = launch_quantize_digits(gather_here ? L->i8_src : own, group_offsets + num_groups, max_rows, c.d_model,
                                    L->i8_rows, L->dq_x, L->dq_ts_x, s);
    if (rc) return rc;
    GroupedGemmArgs g1{};
    g1.tmap_a = L->tm_dq_x;
    g1.tmap_b0 = L->d_tm_gate_i8;
    g1.tmap_b1 = L->d_tm_up_i8;
    g1.group_offsets = group_offsets;
    g1.num_groups = num_groups;
    g1.N = c.d_ff;
    g1.K = c.d_model;
    g1.mode = kSwiGLU;
    g1.out = mid;
    g1.scale0 = L->d_sc_gate;
    g1.scale1 = L->d_sc_up;
    g1.err = L->d_err;
    g1.max_rows = max_rows;
    g1.w8 = 1;
    g1.splitk_ws = L->splitk_ws;
    g1.splitk_cnt = L->splitk_cnt;
    g1.tok_scale = L->dq_ts_x;
    g1.plane_rows = L->i8_rows;
    rc = launch_grouped_gemm_w8_i8_decode(g1, L->num_sms, s);
    if (rc) return rc;
    if (L->timing) cudaEventRecord(L->ev[1], s);
    const DigitSource mid_rows{mid, 0, nullptr, 1, max_rows};
    rc = launch_quantize_digits(mid_rows, group_offsets + num_groups, max_rows, c.d_ff, L->i8_rows, L->dq_h, L->dq_ts_h,
                                s);
    if (rc) return rc;
    GroupedGemmArgs g2 = g1;
    g2.tmap_a = L->tm_dq_h;
    g2.tmap_b0 = L->d_tm_down_i8;
    g2.tmap_b1 = g2.tmap_b0;
    g2.N = c.d_model;
    g2.K = c.d_ff;
    g2.mode = kPlain;
    g2.out = out;
    g2.scale0 = L->d_sc_down;
    g2.scale1 = nullptr;
    g2.tok_scale = L->dq_ts_h;
    rc = launch_grouped_gemm_w8_i8_decode(g2, L->num_sms, s);
    if (rc) return rc;
    if (L->timing) {
      cudaEventRecord(L->ev[2], s);
      L->ev_valid[0] = L->ev_valid[1] = true;
    }
    return ATENIA_OK;
  }
  if (L->use_check_gemm || gemv) {
    GroupedGemmCheckArgs k1{a_ptr, L->d_p_gate, L->d_p_up, q ? 1 : 0, q ? L->d_sc_gate : nullptr,
                            q ? L->d_sc_up : nullptr, group_offsets, num_groups, c.d_ff, c.d_model,
                            kSwiGLU, mid, max_rows};
    int rc = gemv ? launch_grouped_gemv(k1, s) : launch_grouped_gemm_check(k1, s);
    if (rc) return rc;
  } else {
    GroupedGemmArgs g1{};
    g1.tmap_a = tm_a;
    g1.tmap_b0 = tmem ? L->d_tm_gate_sw : L->d_tm_gate;
    g1.tmap_b1 = tmem ? L->d_tm_up_sw : L->d_tm_up;
    g1.group_offsets = group_offsets;
    g1.num_groups = num_groups;
    g1.N = c.d_ff;
    g1.K = c.d_model;
    g1.mode = kSwiGLU;
    g1.out = mid;
    g1.scale0 = q ? L->d_sc_gate : nullptr;
    g1.scale1 = q ? L->d_sc_up : nullptr;
    g1.err = L->d_err;
    g1.max_rows = max_rows;
    g1.w8 = q;
    g1.splitk_ws = L->splitk_ws;
    g1.splitk_cnt = L->splitk_cnt;
    int rc = m256 ? launch_grouped_gemm_w8_m256(g1, L->num_sms, s)
                  : dec ? launch_grouped_gemm_bf16_decode(g1, L->num_sms, s)
                  : tmem ? launch_grouped_gemm_w8_tmem(g1, L->num_sms, s)
                         : pairs ? launch_grouped_gemm_2cta(g1, L->num_sms, s)
                                 : launch_grouped_gemm_tcgen05(g1, L->num_sms, s);
    if (rc) return rc;
  }
  if (L->timing) cudaEventRecord(L->ev[1], s);
  if (L->use_check_gemm || gemv) {
    GroupedGemmCheckArgs k2{mid, L->d_p_down, nullptr, q ? 1 : 0, q ? L->d_sc_down : nullptr, nullptr,
                            group_offsets, num_groups, c.d_model, c.d_ff, kPlain, out, max_rows};
    int rc = gemv ? launch_grouped_gemv(k2, s) : launch_grouped_gemm_check(k2, s);
    if (rc) return rc;
  } else {
    GroupedGemmArgs g2{};
    g2.tmap_a = tm_mid;
    g2.tmap_b0 = tmem ? L->d_tm_down_sw : L->d_tm_down;
    g2.tmap_b1 = g2.tmap_b0;
    g2.group_offsets = group_offsets;
    g2.num_groups = num_groups;
    g2.N = c.d_model;
    g2.K = c.d_ff;
    g2.mode = kPlain;
    g2.out = out;
    g2.scale0 = q ? L->d_sc_down : nullptr;
    g2.scale1 = nullptr;
    g2.err = L->d_err;
    g2.max_rows = max_rows;
    g2.w8 = q;
    g2.splitk_ws = L->splitk_ws;
    g2.splitk_cnt = L->splitk_cnt;
    int rc = m256 ? launch_grouped_gemm_w8_m256(g2, L->num_sms, s)
                  : dec ? launch_grouped_gemm_bf16_decode(g2, L->num_sms, s)
                  : tmem ? launch_grouped_gemm_w8_tmem(g2, L->num_sms, s)
                         : pairs ? launch_grouped_gemm_2cta(g2, L->num_sms, s)
                                 : launch_grouped_gemm_tcgen05(g2, L->num_sms, s);
    if (rc) return rc;
  }
  if (L->timing) {
    cudaEventRecord(L->ev[2], s);
    L->ev_valid[0] = L->ev_valid[1] = true;
  }
  return ATENIA_OK;
}

namespace {

int run_shared_gemms(AteniaMoeLayer* L, const __nv_bfloat16* xb, int T, cudaStream_t s) {
  const AteniaMoeConfig& c = L->cfg;
  const bool q = c.weight_dtype == ATENIA_W_INT8_ROW;
  // (the shared expert is one group: INT8 takes the small-group kernel below 256 tokens and the
  // 256-row-tile kernel above)
  const bool m256 = q && T >= 256 && L->w8_mode != 1 && L->w8_mode != 2 && !L->use_check_gemm;
  const bool tmem = q && !m256 && (L->w8_mode == 1 || (L->w8_mode != 2 && T < 256));
  const bool pairs = !q && (L->pair_mode == 1 || (L->pair_mode == 0 && T >= 512));
  const bool gemv = L->use_gemv && T <= L->gemv_rows && !L->use_check_gemm;
  if (L->timing) cudaEventRecord(L->ev[3], s);
  if (L->use_check_gemm || gemv) {
    GroupedGemmCheckArgs k1{xb, L->d_p_shared, L->d_p_shared + 1, q ? 1 : 0, q ? L->d_sc_shared : nullptr,
                            q ? L->d_sc_shared + 1 : nullptr, L->shared_offsets, 1, c.shared_d_ff, c.d_model,
                            kSwiGLU, L->h_shared, T};
    int rc = gemv ? launch_grouped_gemv(k1, s) : launch_grouped_gemm_check(k1, s);
    if (rc) return rc;
    if (L->timing) cudaEventRecord(L->ev[4], s);
    GroupedGemmCheckArgs k2{L->h_shared, L->d_p_shared + 2, nullptr, q ? 1 : 0, q ? L->d_sc_shared + 2 : nullptr,
                            nullptr, L->shared_offsets, 1, c.d_model, c.shared_d_ff, kPlain, L->y_shared, T};
    rc = gemv ? launch_grouped_gemv(k2, s) : launch_grouped_gemm_check(k2, s);
    if (rc) return rc;
    if (L->timing) {
      cudaEventRecord(L->ev[5], s);
      L->ev_valid[2] = L->ev_valid[3] = true;
    }
    return ATENIA_OK;
  }
  GroupedGemmArgs g1{};
  int rc = encode_tmap_2d_bf16(&g1.tmap_a, xb, (uint64_t)T, (uint64_t)c.d_model, 128, 64);
  if (rc) return rc;
  g1.tmap_b0 = tmem ? L->d_tm_shared_sw : L->d_tm_shared;
  g1.tmap_b1 = g1.tmap_b0 + 1;
  g1.group_offsets = L->shared_offsets;
  g1.num_groups = 1;
  g1.N = c.shared_d_ff;
  g1.K = c.d_model;
  g1.mode = kSwiGLU;
  g1.out = L->h_shared;
  g1.scale0 = q ? L->d_sc_shared : nullptr;
  g1.scale1 = q ? L->d_sc_shared + 1 : nullptr;
  g1.err = L->d_err;
  g1.max_rows = T;
  g1.w8 = q;
  g1.splitk_ws = L->splitk_ws_shared;  // its own: these launches may run beside the routed GEMMs
  rc = m256 ? launch_grouped_gemm_w8_m256(g1, L->num_sms, s)
       : tmem ? launch_grouped_gemm_w8_tmem(g1, L->num_sms, s)
                  : pairs ? launch_grouped_gemm_2cta(g1, L->num_sms, s) : launch_grouped_gemm_tcgen05(g1, L->num_sms, s);
  if (rc) return rc;
  if (L->timing) cudaEventRecord(L->ev[4], s);
  GroupedGemmArgs g2{};
  g2.tmap_a = L->tm_h_shared;
  g2.tmap_b0 = (tmem ? L->d_tm_shared_sw : L->d_tm_shared) + 2;
  g2.tmap_b1 = g2.tmap_b0;
  g2.group_offsets = L->shared_offsets;
  g2.num_groups = 1;
  g2.N = c.d_model;
  g2.K = c.shared_d_ff;
  g2.mode = kPlain;
  g2.out = L->y_shared;
  g2.scale0 = q ? L->d_sc_shared + 2 : nullptr;
  g2.err = L->d_err;
  g2.max_rows = T;
  g2.w8 = q;
  g2.splitk_ws = L->splitk_ws_shared;
  rc = m256 ? launch_grouped_gemm_w8_m256(g2, L->num_sms, s)
       : tmem ? launch_grouped_gemm_w8_tmem(g2, L->num_sms, s)
                  : pairs ? launch_grouped_gemm_2cta(g2, L->num_sms, s) : launch_grouped_gemm_tcgen05(g2, L->num_sms, s);
  if (rc) return rc;
  if (L->timing) {
    cudaEventRecord(L->ev[5], s);
    L->ev_valid[2] = L->ev_valid[3] = true;
  }
  return ATENIA_OK;
}

}  // namespace
}  // namespace atenia

using namespace atenia;

extern "C" {

int atenia_moe_create(const AteniaMoeConfig* cfg, AteniaMoeLayer** out) {
  if (!cfg || !out) return ATENIA_ERR_NULL;
  *out = nullptr;
  int rc = validate_config(*cfg);
  if (rc) return rc;
  AteniaMoeLayer* L = new (std::nothrow) AteniaMoeLayer();
  if (!L) return (int)cudaErrorMemoryAllocation;
  L->cfg = *cfg;
  const AteniaMoeConfig& c = L->cfg;
  cudaError_t e = cudaGetDevice(&L->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&L->num_sms, cudaDevAttrMultiProcessorCount, L->device);
  if (e != cudaSuccess) {
    delete L;
    return (int)e;
  }
  L->e_local = c.num_experts / c.ep_world;
  L->e_begin = c.ep_rank * L->e_local;
  L->n_groups = c.ep_world == 1 ? L->e_local : c.ep_world * L->e_local;
  L->has_shared = c.shared_d_ff > 0;
  L->use_check_gemm = std::getenv("ATENIA_MOE_CHECK_GEMM") && std::atoi(std::getenv("ATENIA_MOE_CHECK_GEMM")) != 0;
  L->w8_mode = std::getenv("ATENIA_MOE_W8_MODE") ? std::atoi(std::getenv("ATENIA_MOE_W8_MODE")) : 0;
  L->pair_mode = std::getenv("ATENIA_MOE_PAIR_MODE") ? std::atoi(std::getenv("ATENIA_MOE_PAIR_MODE")) : 0;
  L->shared_aside = !(std::getenv("ATENIA_MOE_SHARED_ASIDE") && std::atoi(std::getenv("ATENIA_MOE_SHARED_ASIDE")) == 0);
  L->use_gemv = !(std::getenv("ATENIA_MOE_GEMV") && std::atoi(std::getenv("ATENIA_MOE_GEMV")) == 0);
  // ATENIA_MOE_W8_I8=0: INT8 decode calls keep the widening kernels; ATENIA_MOE_W8_I8_ROWS moves the row
  // count up to which the integer-MMA decode kernel is taken (16 .. kI8DecodeMaxRows; A/B runs)
  L->w8_i8 = !(std::getenv("ATENIA_MOE_W8_I8") && std::atoi(std::getenv("ATENIA_MOE_W8_I8")) == 0);

  {
    // ATENIA_MOE_GEMV_ROWS moves the hand-over to the tensor-core kernels (1 .. 4 rows: A/B runs)
    const char* e = std::getenv("ATENIA_MOE_GEMV_ROWS");
    const int r = e ? std::atoi(e) : kGemvMaxRows;
    L->gemv_rows = r < 1 ? 1 : (r > 4 ? 4 : r);
  }
  // Router kernel: by default the split-k kernel for batches of at most 128 tokens (many CTAs share one
  // token block's dot products), the f64 tensor-core kernel for 32 experts and more, the CUDA-core
  // kernel otherwise.  ATENIA_MOE_ROUTER = scalar | dmma | splitk pins one (tests, A/B runs); a pinned
  // split-k serves batches up to 1024 tokens and hands larger ones to the CUDA-core kernel.
  {
    const char* rv = std::getenv("ATENIA_MOE_ROUTER");
    const std::string r(rv ? rv : "");
    L->router_variant = r == "scalar" ? 0 : r == "dmma" ? 1 : r == "splitk" ? 2 : -1;
  }
  L->bf16_decode = c.weight_dtype != ATENIA_W_BF16 ? 0
                   : std::getenv("ATENIA_MOE_BF16_DECODE") ? (std::atoi(std::getenv("ATENIA_MOE_BF16_DECODE")) != 0 ? 1 : 0)
                                                           : -1;
  const size_t Tm = (size_t)c.max_tokens, k = (size_t)c.experts_per_token, E = (size_t)c.num_experts;
  const size_t d = (size_t)c.d_model, F = (size_t)c.d_ff, Fs = (size_t)c.shared_d_ff;
  const size_t R = Tm * k;
  L->rows_cap = (int)R;
  const size_t nblk = (R + kDispatchChunk - 1) / kDispatchChunk;
#define TRY_ALLOC(ptr, n)                  \
  do {                                     \
    rc = dev_alloc(&(ptr), (n));           \
    if (rc) {                              \
      atenia_moe_destroy(L);               \
      return rc;                           \
    }                                      \
  } while (0)
  TRY_ALLOC(L->d_router, E * d);
  TRY_ALLOC(L->d_bias, E);
  TRY_ALLOC(L->d_gate_vec, d);
  if (c.router_mode == ATENIA_ROUTER_V3) {
    TRY_ALLOC(L->d_escore, E);
    TRY_ALLOC(L->logits_ws, Tm * E);
  }
  TRY_ALLOC(L->topk_idx, R);
  TRY_ALLOC(L->topk_w, R);
  TRY_ALLOC(L->gate_scale, Tm);
  TRY_ALLOC(L->perm, R);
  TRY_ALLOC(L->inv_perm, R);
  TRY_ALLOC(L->expert_offsets, E + 1);
  TRY_ALLOC(L->shared_offsets, 2);
  TRY_ALLOC(L->block_counts, nblk * E);
  TRY_ALLOC(L->block_base, nblk * E);
  TRY_ALLOC(L->x_perm, R * d);
  TRY_ALLOC(L->y_perm, R * d);
  if (c.ep_world == 1) TRY_ALLOC(L->h, R * F);
  TRY_ALLOC(L->x_bf16, Tm * d);
  if (L->has_shared) {
    TRY_ALLOC(L->h_shared, Tm * Fs);
    TRY_ALLOC(L->y_shared, Tm * d);
  }
  TRY_ALLOC(L->d_err, 1);
  TRY_ALLOC(L->d_tm_gate, (size_t)L->n_groups);
  TRY_ALLOC(L->d_tm_up, (size_t)L->n_groups);
  TRY_ALLOC(L->d_tm_down, (size_t)L->n_groups);
  TRY_ALLOC(L->d_tm_shared, 3);
  if (L->bf16_decode != 0 || c.weight_dtype == ATENIA_W_INT8_ROW) {
    TRY_ALLOC(L->splitk_ws, (size_t)L->num_sms * 2 * kW8SplitKSlotFloats);
    // ATENIA_MOE_SPLITK_FIXUP=0: a second kernel adds the pieces of split tiles (A/B runs)
    if (!(std::getenv("ATENIA_MOE_SPLITK_FIXUP") && std::atoi(std::getenv("ATENIA_MOE_SPLITK_FIXUP")) == 0)) {
      TRY_ALLOC(L->splitk_cnt, (size_t)kSplitKMaxTiles * 8);
      if (cudaMemset(L->splitk_cnt, 0, (size_t)kSplitKMaxTiles * 8 * sizeof(unsigned int)) != cudaSuccess) {
        atenia_moe_destroy(L);
        return ATENIA_ERR_STATE;
      }
    }
  }
  {
    const int sk_cap = L->router_variant == 2 ? 1024 : (L->router_variant == -1 ? 128 : 0);
    L->sk_tokens = c.max_tokens < sk_cap ? c.max_tokens : sk_cap;
  }
  if (L->sk_tokens > 0) {
    size_t np = 0, ng = 0, nc = 0;
    router_splitk_workspace(L->sk_tokens, c.d_model, c.num_experts, &np, &ng, &nc);
    TRY_ALLOC(L->sk_part, np);
    TRY_ALLOC(L->sk_gate, ng);
    TRY_ALLOC(L->sk_counters, nc);
    if (cudaMemset(L->sk_counters, 0, nc * sizeof(unsigned int)) != cudaSuccess) {
      atenia_moe_destroy(L);
      return ATENIA_ERR_STATE;
    }
  }
  if (c.weight_dtype == ATENIA_W_INT8_ROW) {
    if (L->has_shared) TRY_ALLOC(L->splitk_ws_shared, (size_t)L->num_sms * 2 * kW8SplitKSlotFloats);
    // integer-MMA decode kernel: int8 weight maps with the 128-byte swizzle, digit planes of the token rows
  {
    const char* e = std::getenv("ATENIA_MOE_W8_I8_ROWS");
    int r = e ? std::atoi(e) : kI8DecodeDefaultRows;
    r = r < 16 ? 16 : (r > kI8DecodeMaxRows ? kI8DecodeMaxRows : r);
    const int cap = (int)((R + 15) / 16 * 16);  // never more planes than the layer has rows
    L->i8_rows = r < cap ? r : cap;
  }
    TRY_ALLOC(L->d_tm_gate_i8, (size_t)L->n_groups);
    TRY_ALLOC(L->d_tm_up_i8, (size_t)L->n_groups);
    TRY_ALLOC(L->d_tm_down_i8, (size_t)L->n_groups);
    TRY_ALLOC(L->dq_x, (size_t)4 * L->i8_rows * c.d_model);
    TRY_ALLOC(L->dq_h, (size_t)4 * L->i8_rows * c.d_ff);
    TRY_ALLOC(L->dq_ts_x, (size_t)L->i8_rows);
    TRY_ALLOC(L->dq_ts_h, (size_t)L->i8_rows);
    TRY_ALLOC(L->d_tm_gate_sw, (size_t)L->n_groups);
    TRY_ALLOC(L->d_tm_up_sw, (size_t)L->n_groups);
    TRY_ALLOC(L->d_tm_down_sw, (size_t)L->n_groups);
    TRY_ALLOC(L->d_tm_shared_sw, 3);
  }
  TRY_ALLOC(L->d_sc_gate, (size_t)L->n_groups);
  TRY_ALLOC(L->d_sc_up, (size_t)L->n_groups);
  TRY_ALLOC(L->d_sc_down, (size_t)L->n_groups);
  TRY_ALLOC(L->d_sc_shared, 3);
  TRY_ALLOC(L->d_p_gate, (size_t)L->n_groups);
  TRY_ALLOC(L->d_p_up, (size_t)L->n_groups);
  TRY_ALLOC(L->d_p_down, (size_t)L->n_groups);
  TRY_ALLOC(L->d_p_shared, 3);
  if (c.ep_world > 1) {
    // Worst case every token of every rank selects only experts of this rank.
    const size_t RC = R * (size_t)c.ep_world;
    L->recv_cap = (int)RC;
    TRY_ALLOC(L->recv_x, RC * d);
    TRY_ALLOC(L->recv_h, RC * F);
    TRY_ALLOC(L->recv_y, RC * d);
    TRY_ALLOC(L->d_counts_all, (size_t)c.ep_world * E);
    TRY_ALLOC(L->d_group_offsets, (size_t)L->n_groups + 1);
    e = cudaMallocHost(reinterpret_cast<void**>(&L->h_counts_all), (size_t)c.ep_world * E * sizeof(int32_t));
    if (e != cudaSuccess) {
      atenia_moe_destroy(L);
      return (int)e;
    }
  }
#undef TRY_ALLOC
  e = cudaMemset(L->d_err, 0, sizeof(DeviceError));
  if (e == cudaSuccess) e = cudaMemset(L->perm, 0, R * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMemset(L->inv_perm, 0, R * sizeof(int32_t));
  if (e != cudaSuccess) {
    atenia_moe_destroy(L);
    return (int)e;
  }
  rc = encode_tmap_2d_bf16(&L->tm_x_perm, L->x_perm, R, d, 128, 64);
  if (!rc && L->h) rc = encode_tmap_2d_bf16(&L->tm_h, L->h, R, F, 128, 64);
  if (!rc && L->dq_x) rc = encode_tmap_2d_u8(&L->tm_dq_x, L->dq_x, (uint64_t)4 * L->i8_rows, d, 16, 128, 2);
  if (!rc && L->dq_h) rc = encode_tmap_2d_u8(&L->tm_dq_h, L->dq_h, (uint64_t)4 * L->i8_rows, F, 16, 128, 2);
  if (!rc && L->has_shared) rc = encode_tmap_2d_bf16(&L->tm_h_shared, L->h_shared, Tm, Fs, 128, 64);
  if (!rc && c.ep_world > 1) {
    rc = encode_tmap_2d_bf16(&L->tm_recv_x, L->recv_x, (uint64_t)L->recv_cap, d, 128, 64);
    if (!rc) rc = encode_tmap_2d_bf16(&L->tm_recv_h, L->recv_h, (uint64_t)L->recv_cap, F, 128, 64);
  }
  if (rc) {
    atenia_moe_destroy(L);
    return rc;
  }
  for (int i = 0; i < 8; ++i) cudaEventCreate(&L->ev[i]);
  for (int i = 0; i < 6; ++i) cudaEventCreate(&L->ph[i]);
  if (L->has_shared) {
    e = cudaStreamCreateWithFlags(&L->aux_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&L->ev_join, cudaEventDisableTiming);
    if (e != cudaSuccess) {
      atenia_moe_destroy(L);
      return (int)e;
    }
  }
  *out = L;
  return ATENIA_OK;
}

int atenia_moe_destroy(AteniaMoeLayer* L) {
  if (!L) return ATENIA_OK;
  cudaDeviceSynchronize();
  ep_destroy(L);
  void* ptrs[] = {L->d_router, L->d_bias, L->d_gate_vec, L->topk_idx, L->topk_w, L->gate_scale, L->perm,
                  L->inv_perm, L->expert_offsets, L->shared_offsets, L->block_counts, L->block_base, L->x_perm,
                  L->h, L->y_perm, L->x_bf16, L->h_shared, L->y_shared, L->d_err, L->d_tm_gate, L->d_tm_up,
                  L->d_tm_down, L->d_tm_shared, L->d_sc_gate, L->d_sc_up, L->d_sc_down, L->d_sc_shared,
                  L->d_p_gate, L->d_p_up, L->d_p_down, L->d_p_shared, L->d_tm_gate_sw, L->d_tm_up_sw,
                  L->d_tm_down_sw, L->d_tm_shared_sw,
                  L->splitk_ws, L->splitk_cnt, L->splitk_ws_shared, L->d_tm_gate_i8, L->d_tm_up_i8, L->d_tm_down_i8, L->dq_x, L->dq_h,
                  L->dq_ts_x, L->dq_ts_h, L->d_escore, L->logits_ws, L->recv_x, L->recv_h, L->recv_y, L->d_counts_all,
                  L->d_group_offsets, L->d_peer_recv_x, L->d_peer_y_perm, L->d_dst_base, L->d_src_base,
                  L->d_gemm_offsets, L->d_bar, L->d_sync, L->d_peer_sync, L->d_ep_state, L->sk_part, L->sk_gate, L->sk_counters, L->block_normed};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  for (void* p : L->owned) cudaFree(p);
  if (L->h_counts_all) cudaFreeHost(L->h_counts_all);
  for (int i = 0; i < 8; ++i)
    if (L->ev[i]) cudaEventDestroy(L->ev[i]);
  for (int i = 0; i < 6; ++i)
    if (L->ph[i]) cudaEventDestroy(L->ph[i]);
  if (L->ev_fork) cudaEventDestroy(L->ev_fork);
  if (L->ev_join) cudaEventDestroy(L->ev_join);
  if (L->aux_stream) cudaStreamDestroy(L->aux_stream);
  delete L;
  return ATENIA_OK;
}

int atenia_moe_set_weights(AteniaMoeLayer* L, const AteniaMoeWeights* w) {
  if (!L || !w || !w->w_router || !w->w_gate || !w->w_up || !w->w_down) return ATENIA_ERR_NULL;
  const AteniaMoeConfig& c = L->cfg;
  const bool q = c.weight_dtype == ATENIA_W_INT8_ROW;
  if (q && (!w->s_gate || !w->s_up || !w->s_down)) return ATENIA_ERR_NULL;
  if (L->has_shared && (!w->shared_w_gate || !w->shared_w_up || !w->shared_w_down)) return ATENIA_ERR_NULL;
  if (L->has_shared && q && (!w->shared_s_gate || !w->shared_s_up || !w->shared_s_down)) return ATENIA_ERR_NULL;
  if (c.shared_gated && L->has_shared && !w->shared_gate_vec) return ATENIA_ERR_NULL;
  const size_t d = (size_t)c.d_model, F = (size_t)c.d_ff, Fs = (size_t)c.shared_d_ff, E = (size_t)c.num_experts;
  for (void* p : L->owned) cudaFree(p);
  L->owned.clear();
  L->weights_set = false;

  ATENIA_CUDA_TRY(cudaMemcpy(L->d_router, w->w_router, E * d * sizeof(float), cudaMemcpyDeviceToDevice));
  L->has_bias = w->router_bias != nullptr;
  if (L->has_bias)
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_bias, w->router_bias, E * sizeof(float), cudaMemcpyDeviceToDevice));
  if (c.router_mode == ATENIA_ROUTER_V3) {
    if (w->e_score_bias)
      ATENIA_CUDA_TRY(cudaMemcpy(L->d_escore, w->e_score_bias, E * sizeof(float), cudaMemcpyDeviceToDevice));
    else
      ATENIA_CUDA_TRY(cudaMemset(L->d_escore, 0, E * sizeof(float)));
  }
  // kept whenever given: a call may ask for the gated convention of a layer configured ungated
  L->gate_vec_bound = w->shared_gate_vec != nullptr && L->has_shared;
  L->has_gate_vec = L->gate_vec_bound && c.shared_gated;
  if (L->gate_vec_bound)
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_gate_vec, w->shared_gate_vec, d * sizeof(float), cudaMemcpyDeviceToDevice));

  // INT8 matrices are borrowed as they are: their tensor maps describe bytes and the grouped GEMM
  // widens the codes to bf16 on chip.
  auto encode = [&](CUtensorMap* m, const void* src, size_t rows, size_t cols, int sw64 = 0) -> int {
    if (!src) return ATENIA_ERR_NULL;
    return q ? encode_tmap_2d_u8(m, src, rows, cols, 128, 64, sw64) : encode_tmap_2d_bf16(m, src, rows, cols, 128, 64);
  };

  const int G = L->n_groups, El = L->e_local;
  std::vector<CUtensorMap> tg(G), tu(G), td(G), tgs(G), tus(G), tds(G), tgi(G), tui(G), tdi(G);
  std::vector<const void*> pg(G), pu(G), pd(G);
  std::vector<const float*> sg(G, nullptr), su(G, nullptr), sd(G, nullptr);
  for (int e = 0; e < El; ++e) {
    pg[e] = w->w_gate[e];
    pu[e] = w->w_up[e];
    pd[e] = w->w_down[e];
    int rc = encode(&tg[e], pg[e], F, d);
    if (!rc) rc = encode(&tu[e], pu[e], F, d);
    if (!rc) rc = encode(&td[e], pd[e], d, F);
    if (!rc && q) rc = encode(&tgs[e], pg[e], F, d, 1);
    if (!rc && q) rc = encode(&tus[e], pu[e], F, d, 1);
    if (!rc && q) rc = encode(&tds[e], pd[e], d, F, 1);
    // integer-MMA decode kernel: 128 codes of 128 rows per box, 128-byte swizzle
    if (!rc && q) rc = encode_tmap_2d_u8(&tgi[e], pg[e], F, d, 128, 128, 2);
    if (!rc && q) rc = encode_tmap_2d_u8(&tui[e], pu[e], F, d, 128, 128, 2);
    if (!rc && q) rc = encode_tmap_2d_u8(&tdi[e], pd[e], d, F, 128, 128, 2);
    if (rc) return rc;
    if (q) {
      if (!w->s_gate[e] || !w->s_up[e] || !w->s_down[e]) return ATENIA_ERR_NULL;
      sg[e] = w->s_gate[e];
      su[e] = w->s_up[e];
      sd[e] = w->s_down[e];
    }
  }
  // Under expert parallelism the groups are (source rank, local expert) pairs: replicate.
  for (int g = El; g < G; ++g) {
    tg[g] = tg[g % El];
    tu[g] = tu[g % El];
    td[g] = td[g % El];
    tgs[g] = tgs[g % El];
    tus[g] = tus[g % El];
    tds[g] = tds[g % El];
    tgi[g] = tgi[g % El];
    tui[g] = tui[g % El];
    tdi[g] = tdi[g % El];
    pg[g] = pg[g % El];
    pu[g] = pu[g % El];
    pd[g] = pd[g % El];
    sg[g] = sg[g % El];
    su[g] = su[g % El];
    sd[g] = sd[g % El];
  }
  const size_t mb = (size_t)G * sizeof(CUtensorMap), pb = (size_t)G * sizeof(void*);
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_gate, tg.data(), mb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_up, tu.data(), mb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_down, td.data(), mb, cudaMemcpyHostToDevice));
  if (q) {
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_gate_sw, tgs.data(), mb, cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_up_sw, tus.data(), mb, cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_down_sw, tds.data(), mb, cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_gate_i8, tgi.data(), mb, cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_up_i8, tui.data(), mb, cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_down_i8, tdi.data(), mb, cudaMemcpyHostToDevice));
  }
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_p_gate, pg.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_p_up, pu.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_p_down, pd.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_sc_gate, sg.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_sc_up, su.data(), pb, cudaMemcpyHostToDevice));
  ATENIA_CUDA_TRY(cudaMemcpy(L->d_sc_down, sd.data(), pb, cudaMemcpyHostToDevice));
  if (L->has_shared) {
    CUtensorMap ts[3], tss[3];
    const void* ps[3];
    const float* ss[3] = {q ? w->shared_s_gate : nullptr, q ? w->shared_s_up : nullptr,
                          q ? w->shared_s_down : nullptr};
    ps[0] = w->shared_w_gate;
    ps[1] = w->shared_w_up;
    ps[2] = w->shared_w_down;
    int rc = encode(&ts[0], ps[0], Fs, d);
    if (!rc) rc = encode(&ts[1], ps[1], Fs, d);
    if (!rc) rc = encode(&ts[2], ps[2], d, Fs);
    if (!rc && q) rc = encode(&tss[0], ps[0], Fs, d, 1);
    if (!rc && q) rc = encode(&tss[1], ps[1], Fs, d, 1);
    if (!rc && q) rc = encode(&tss[2], ps[2], d, Fs, 1);
    if (rc) return rc;
    if (q) ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_shared_sw, tss, sizeof(tss), cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_tm_shared, ts, sizeof(ts), cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_p_shared, ps, sizeof(ps), cudaMemcpyHostToDevice));
    ATENIA_CUDA_TRY(cudaMemcpy(L->d_sc_shared, ss, sizeof(ss), cudaMemcpyHostToDevice));
  }
  ATENIA_CUDA_TRY(cudaDeviceSynchronize());
  L->weights_set = true;
  return ATENIA_OK;
}

static int forward_impl(AteniaMoeLayer* L, const void* x, int x_dtype, int T, void* out, int out_dtype,
                        const AteniaMoeAux* aux, void* stream, const int32_t* sel_idx, const float* sel_w,
                        int convention = ATENIA_CONVENTION_LAYER);

int atenia_moe_forward(AteniaMoeLayer* L, const void* x, int x_dtype, int T, void* out, int out_dtype,
                       const AteniaMoeAux* aux, void* stream) {
  return forward_impl(L, x, x_dtype, T, out, out_dtype, aux, stream, nullptr, nullptr);
}

int atenia_moe_forward_with(AteniaMoeLayer* L, const void* x, int x_dtype, int T, void* out, int out_dtype,
                            const AteniaMoeAux* aux, void* stream, int convention) {
  if (convention != ATENIA_CONVENTION_LAYER && convention != ATENIA_CONVENTION_ATENIA &&
      convention != ATENIA_CONVENTION_HF_QWEN)
    return ATENIA_ERR_SHAPE;
  if (L && convention != ATENIA_CONVENTION_LAYER && L->cfg.router_mode == ATENIA_ROUTER_V3) return ATENIA_ERR_UNSUPPORTED;
  return forward_impl(L, x, x_dtype, T, out, out_dtype, aux, stream, nullptr, nullptr, convention);
}

int atenia_moe_forward_selected(AteniaMoeLayer* L, const void* x, int x_dtype, int T, const int32_t* topk_idx,
                                const float* topk_w, void* out, int out_dtype, void* stream) {
  if (!topk_idx || !topk_w) return ATENIA_ERR_NULL;
  return forward_impl(L, x, x_dtype, T, out, out_dtype, nullptr, stream, topk_idx, topk_w);
}

static int forward_impl(AteniaMoeLayer* L, const void* x, int x_dtype, int T, void* out, int out_dtype,
                        const AteniaMoeAux* aux, void* stream, const int32_t* sel_idx, const float* sel_w,
                        int convention) {
  if (!L) return ATENIA_ERR_NULL;
  if (!L->weights_set) return ATENIA_ERR_STATE;
  if (T < 0) return ATENIA_ERR_SHAPE;
  // an empty batch has no buffers to check (token-sharded expert parallelism still joins the exchange)
  const bool no_exchange = L->cfg.ep_world == 1 || L->ep_replicated;
  if (T == 0 && no_exchange) return ATENIA_OK;
  if (T > 0 && (!x || !out)) return ATENIA_ERR_NULL;  // an empty rank may pass NULL and still joins the exchange
  if (T > L->cfg.max_tokens) return ATENIA_ERR_CAPACITY;
  if ((x_dtype != ATENIA_IO_BF16 && x_dtype != ATENIA_IO_F32) ||
      (out_dtype != ATENIA_IO_BF16 && out_dtype != ATENIA_IO_F32))
    return ATENIA_ERR_SHAPE;
  if (L->cfg.ep_world > 1 && !ep_ready(L)) return ATENIA_ERR_STATE;
  g_counters[ATENIA_COUNTER_FORWARD_CALLS] += 1;
  const AteniaMoeConfig& c = L->cfg;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k = c.experts_per_token, n = T * k;
  const bool x_f32 = x_dtype == ATENIA_IO_F32;
  int rc0 = ATENIA_OK;
  // the convention of this call (RealMoeLayer::forward_with): Atenia renormalises and ignores the gate;
  // HuggingFaceQwen keeps the raw weights and gates the shared expert when a gate vector is bound
  const int renorm = convention == ATENIA_CONVENTION_LAYER ? c.renormalize : (convention == ATENIA_CONVENTION_ATENIA ? 1 : 0);
  const bool gated = convention == ATENIA_CONVENTION_LAYER ? L->has_gate_vec
                                                           : (convention == ATENIA_CONVENTION_HF_QWEN && L->gate_vec_bound);

  if (L->timing) cudaEventRecord(L->ph[0], s);
  // The shared expert needs only this call's tokens, so its GEMMs run on the layer's second stream from
  // the start of the forward, beside the routing phase (an FP64-bound router, an HBM-bound gather: the
  // tensor cores are idle there) and, under expert parallelism, beside the exchanges; the combine waits
  // for them.  f32 input is converted to bf16 first.  Tiny batches keep the one-stream order (the two
  // event hops would cost more than the overlap gives); ATENIA_MOE_SHARED_ASIDE=0 turns it off.
  const bool shared_aside = L->has_shared && T >= 64 && L->aux_stream && L->shared_aside;
  if (shared_aside) {
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    if (x_f32) {
      rc0 = launch_f32_to_bf16(static_cast<const float*>(x), L->x_bf16, (int64_t)T * c.d_model, s);
      if (rc0) return rc0;
      xb = L->x_bf16;
    }
    ATENIA_CUDA_TRY(cudaEventRecord(L->ev_fork, s));
    ATENIA_CUDA_TRY(cudaStreamWaitEvent(L->aux_stream, L->ev_fork, 0));
    // (the dispatch kernels, which write the one-group offsets {0, T} otherwise, run later on `s`)
    rc0 = launch_set_pair(L->shared_offsets, 0, T, L->aux_stream);
    if (rc0) return rc0;
    rc0 = run_shared_gemms(L, xb, T, L->aux_stream);
    if (rc0) return rc0;
    ATENIA_CUDA_TRY(cudaEventRecord(L->ev_join, L->aux_stream));
  }
  RouterArgs ra{};
  ra.x = x;
  ra.x_is_f32 = x_f32;
  ra.w_router = L->d_router;
  ra.bias = L->has_bias ? L->d_bias : nullptr;
  ra.gate_vec = gated ? L->d_gate_vec : nullptr;
  ra.T = T;
  ra.d = c.d_model;
  ra.E = c.num_experts;
  ra.k = k;
  ra.renormalize = renorm;
  ra.topk_idx = L->topk_idx;
  ra.topk_w = L->topk_w;
  ra.gate_scale = gated ? L->gate_scale : nullptr;
  const bool v3 = c.router_mode == ATENIA_ROUTER_V3;
  ra.logits = (aux && aux->logits) ? aux->logits : (v3 ? L->logits_ws : nullptr);
  ra.err = L->d_err;
  ra.variant = L->router_variant;
  ra.sk_part = L->sk_part;
  ra.sk_gate = L->sk_gate;
  ra.sk_counters = L->sk_counters;
  ra.sk_tokens = L->sk_tokens;
  int rc = launch_router(ra, s);
  if (rc) return rc;
  if (v3) {
    // the router kernel supplied the f64-accumulated logits; the V3 rule replaces its selection
    rc = launch_v3_route(ra.logits, L->d_escore, T, c.num_experts, k, c.n_group, c.topk_group, c.renormalize,
                         c.routed_scaling_factor, L->topk_idx, L->topk_w, L->d_err, s);
    if (rc) return rc;
  }
  if (sel_idx && n > 0) {
    // the caller's selection replaces the router's (the router still ran: it owns the shared gate)
    ATENIA_CUDA_TRY(cudaMemcpyAsync(L->topk_idx, sel_idx, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    ATENIA_CUDA_TRY(cudaMemcpyAsync(L->topk_w, sel_w, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
  }

  DispatchArgs da{};
  da.topk_idx = L->topk_idx;
  da.n = n;
  da.E = c.num_experts;
  da.block_counts = L->block_counts;
  da.block_base = L->block_base;
  da.expert_offsets = L->expert_offsets;
  da.perm = L->perm;
  da.inv_perm = L->inv_perm;
  da.extra_offsets = shared_aside ? nullptr : L->shared_offsets;
  da.T = T;
  da.err = L->d_err;
  rc = launch_dispatch(da, s);
  if (rc) return rc;

  const bool need_xb = x_f32 && L->has_shared && !shared_aside;  // (aside: converted at the start already)
  // the direct expert-parallel exchange gathers rows straight into the owners' buffers
  const bool direct = c.ep_world > 1 && !L->ep_replicated && L->ep_direct;
  // an INT8 decode call (integer-MMA kernel) never reads x_perm: its digit kernel gathers the rows itself
  const bool i8_gather = c.weight_dtype == ATENIA_W_INT8_ROW && L->w8_i8 && L->dq_x && n <= L->i8_rows &&
                         !L->use_check_gemm && L->w8_mode == 0 && (c.ep_world == 1 || L->ep_replicated);
  rc = launch_gather_rows(x, x_f32, L->perm, L->expert_offsets + c.num_experts, (direct || i8_gather) ? 0 : n, k,
                          c.d_model, L->x_perm, need_xb ? L->x_bf16 : nullptr, T, s);
  if (rc) return rc;
  L->i8_src = DigitSource{x, x_f32 ? 1 : 0, L->perm, k, T};
  L->i8_src_set = i8_gather;
  if (L->timing) cudaEventRecord(L->ph[1], s);

  if (c.ep_world == 1) {
    if (L->timing) cudaEventRecord(L->ph[2], s);
    rc = run_expert_gemms(L, L->tm_x_perm, L->tm_h, L->x_perm, L->h, L->y_perm, L->expert_offsets,
                          c.num_experts, n, s);
  } else if (L->ep_replicated) {
    rc = ep_forward_replicated(L, n, s);
  } else if (direct) {
    // rows leave for their owners, then the routed experts
    rc = ep_direct_send(L, x, x_f32 ? 1 : 0, T, s);
    if (!rc) rc = ep_direct_finish(L, s);
  } else {
    rc = ep_forward_exchange(L, T, s);
  }
  if (rc) return rc;
  if (L->timing && c.ep_world == 1) {
    cudaEventRecord(L->ph[3], s);  // one GPU: no exchange either way
    cudaEventRecord(L->ph[4], s);
  }

  if (shared_aside) {
    ATENIA_CUDA_TRY(cudaStreamWaitEvent(s, L->ev_join, 0));
  } else if (L->has_shared && T > 0) {
    const __nv_bfloat16* xb = x_f32 ? L->x_bf16 : static_cast<const __nv_bfloat16*>(x);
    rc = run_shared_gemms(L, xb, T, s);
    if (rc) return rc;
  }

  CombineArgs ca{};
  ca.y_rows = L->y_perm;
  ca.inv_perm = L->inv_perm;
  ca.topk_w = L->topk_w;
  ca.y_shared = L->has_shared ? L->y_shared : nullptr;
  ca.gate_scale = gated ? L->gate_scale : nullptr;
  ca.residual = L->residual;
  ca.out = out;
  ca.out_is_f32 = out_dtype == ATENIA_IO_F32;
  ca.T = T;
  ca.k = k;
  ca.d = c.d_model;
  rc = launch_combine(ca, s);
  if (rc) return rc;
  if (L->timing) {
    cudaEventRecord(L->ph[5], s);
    L->ph_valid = true;
  }

  if (aux) {
    if (aux->topk_idx)
      ATENIA_CUDA_TRY(cudaMemcpyAsync(aux->topk_idx, L->topk_idx, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    if (aux->topk_w)
      ATENIA_CUDA_TRY(cudaMemcpyAsync(aux->topk_w, L->topk_w, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    if (aux->perm) ATENIA_CUDA_TRY(cudaMemcpyAsync(aux->perm, L->perm, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    if (aux->expert_offsets)
      ATENIA_CUDA_TRY(cudaMemcpyAsync(aux->expert_offsets, L->expert_offsets, (size_t)(c.num_experts + 1) * 4,
                                      cudaMemcpyDeviceToDevice, s));
  }
  return ATENIA_OK;
}

int atenia_moe_block_forward(AteniaMoeLayer* L, const float* x, const float* gamma, float eps, int T, float* out,
                             void* stream) {
  if (!L) return ATENIA_ERR_NULL;
  if (!L->weights_set) return ATENIA_ERR_STATE;
  if (T < 0 || !(eps >= 0.f)) return ATENIA_ERR_SHAPE;
  if (T > L->cfg.max_tokens) return ATENIA_ERR_CAPACITY;
  if (T > 0 && (!x || !out)) return ATENIA_ERR_NULL;
  if (!L->block_normed) {
    ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&L->block_normed),
                               (size_t)L->cfg.max_tokens * (size_t)L->cfg.d_model * sizeof(float)));
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = launch_rmsnorm_rows(x, gamma, eps, L->block_normed, T, L->cfg.d_model, s);
  if (rc) return rc;
  L->residual = x;  // added last by the combine kernel: out = x + MoE(h)
  rc = forward_impl(L, L->block_normed, ATENIA_IO_F32, T, out, ATENIA_IO_F32, nullptr, stream, nullptr, nullptr);
  L->residual = nullptr;
  return rc;
}

int atenia_moe_check(AteniaMoeLayer* L, void* stream) {
  if (!L) return ATENIA_ERR_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (L->cfg.ep_world > 1 && ep_ready(L)) {
    // every expert-parallel forward holds collectives: wait with the deadline, not for ever
    int wrc = ep_bounded_wait(L, s);
    if (wrc) return wrc;
  } else {
    ATENIA_CUDA_TRY(cudaStreamSynchronize(s));
  }
  DeviceError he{};
  ATENIA_CUDA_TRY(cudaMemcpy(&he, L->d_err, sizeof(he), cudaMemcpyDeviceToHost));
  if (he.code != 0) {
    ATENIA_CUDA_TRY(cudaMemset(L->d_err, 0, sizeof(DeviceError)));
    return he.code;
  }
  return ATENIA_OK;
}

int atenia_moe_forward_sync(AteniaMoeLayer* L, const void* x, int x_dtype, int T, void* out, int out_dtype,
                            const AteniaMoeAux* aux, void* stream) {
  int rc = atenia_moe_forward(L, x, x_dtype, T, out, out_dtype, aux, stream);
  if (rc) return rc;
  return atenia_moe_check(L, stream);
}

int atenia_moe_route_from_logits(AteniaMoeLayer* L, const float* logits, int T, int32_t* topk_idx, float* topk_w,
                                 int32_t* perm, int32_t* inv_perm, int32_t* expert_offsets, void* stream) {
  if (!L || !logits || !topk_idx || !topk_w) return ATENIA_ERR_NULL;
  if (T < 0) return ATENIA_ERR_SHAPE;
  if (T > L->cfg.max_tokens) return ATENIA_ERR_CAPACITY;
  if (T == 0) return ATENIA_OK;
  const AteniaMoeConfig& c = L->cfg;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = c.router_mode == ATENIA_ROUTER_V3
               ? launch_v3_route(logits, L->d_escore, T, c.num_experts, c.experts_per_token, c.n_group, c.topk_group,
                                 c.renormalize, c.routed_scaling_factor, topk_idx, topk_w, L->d_err, s)
               : launch_route_from_logits(logits, T, c.num_experts, c.experts_per_token, c.renormalize, topk_idx,
                                          topk_w, L->d_err, s);
  if (rc) return rc;
  if (perm || inv_perm || expert_offsets) {
    const int n = T * c.experts_per_token;
    DispatchArgs da{};
    da.topk_idx = topk_idx;
    da.n = n;
    da.E = c.num_experts;
    da.block_counts = L->block_counts;
    da.block_base = L->block_base;
    da.expert_offsets = L->expert_offsets;
    da.perm = L->perm;
    da.inv_perm = L->inv_perm;
    da.extra_offsets = nullptr;
    da.T = T;
    da.err = L->d_err;
    rc = launch_dispatch(da, s);
    if (rc) return rc;
    if (perm) ATENIA_CUDA_TRY(cudaMemcpyAsync(perm, L->perm, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    if (inv_perm) ATENIA_CUDA_TRY(cudaMemcpyAsync(inv_perm, L->inv_perm, (size_t)n * 4, cudaMemcpyDeviceToDevice, s));
    if (expert_offsets)
      ATENIA_CUDA_TRY(cudaMemcpyAsync(expert_offsets, L->expert_offsets, (size_t)(c.num_experts + 1) * 4,
                                      cudaMemcpyDeviceToDevice, s));
  }
  return ATENIA_OK;
}

const char* atenia_moe_status_str(int status) {
  switch (status) {
    case ATENIA_OK: return "ok";
    case ATENIA_ERR_NULL: return "a required pointer is NULL";
    case ATENIA_ERR_SHAPE: return "sizes violate a stated constraint";
    case ATENIA_ERR_CAPACITY: return "more tokens than the layer's max_tokens";
    case ATENIA_ERR_STATE: return "layer not ready (weights or expert-parallel group not set)";
    case ATENIA_ERR_LAYER_NOT_FOUND: return "moe layer id not found";
    case ATENIA_ERR_DIM_MISMATCH: return "input length is not a positive multiple of d_model";
    case ATENIA_ERR_UNSUPPORTED: return "not supported by this build";
    case ATENIA_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    case ATENIA_ERR_ROUTING: return "routing weights non-finite or selected sum <= 0";
    case ATENIA_ERR_NCCL: return "an NCCL call failed";
    case ATENIA_ERR_DRIVER: return "tensor-map encode or driver entry point unavailable";
    case ATENIA_ERR_IO: return "a tier file is missing or could not be read";
    case ATENIA_ERR_TIER_FORMAT: return "tier file length matches none of its encodings (or not the one asked for)";
    case ATENIA_ERR_POLICY:
      return "the selected numeric policy (certified / strict) keeps the MoE block on the host's CPU arms";
    case ATENIA_ERR_SCRATCH_LIMIT:
      return "request exceeds the fixed scratch of atenia_moe_dispatch_noalloc (T*k <= 65536, E <= 128)";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown status";
}

uint64_t atenia_moe_counter(int which) {
  if (which < 0 || which >= 8) return 0;
  return g_counters[which].load();
}

int atenia_moe_enable_timing(AteniaMoeLayer* L, int enable) {
  if (!L) return ATENIA_ERR_NULL;
  L->timing = enable != 0;
  for (bool& v : L->ev_valid) v = false;
  L->ph_valid = false;
  return ATENIA_OK;
}

int atenia_moe_last_recv_rows(AteniaMoeLayer* L) {
  if (!L) return -1;
  if (L->ep_direct && L->d_gemm_offsets) {
    // the direct exchange keeps the count on the device: fetch it (synchronous; diagnostics only)
    int32_t v = -1;
    if (cudaMemcpy(&v, L->d_gemm_offsets + L->e_local, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    return v;
  }
  return L->last_recv_rows;
}

float atenia_moe_last_phase_ms(AteniaMoeLayer* L, int which) {
  if (!L || which < 0 || which > 5 || !L->ph_valid) return -1.0f;
  float ms = -1.0f;
  const int a = which == 5 ? 0 : which, b = which == 5 ? 5 : which + 1;
  if (cudaEventElapsedTime(&ms, L->ph[a], L->ph[b]) != cudaSuccess) return -1.0f;
  return ms;
}

float atenia_moe_last_gemm_ms(AteniaMoeLayer* L, int which) {
  if (!L || which < 0 || which > 3 || !L->ev_valid[which]) return -1.0f;
  static const int first[4] = {0, 1, 3, 4};
  float ms = -1.0f;
  if (cudaEventElapsedTime(&ms, L->ev[first[which]], L->ev[first[which] + 1]) != cudaSuccess) return -1.0f;
  return ms;
}

}  // extern "C"
