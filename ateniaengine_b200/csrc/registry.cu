// Operator registry: the host-memory interface of the reference's graph op
// (register_real_moe_layer / execute_real_moe_layer, src/moe/graph_op.rs:221-350).
// Ids are append-only and stable for the process; one mutex guards the table and is held across a
// forward, like the reference's registry lock (src/moe/graph_op.rs:304-316).
#include <cstdlib>
#include <mutex>
#include <vector>

#include "layer.cuh"

namespace atenia {
namespace {

struct Registered {
  AteniaMoeLayer* layer = nullptr;
  bool owns_layer = true;
  std::vector<void*> weights;  // device buffers owned by the registry entry
  void* d_in = nullptr;        // [max_tokens, d] f32
  void* d_out = nullptr;
  cudaStream_t stream = nullptr;
  // copy/compute overlap (on request): second pair of staging buffers, copy streams, events
  void* d_in2 = nullptr;
  void* d_out2 = nullptr;
  cudaStream_t s_h2d = nullptr, s_d2h = nullptr;
  cudaEvent_t ev_in_ready[2] = {}, ev_in_free[2] = {}, ev_out_ready[2] = {}, ev_out_free[2] = {};
  bool pipe_ready = false;
  // timings of the pipelined calls (forward of each piece, one copy in) that refine the sub-batch plan
  static constexpr int kMaxTimed = 8;
  cudaEvent_t ev_f0[kMaxTimed] = {}, ev_f1[kMaxTimed] = {}, ev_c0 = nullptr, ev_c1 = nullptr;
  ExecFit fit;
  // the cut of the last pipelined call: kept for a batch of the same size unless a new one is modelled
  // at least 3 % faster (timing noise must not make the cut flip from call to call)
  size_t last_n = 0;
  std::vector<uint64_t> last_pieces;
};

std::mutex g_mu;
std::vector<Registered> g_layers;

// Upload a host f32 matrix and store it as bf16 (round to nearest even) or per-row int8 + scales.
int upload_matrix(const float* host, size_t rows, size_t cols, bool int8, Registered& reg, const void** w_out,
                  const float** s_out, float* staging) {
  if (!host) return ATENIA_ERR_NULL;
  const size_t n = rows * cols;
  ATENIA_CUDA_TRY(cudaMemcpy(staging, host, n * sizeof(float), cudaMemcpyHostToDevice));
  count_bytes(ATENIA_COUNTER_H2D_BYTES, n * sizeof(float));
  if (int8) {
    int8_t* q = nullptr;
    float* sc = nullptr;
    ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&q), n));
    reg.weights.push_back(q);
    ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&sc), rows * sizeof(float)));
    reg.weights.push_back(sc);
    int rc = atenia_quantize_per_row_i8(staging, (int64_t)rows, (int64_t)cols, q, sc, nullptr);
    if (rc) return rc;
    *w_out = q;
    *s_out = sc;
  } else {
    __nv_bfloat16* b = nullptr;
    ATENIA_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&b), n * sizeof(__nv_bfloat16)));
    reg.weights.push_back(b);
    int rc = launch_f32_to_bf16(staging, b, (int64_t)n, nullptr);
    if (rc) return rc;
    *w_out = b;
    *s_out = nullptr;
  }
  ATENIA_CUDA_TRY(cudaDeviceSynchronize());
  return ATENIA_OK;
}

void release(Registered& r) {
  if (r.layer && r.owns_layer) atenia_moe_destroy(r.layer);
  for (void* p : r.weights) cudaFree(p);
  if (r.d_in) cudaFree(r.d_in);
  if (r.d_out) cudaFree(r.d_out);
  if (r.stream) cudaStreamDestroy(r.stream);
  if (r.d_in2) cudaFree(r.d_in2);
  if (r.d_out2) cudaFree(r.d_out2);
  if (r.s_h2d) cudaStreamDestroy(r.s_h2d);
  if (r.s_d2h) cudaStreamDestroy(r.s_d2h);
  for (int i = 0; i < 2; ++i) {
    if (r.ev_in_ready[i]) cudaEventDestroy(r.ev_in_ready[i]);
    if (r.ev_in_free[i]) cudaEventDestroy(r.ev_in_free[i]);
    if (r.ev_out_ready[i]) cudaEventDestroy(r.ev_out_ready[i]);
    if (r.ev_out_free[i]) cudaEventDestroy(r.ev_out_free[i]);
  }
  for (int i = 0; i < Registered::kMaxTimed; ++i) {
    if (r.ev_f0[i]) cudaEventDestroy(r.ev_f0[i]);
    if (r.ev_f1[i]) cudaEventDestroy(r.ev_f1[i]);
  }
  if (r.ev_c0) cudaEventDestroy(r.ev_c0);
  if (r.ev_c1) cudaEventDestroy(r.ev_c1);
  r = Registered();
}

// execute_real_moe_layer cuts a large input into sub-batches and overlaps the host->device copy of
// sub-batch i+1 and the device->host copy of sub-batch i-1 with the forward of sub-batch i (two staging
// buffers each way, two copy streams, events).  The forwards themselves stay in order on one stream: the
// layer has one workspace.  Host buffers must be pinned for the copies to be asynchronous.
// The cut comes from plan_exec_pieces (planner.cu): a layer that is slower than the PCIe link gets a short
// piece at each end and the bulk in the middle, a layer that is faster gets equal pieces, a small batch
// stays whole.  The first call plans with the analytical model; every pipelined call times the forward of
// each of its pieces and one copy in, and the next call plans with the line fitted to those timings.  ATENIA_MOE_EXEC_CHUNK=<tokens> pins one sub-batch size for all, 0 turns the overlap off.
long exec_chunk_setting() {
  static const long v = [] {
    const char* e = std::getenv("ATENIA_MOE_EXEC_CHUNK");
    if (!e) return -1L;
    const long n = std::atol(e);
    return n > 0 ? n : 0L;
  }();
  return v;
}

// sub-batch sizes of one call (fewer than two: no overlap, one pass per max_tokens)
std::vector<size_t> exec_schedule(Registered& r, size_t n, size_t cap) {
  const AteniaMoeConfig& cfg = r.layer->cfg;
  std::vector<size_t> out;
  const long set = exec_chunk_setting();
  if (set == 0) return out;
  if (set < 0) {
    std::vector<uint64_t> plan = plan_exec_pieces(cfg, (uint64_t)n, (uint64_t)cap, &r.fit);
    if (r.last_n == n && !r.last_pieces.empty() && plan != r.last_pieces &&
        model_exec_ms(cfg, plan, &r.fit) > 0.97 * model_exec_ms(cfg, r.last_pieces, &r.fit))
      plan = r.last_pieces;
    r.last_n = n;
    r.last_pieces = plan;
    for (uint64_t v : plan) out.push_back((size_t)v);
    return out;
  }
  const size_t chunk = (size_t)set > cap ? cap : (size_t)set;
  if (n <= chunk) return out;
  for (size_t t0 = 0; t0 < n; t0 += chunk) out.push_back(n - t0 < chunk ? n - t0 : chunk);
  return out;
}

int ensure_pipe(Registered& r) {
  if (r.pipe_ready) return ATENIA_OK;
  const size_t io = (size_t)r.layer->cfg.max_tokens * (size_t)r.layer->cfg.d_model * sizeof(float);
  ATENIA_CUDA_TRY(cudaMalloc(&r.d_in2, io));
  ATENIA_CUDA_TRY(cudaMalloc(&r.d_out2, io));
  ATENIA_CUDA_TRY(cudaStreamCreateWithFlags(&r.s_h2d, cudaStreamNonBlocking));
  ATENIA_CUDA_TRY(cudaStreamCreateWithFlags(&r.s_d2h, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) {
    ATENIA_CUDA_TRY(cudaEventCreateWithFlags(&r.ev_in_ready[i], cudaEventDisableTiming));
    ATENIA_CUDA_TRY(cudaEventCreateWithFlags(&r.ev_in_free[i], cudaEventDisableTiming));
    ATENIA_CUDA_TRY(cudaEventCreateWithFlags(&r.ev_out_ready[i], cudaEventDisableTiming));
    ATENIA_CUDA_TRY(cudaEventCreateWithFlags(&r.ev_out_free[i], cudaEventDisableTiming));
  }
  for (int i = 0; i < Registered::kMaxTimed; ++i) {
    ATENIA_CUDA_TRY(cudaEventCreate(&r.ev_f0[i]));
    ATENIA_CUDA_TRY(cudaEventCreate(&r.ev_f1[i]));
  }
  ATENIA_CUDA_TRY(cudaEventCreate(&r.ev_c0));
  ATENIA_CUDA_TRY(cudaEventCreate(&r.ev_c1));
  r.pipe_ready = true;
  return ATENIA_OK;
}

int execute_pipelined(Registered& r, const float* input, float* output, const std::vector<size_t>& pieces,
                      int convention) {
  int rc = ensure_pipe(r);
  if (rc) return rc;
  const size_t d = (size_t)r.layer->cfg.d_model;
  void* din[2] = {r.d_in, r.d_in2};
  void* dout[2] = {r.d_out, r.d_out2};
  // the copy in that is timed: the largest piece's (it overlaps a forward, as most copies of a call do)
  size_t timed_copy = 0;
  for (size_t i = 1; i < pieces.size(); ++i)
    if (pieces[i] > pieces[timed_copy]) timed_copy = i;
  size_t t0 = 0;
  for (size_t i = 0; i < pieces.size(); t0 += pieces[i], ++i) {
    const size_t tn = pieces[i];
    const size_t bytes = tn * d * sizeof(float);
    const int b = (int)(i & 1);
    // host -> device, once the forward that last read this input buffer is done
    if (i >= 2) ATENIA_CUDA_TRY(cudaStreamWaitEvent(r.s_h2d, r.ev_in_free[b], 0));
    const bool time_copy = i == timed_copy;
    if (time_copy) ATENIA_CUDA_TRY(cudaEventRecord(r.ev_c0, r.s_h2d));
    ATENIA_CUDA_TRY(cudaMemcpyAsync(din[b], input + t0 * d, bytes, cudaMemcpyHostToDevice, r.s_h2d));
    if (time_copy) ATENIA_CUDA_TRY(cudaEventRecord(r.ev_c1, r.s_h2d));
    ATENIA_CUDA_TRY(cudaEventRecord(r.ev_in_ready[b], r.s_h2d));
    // forward, once its input has landed and the copy that last read this output buffer is done
    ATENIA_CUDA_TRY(cudaStreamWaitEvent(r.stream, r.ev_in_ready[b], 0));
    if (i >= 2) ATENIA_CUDA_TRY(cudaStreamWaitEvent(r.stream, r.ev_out_free[b], 0));
    if (i < (size_t)Registered::kMaxTimed) ATENIA_CUDA_TRY(cudaEventRecord(r.ev_f0[i], r.stream));
    rc = atenia_moe_forward_with(r.layer, din[b], ATENIA_IO_F32, (int)tn, dout[b], ATENIA_IO_F32, nullptr, r.stream,
                                 convention);
    if (rc) break;
    if (i < (size_t)Registered::kMaxTimed) ATENIA_CUDA_TRY(cudaEventRecord(r.ev_f1[i], r.stream));
    ATENIA_CUDA_TRY(cudaEventRecord(r.ev_in_free[b], r.stream));
    ATENIA_CUDA_TRY(cudaEventRecord(r.ev_out_ready[b], r.stream));
    // device -> host
    ATENIA_CUDA_TRY(cudaStreamWaitEvent(r.s_d2h, r.ev_out_ready[b], 0));
    ATENIA_CUDA_TRY(cudaMemcpyAsync(output + t0 * d, dout[b], bytes, cudaMemcpyDeviceToHost, r.s_d2h));
    ATENIA_CUDA_TRY(cudaEventRecord(r.ev_out_free[b], r.s_d2h));
    count_bytes(ATENIA_COUNTER_H2D_BYTES, bytes);
    count_bytes(ATENIA_COUNTER_D2H_BYTES, bytes);
  }
  // everything issued must finish before the buffers are reused or the caller reads its output
  cudaError_t e1 = cudaStreamSynchronize(r.s_h2d), e2 = cudaStreamSynchronize(r.stream),
              e3 = cudaStreamSynchronize(r.s_d2h);
  if (rc) return rc;
  if (e1 != cudaSuccess) return (int)e1;
  if (e2 != cudaSuccess) return (int)e2;
  if (e3 != cudaSuccess) return (int)e3;
  {
    // what this call took refines the plan of the next one
    uint64_t tok[Registered::kMaxTimed];
    float ms[Registered::kMaxTimed];
    int np = 0;
    for (size_t i = 0; i < pieces.size() && i < (size_t)Registered::kMaxTimed; ++i, ++np) {
      tok[np] = pieces[i];
      if (cudaEventElapsedTime(&ms[np], r.ev_f0[i], r.ev_f1[i]) != cudaSuccess) ms[np] = 0.f;
    }
    float cms = 0.f;
    if (cudaEventElapsedTime(&cms, r.ev_c0, r.ev_c1) != cudaSuccess) cms = 0.f;
    update_exec_fit(r.layer->cfg, tok, ms, np, pieces[timed_copy], cms, &r.fit);
  }
  return atenia_moe_check(r.layer, r.stream);
}

}  // namespace
}  // namespace atenia

using namespace atenia;

extern "C" {

int64_t atenia_register_real_moe_layer(const AteniaHostMoeLayer* h) {
  if (!h || !h->w_router || !h->w_gate || !h->w_up || !h->w_down) return ATENIA_ERR_NULL;
  AteniaMoeConfig cfg = h->config;
  if (cfg.max_tokens <= 0) cfg.max_tokens = 4096;
  if (cfg.ep_world <= 0) {
    cfg.ep_world = 1;
    cfg.ep_rank = 0;
  }
  if (cfg.ep_world != 1) return ATENIA_ERR_UNSUPPORTED;  // the registry path is single GPU
  Registered reg;
  int rc = atenia_moe_create(&cfg, &reg.layer);
  if (rc) return rc;
  const size_t E = (size_t)cfg.num_experts, d = (size_t)cfg.d_model, F = (size_t)cfg.d_ff,
               Fs = (size_t)cfg.shared_d_ff;
  const bool q = cfg.weight_dtype == ATENIA_W_INT8_ROW;
  size_t stage_elems = E * d;
  if (F * d > stage_elems) stage_elems = F * d;
  if (Fs * d > stage_elems) stage_elems = Fs * d;
  float* staging = nullptr;
  cudaError_t ce = cudaMalloc(reinterpret_cast<void**>(&staging), stage_elems * sizeof(float));
  if (ce != cudaSuccess) {
    release(reg);
    return (int)ce;
  }
  std::vector<const void*> pg(E), pu(E), pd(E);
  std::vector<const float*> sg(E), su(E), sd(E);
  AteniaMoeWeights w{};
  float* d_router = nullptr;
  float* d_gate_vec = nullptr;
  float* d_escore = nullptr;
  auto fail = [&](int code) -> int64_t {
    cudaFree(staging);
    if (d_router) cudaFree(d_router);
    if (d_gate_vec) cudaFree(d_gate_vec);
    if (d_escore) cudaFree(d_escore);
    release(reg);
    return code;
  };
  ce = cudaMalloc(reinterpret_cast<void**>(&d_router), E * d * sizeof(float));
  if (ce != cudaSuccess) return fail((int)ce);
  ce = cudaMemcpy(d_router, h->w_router, E * d * sizeof(float), cudaMemcpyHostToDevice);
  if (ce != cudaSuccess) return fail((int)ce);
  w.w_router = d_router;
  for (size_t e = 0; e < E; ++e) {
    rc = upload_matrix(h->w_gate[e], F, d, q, reg, &pg[e], &sg[e], staging);
    if (!rc) rc = upload_matrix(h->w_up[e], F, d, q, reg, &pu[e], &su[e], staging);
    if (!rc) rc = upload_matrix(h->w_down[e], d, F, q, reg, &pd[e], &sd[e], staging);
    if (rc) return fail(rc);
  }
  w.w_gate = pg.data();
  w.w_up = pu.data();
  w.w_down = pd.data();
  w.s_gate = sg.data();
  w.s_up = su.data();
  w.s_down = sd.data();
  if (Fs > 0) {
    rc = upload_matrix(h->shared_w_gate, Fs, d, q, reg, &w.shared_w_gate, &w.shared_s_gate, staging);
    if (!rc) rc = upload_matrix(h->shared_w_up, Fs, d, q, reg, &w.shared_w_up, &w.shared_s_up, staging);
    if (!rc) rc = upload_matrix(h->shared_w_down, d, Fs, q, reg, &w.shared_w_down, &w.shared_s_down, staging);
    if (rc) return fail(rc);
    if (h->shared_gate_vec) {  // kept even when the layer's own convention is ungated (execute_..._with)
      ce = cudaMalloc(reinterpret_cast<void**>(&d_gate_vec), d * sizeof(float));
      if (ce == cudaSuccess) ce = cudaMemcpy(d_gate_vec, h->shared_gate_vec, d * sizeof(float), cudaMemcpyHostToDevice);
      if (ce != cudaSuccess) return fail((int)ce);
      w.shared_gate_vec = d_gate_vec;
    }
  }
  if (h->e_score_bias && cfg.router_mode == ATENIA_ROUTER_V3) {
    ce = cudaMalloc(reinterpret_cast<void**>(&d_escore), E * sizeof(float));
    if (ce == cudaSuccess) ce = cudaMemcpy(d_escore, h->e_score_bias, E * sizeof(float), cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) return fail((int)ce);
    w.e_score_bias = d_escore;
  }
  rc = atenia_moe_set_weights(reg.layer, &w);
  if (rc) return fail(rc);
  cudaFree(staging);
  cudaFree(d_router);  // copied by set_weights
  if (d_gate_vec) cudaFree(d_gate_vec);
  if (d_escore) cudaFree(d_escore);
  const size_t io = (size_t)cfg.max_tokens * d * sizeof(float);
  ce = cudaMalloc(&reg.d_in, io);
  if (ce == cudaSuccess) ce = cudaMalloc(&reg.d_out, io);
  if (ce == cudaSuccess) ce = cudaStreamCreateWithFlags(&reg.stream, cudaStreamNonBlocking);
  if (ce != cudaSuccess) {
    release(reg);
    return (int)ce;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_layers.push_back(reg);
  return (int64_t)g_layers.size() - 1;
}

int64_t atenia_register_resident_moe_layer(AteniaMoeLayer* layer) {
  if (!layer) return ATENIA_ERR_NULL;
  if (!layer->weights_set || layer->cfg.ep_world != 1) return ATENIA_ERR_STATE;
  Registered reg;
  reg.layer = layer;
  reg.owns_layer = false;
  cudaError_t ce = cudaSetDevice(layer->device);
  const size_t io = (size_t)layer->cfg.max_tokens * (size_t)layer->cfg.d_model * sizeof(float);
  if (ce == cudaSuccess) ce = cudaMalloc(&reg.d_in, io);
  if (ce == cudaSuccess) ce = cudaMalloc(&reg.d_out, io);
  if (ce == cudaSuccess) ce = cudaStreamCreateWithFlags(&reg.stream, cudaStreamNonBlocking);
  if (ce != cudaSuccess) {
    release(reg);
    return (int)ce;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_layers.push_back(reg);
  return (int64_t)g_layers.size() - 1;
}

int atenia_execute_real_moe_layer(int64_t layer_id, const float* input, size_t len, float* output) {
  return atenia_execute_real_moe_layer_with(layer_id, input, len, output, ATENIA_CONVENTION_LAYER);
}

int atenia_execute_real_moe_layer_with(int64_t layer_id, const float* input, size_t len, float* output,
                                       int convention) {
  {
    // a host that selected the certified or strict numeric policy runs its own CPU arm
    const int prc = atenia_numeric_policy_gate();
    if (prc) return prc;
  }
  if (convention != ATENIA_CONVENTION_LAYER && convention != ATENIA_CONVENTION_ATENIA &&
      convention != ATENIA_CONVENTION_HF_QWEN)
    return ATENIA_ERR_SHAPE;
  std::lock_guard<std::mutex> lk(g_mu);
  if (layer_id < 0 || (size_t)layer_id >= g_layers.size() || !g_layers[(size_t)layer_id].layer)
    return ATENIA_ERR_LAYER_NOT_FOUND;
  Registered& r = g_layers[(size_t)layer_id];
  const size_t d = (size_t)r.layer->cfg.d_model;
  if (len == 0 || len % d != 0) return ATENIA_ERR_DIM_MISMATCH;
  if (!input || !output) return ATENIA_ERR_NULL;
  ATENIA_CUDA_TRY(cudaSetDevice(r.layer->device));
  const size_t n = len / d, cap = (size_t)r.layer->cfg.max_tokens;
  {
    const std::vector<size_t> pieces = exec_schedule(r, n, cap);
    if (pieces.size() > 1) return execute_pipelined(r, input, output, pieces, convention);
  }
  for (size_t t0 = 0; t0 < n; t0 += cap) {
    const size_t tn = n - t0 < cap ? n - t0 : cap;
    const size_t bytes = tn * d * sizeof(float);
    ATENIA_CUDA_TRY(cudaMemcpyAsync(r.d_in, input + t0 * d, bytes, cudaMemcpyHostToDevice, r.stream));
    int rc = atenia_moe_forward_with(r.layer, r.d_in, ATENIA_IO_F32, (int)tn, r.d_out, ATENIA_IO_F32, nullptr,
                                     r.stream, convention);
    if (rc) return rc;
    ATENIA_CUDA_TRY(cudaMemcpyAsync(output + t0 * d, r.d_out, bytes, cudaMemcpyDeviceToHost, r.stream));
    count_bytes(ATENIA_COUNTER_H2D_BYTES, bytes);
    count_bytes(ATENIA_COUNTER_D2H_BYTES, bytes);
  }
  return atenia_moe_check(r.layer, r.stream);
}

AteniaMoeLayer* atenia_get_real_moe_layer(int64_t layer_id) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (layer_id < 0 || (size_t)layer_id >= g_layers.size()) return nullptr;
  return g_layers[(size_t)layer_id].layer;
}

}  // extern "C"
