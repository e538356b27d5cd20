// A stack of MoE layers: x <- layer_l(x) in sequence (RealMoeStack::forward, src/moe/stack.rs:197-210),
// optionally with a residual add per layer, x <- x + layer_l(x).  Activations between layers stay in
// f32 on the device.  On a non-default stream the whole stack is captured once into a CUDA graph per
// (token count, input, output) and replayed: at decode sizes a layer is ten short launches and the
// launch overhead of 32 layers would otherwise dominate.
#include <cstdlib>
#include <vector>

#include "layer.cuh"

struct AteniaMoeStack {
  std::vector<AteniaMoeLayer*> layers;
  bool residual = false;
  bool prenorm = false;       // residual == 2: x <- x + layer(rmsnorm(x))
  float* normed = nullptr;    // [max_tokens, d] f32
  std::vector<const float*> gammas;  // per layer device [d] gain of the norm, or empty = unit gain
  float eps = 1e-5f;
  int d_model = 0;
  int max_tokens = 0;
  float* buf[2] = {nullptr, nullptr};  // ping-pong [max_tokens, d] f32
  bool use_graph = true;
  // cached graph
  cudaGraphExec_t exec = nullptr;
  const void* g_x = nullptr;
  void* g_out = nullptr;
  int g_T = -1, g_xdt = -1, g_odt = -1;
  bool g_warm = false;  // the signature above has run once eagerly (one-time kernel set-up is done)
};

namespace {

// y[t, :] = (x[t, :] * inv_rms) * gamma with inv_rms = 1 / sqrt(mean(x[t, :]^2) + eps): the post-attention
// RMSNorm and its gain as the reference applies them before the MoE block (rms_norm,
// src/nn/normalization.rs:8-37, then broadcast_mul by gamma, src/moe/full_forward.rs:239-242): f32
// throughout, the normalised value rounded before the gain multiplies it.  The reference adds the
// squares in index order; here they are added by a block reduction (fixed order), which can move inv_rms
// by an ulp.  gamma == nullptr means unit gain.  One block of 1024 threads per row; a thread keeps its (up
// to two) float4 vectors in registers between the two passes, so a row of up to 8192 elements is read once.
constexpr int kNormThreads = 1024;
constexpr int kNormVecs = 2;

__global__ void __launch_bounds__(kNormThreads) rmsnorm_rows_kernel(const float* __restrict__ x,
                                                                     const float* __restrict__ gamma, float eps,
                                                                     float* __restrict__ y, int d) {
  __shared__ float red[kNormThreads / 32];
  __shared__ float s_inv;
  const float* row = x + (size_t)blockIdx.x * d;
  float* yrow = y + (size_t)blockIdx.x * d;
  // 16-byte vectors when every row starts on a 16-byte boundary
  const bool vec = (d & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  const int nvec = vec ? d / 4 : 0;
  float4 keep[kNormVecs];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kNormVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    keep[j] = v < nvec ? reinterpret_cast<const float4*>(row)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int j = 0; j < kNormVecs; ++j) {
    ss = __fmaf_rn(keep[j].x, keep[j].x, ss);
    ss = __fmaf_rn(keep[j].y, keep[j].y, ss);
    ss = __fmaf_rn(keep[j].z, keep[j].z, ss);
    ss = __fmaf_rn(keep[j].w, keep[j].w, ss);
  }
  // what the registers do not hold: the tail of a long row, or all of a row whose length is not a multiple of 4
  for (int c = (vec ? 4 * kNormVecs * kNormThreads : 0) + threadIdx.x; c < d; c += kNormThreads)
    ss = __fmaf_rn(row[c], row[c], ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = red[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) {
      const float mean_sq = __fdiv_rn(t, (float)d);
      s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
    }
  }
  __syncthreads();
  const float inv = s_inv;
  auto norm1 = [&](float xv, int c) {
    const float n = __fmul_rn(xv, inv);
    return gamma ? __fmul_rn(n, gamma[c]) : n;
  };
#pragma unroll
  for (int j = 0; j < kNormVecs; ++j) {
    const int v = threadIdx.x + j * kNormThreads;
    if (v < nvec)
      reinterpret_cast<float4*>(yrow)[v] = make_float4(norm1(keep[j].x, 4 * v), norm1(keep[j].y, 4 * v + 1),
                                                       norm1(keep[j].z, 4 * v + 2), norm1(keep[j].w, 4 * v + 3));
  }
  for (int c = (vec ? 4 * kNormVecs * kNormThreads : 0) + threadIdx.x; c < d; c += kNormThreads) yrow[c] = norm1(row[c], c);
}

}  // namespace

namespace atenia {
int launch_rmsnorm_rows(const float* x, const float* gamma, float eps, float* y, int T, int d, cudaStream_t s) {
  if (T <= 0) return ATENIA_OK;
  rmsnorm_rows_kernel<<<T, kNormThreads, 0, s>>>(x, gamma, eps, y, d);
  count_launch();
  return (int)cudaGetLastError();
}
}  // namespace atenia

namespace {

int run_layers(AteniaMoeStack* S, const void* x, int x_dtype, int T, void* out, int out_dtype, cudaStream_t s) {
  const int n = (int)S->layers.size();
  const void* cur = x;
  int cur_dt = x_dtype;
  for (int l = 0; l < n; ++l) {
    const bool last = l == n - 1;
    void* dst = last ? out : (void*)S->buf[l & 1];
    const int dst_dt = last ? out_dtype : ATENIA_IO_F32;
    AteniaMoeLayer* L = S->layers[l];
    // the residual operand is the layer's own f32 input
    const float* res = nullptr;
    if (S->residual) {
      if (cur_dt != ATENIA_IO_F32) return ATENIA_ERR_UNSUPPORTED;
      res = static_cast<const float*>(cur);
    }
    const void* in = cur;
    if (S->prenorm) {
      const float* g = S->gammas.empty() ? nullptr : S->gammas[(size_t)l];
      int nrc = atenia::launch_rmsnorm_rows(static_cast<const float*>(cur), g, S->eps, S->normed, T, S->d_model, s);
      if (nrc) return nrc;
      in = S->normed;
    }
    L->residual = res;
    int rc = atenia_moe_forward(L, in, cur_dt, T, dst, dst_dt, nullptr, s);
    L->residual = nullptr;
    if (rc) return rc;
    cur = dst;
    cur_dt = dst_dt;
  }
  return ATENIA_OK;
}

}  // namespace

extern "C" {

int atenia_moe_stack_create(AteniaMoeLayer* const* layers, int n_layers, int residual, AteniaMoeStack** out) {
  if (!layers || !out) return ATENIA_ERR_NULL;
  *out = nullptr;
  if (n_layers < 1) return ATENIA_ERR_SHAPE;
  AteniaMoeStack* S = new AteniaMoeStack();
  S->residual = residual != 0;
  S->prenorm = residual == 2;
  for (int l = 0; l < n_layers; ++l) {
    AteniaMoeLayer* L = layers[l];
    if (!L) {
      delete S;
      return ATENIA_ERR_NULL;
    }
    // expert-parallel layers qualify when their forward reads nothing on the host
    if (!L->weights_set || (L->cfg.ep_world != 1 && !L->ep_replicated && !L->ep_direct)) {
      delete S;
      return ATENIA_ERR_STATE;
    }
    if (l == 0) {
      S->d_model = L->cfg.d_model;
      S->max_tokens = L->cfg.max_tokens;
    } else {
      if (L->cfg.d_model != S->d_model) {  // MoeStackError::DModelMismatch
        delete S;
        return ATENIA_ERR_DIM_MISMATCH;
      }
      if (L->cfg.max_tokens < S->max_tokens) S->max_tokens = L->cfg.max_tokens;
    }
    S->layers.push_back(L);
  }
  const size_t bytes = (size_t)S->max_tokens * S->d_model * sizeof(float);
  for (int i = 0; i < 2; ++i) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&S->buf[i]), bytes);
    if (e != cudaSuccess) {
      atenia_moe_stack_destroy(S);
      return (int)e;
    }
  }
  if (S->prenorm) {
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&S->normed), bytes);
    if (e != cudaSuccess) {
      atenia_moe_stack_destroy(S);
      return (int)e;
    }
  }
  const char* g = std::getenv("ATENIA_MOE_STACK_GRAPH");
  S->use_graph = !(g && std::atoi(g) == 0);
  *out = S;
  return ATENIA_OK;
}

int atenia_moe_stack_set_norm(AteniaMoeStack* S, const float* const* gammas, float eps) {
  if (!S) return ATENIA_ERR_NULL;
  if (!S->prenorm) return ATENIA_ERR_STATE;
  if (!(eps >= 0.f)) return ATENIA_ERR_SHAPE;
  S->gammas.clear();
  if (gammas) S->gammas.assign(gammas, gammas + S->layers.size());
  S->eps = eps;
  if (S->exec) {  // a captured graph holds the old arguments
    cudaGraphExecDestroy(S->exec);
    S->exec = nullptr;
  }
  S->g_warm = false;
  return ATENIA_OK;
}

int atenia_moe_stack_destroy(AteniaMoeStack* S) {
  if (!S) return ATENIA_OK;
  cudaDeviceSynchronize();
  if (S->exec) cudaGraphExecDestroy(S->exec);
  for (int i = 0; i < 2; ++i)
    if (S->buf[i]) cudaFree(S->buf[i]);
  if (S->normed) cudaFree(S->normed);
  delete S;
  return ATENIA_OK;
}

int atenia_moe_stack_forward(AteniaMoeStack* S, const void* x, int x_dtype, int T, void* out, int out_dtype,
                             void* stream) {
  if (!S || !x || !out) return ATENIA_ERR_NULL;
  if (T < 0) return ATENIA_ERR_SHAPE;
  if (T > S->max_tokens) return ATENIA_ERR_CAPACITY;
  if (T == 0) return ATENIA_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  bool timing = false;
  for (AteniaMoeLayer* L : S->layers) timing = timing || L->timing;
  if (!S->use_graph || s == nullptr || timing) return run_layers(S, x, x_dtype, T, out, out_dtype, s);
  const bool same = S->g_x == x && S->g_out == out && S->g_T == T && S->g_xdt == x_dtype && S->g_odt == out_dtype;
  if (!same || !S->g_warm) {
    // first call with this signature: run eagerly (kernels do their one-time attribute set-up outside
    // of any capture), capture on the next one
    if (S->exec) {
      cudaGraphExecDestroy(S->exec);
      S->exec = nullptr;
    }
    S->g_x = x;
    S->g_out = out;
    S->g_T = T;
    S->g_xdt = x_dtype;
    S->g_odt = out_dtype;
    S->g_warm = true;
    return run_layers(S, x, x_dtype, T, out, out_dtype, s);
  }
  if (!S->exec) {
    // Everything a forward does here is launches on `s` (kernels, and with replicated-token expert
    // parallelism one NCCL all-reduce per layer), so it can be captured.
    ATENIA_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int rc = run_layers(S, x, x_dtype, T, out, out_dtype, s);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(s, &graph);
    if (rc) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    if (e != cudaSuccess) return (int)e;
    e = cudaGraphInstantiate(&S->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return (int)e;
  }
  ATENIA_CUDA_TRY(cudaGraphLaunch(S->exec, s));
  atenia::count_launch((int)S->layers.size());  // at least one kernel per layer was replayed
  return ATENIA_OK;
}

int atenia_moe_stack_check(AteniaMoeStack* S, void* stream) {
  if (!S) return ATENIA_ERR_NULL;
  int first = ATENIA_OK;
  for (AteniaMoeLayer* L : S->layers) {
    int rc = atenia_moe_check(L, stream);
    if (rc && !first) first = rc;
  }
  return first;
}

}  // extern "C"
