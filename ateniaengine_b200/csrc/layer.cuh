// Internal definition of AteniaMoeLayer (shared by moe_layer.cu, ep.cu, registry.cu).
#pragma once
#include <memory>
#include <vector>

#include "common.cuh"

namespace atenia {
struct EpComm;  // ep.cu: an NCCL communicator, destroyed with its last holder
}

struct AteniaMoeLayer {
  AteniaMoeConfig cfg{};
  int device = 0;
  int num_sms = 0;
  int e_local = 0;   // experts owned by this rank
  int e_begin = 0;   // first owned expert id
  int n_groups = 0;  // GEMM groups per launch: e_local (single GPU) or ep_world * e_local
  bool weights_set = false;
  bool use_check_gemm = false;  // diagnostic: CUDA-core contraction instead of tcgen05
  bool use_gemv = true;         // small calls take the matrix-vector kernel (decode_gemv.cu)
  int gemv_rows = 2;   // calls of at most this many rows take it
  bool timing = false;
  const float* residual = nullptr;  // set by a stack around one forward: added by the combine kernel
  float* block_normed = nullptr;    // [max_tokens, d] f32, allocated by the first atenia_moe_block_forward
  // INT8: 0 = pick per call (tensor-memory operand kernel of w8_gemm.cu for small groups, the 256-row
  // tile kernel of w8_gemm_m256.cu for large ones), 1 = always the small-group kernel,
  // 2 = always the 128-row shared-memory widening kernel (grouped_gemm.cu)
  int w8_mode = 0;
  // bf16: 0 = pick per call (CTA-pair kernel once groups average >= 512 rows), 1 = always pairs,
  // 2 = always the single-CTA kernel
  int pair_mode = 0;
  // bf16 stream-K decode kernel: -1 = calls of at most 16 rows, 1 = every call of at most 128 rows
  // (ATENIA_MOE_BF16_DECODE=1), 0 = never (=0, or INT8 weights)
  int bf16_decode = -1;
  // router kernel: -1 by size, 0 CUDA cores (router.cu), 1 f64 tensor cores (router_dmma.cu),
  // 2 split-k for batches of at most sk_tokens (router_splitk.cu); see atenia_moe_create
  int router_variant = -1;
  double* sk_part = nullptr;
  double* sk_gate = nullptr;
  unsigned int* sk_counters = nullptr;
  int sk_tokens = 0;

  // weights (device)
  float* d_router = nullptr;    // [E, d]
  float* d_bias = nullptr;      // [E]
  float* d_gate_vec = nullptr;  // [d]
  float* d_escore = nullptr;    // [E] V3 e_score_correction_bias (zeros if none given)
  float* logits_ws = nullptr;   // [max_tokens, E] V3: logits between the router and the V3 selection
  bool has_bias = false, has_shared = false;
  bool gate_vec_bound = false;  // a shared gate vector was given with the weights
  bool has_gate_vec = false;    // ... and the layer's own convention uses it
  CUtensorMap* d_tm_gate = nullptr;  // [n_groups]
  CUtensorMap* d_tm_up = nullptr;
  CUtensorMap* d_tm_down = nullptr;
  CUtensorMap* d_tm_shared = nullptr;  // [3]: gate, up, down
  // INT8 only: the same matrices described with the 64-byte swizzle the tensor-memory kernel reads
  CUtensorMap* d_tm_gate_sw = nullptr;
  CUtensorMap* d_tm_up_sw = nullptr;
  CUtensorMap* d_tm_down_sw = nullptr;
  CUtensorMap* d_tm_shared_sw = nullptr;
  const float** d_sc_gate = nullptr;   // [n_groups] device pointers (INT8) or null
  const float** d_sc_up = nullptr;
  const float** d_sc_down = nullptr;
  const float** d_sc_shared = nullptr;  // [3]
  const void** d_p_gate = nullptr;      // [n_groups] raw matrix pointers (checking kernel)
  const void** d_p_up = nullptr;
  const void** d_p_down = nullptr;
  const void** d_p_shared = nullptr;  // [3]
  std::vector<void*> owned;           // device buffers this layer allocated for weights

  // workspace (device), sized by cfg.max_tokens
  int rows_cap = 0;  // rows of the dispatch-ordered buffers
  int32_t* topk_idx = nullptr;
  float* topk_w = nullptr;
  float* gate_scale = nullptr;
  int32_t* perm = nullptr;
  int32_t* inv_perm = nullptr;
  int32_t* expert_offsets = nullptr;  // [E + 1]
  int32_t* shared_offsets = nullptr;  // [2]
  int32_t* block_counts = nullptr;
  int32_t* block_base = nullptr;
  __nv_bfloat16* x_perm = nullptr;  // [rows_cap, d]
  __nv_bfloat16* h = nullptr;       // [rows_cap, F]
  __nv_bfloat16* y_perm = nullptr;  // [rows_cap, d]
  __nv_bfloat16* x_bf16 = nullptr;  // [max_tokens, d]
  __nv_bfloat16* h_shared = nullptr;  // [max_tokens, Fs]
  __nv_bfloat16* y_shared = nullptr;  // [max_tokens, d]
  atenia::DeviceError* d_err = nullptr;
  float* splitk_ws = nullptr;  // stream-K partial sums of the decode kernels, 2 slots per SM
  unsigned int* splitk_cnt = nullptr;  // [kSplitKMaxTiles * 8] arrival counters of split tiles (zero between launches)
  // INT8, integer-MMA decode kernel: weight maps (box {128, 128}, 128B swizzle), digit planes [4][128][K] of
  // the token rows and of the intermediate rows with their row scales, and the planes' tensor maps
  bool w8_i8 = true;
  int i8_rows = 128;  // rows of one digit plane = the largest call the kernel takes
  CUtensorMap* d_tm_gate_i8 = nullptr;
  CUtensorMap* d_tm_up_i8 = nullptr;
  CUtensorMap* d_tm_down_i8 = nullptr;
  int8_t* dq_x = nullptr;
  int8_t* dq_h = nullptr;
  float* dq_ts_x = nullptr;
  float* dq_ts_h = nullptr;
  CUtensorMap tm_dq_x{}, tm_dq_h{};
  atenia::DigitSource i8_src{};  // the caller's batch and the permutation, when the digit kernel does the row gather
  bool i8_src_set = false;
  float* splitk_ws_shared = nullptr;  // the same for the shared expert's launches (INT8 with a shared expert)
  CUtensorMap tm_x_perm{}, tm_h{}, tm_h_shared{};

  // expert parallelism
  std::shared_ptr<atenia::EpComm> ep;  // layers of one stack may share a communicator (atenia_moe_ep_attach)
  bool ep_replicated = false;          // every rank holds the same tokens (atenia_moe_ep_set_token_layout)
  int recv_cap = 0;                    // rows of the receive-side buffers
  int last_recv_rows = -1;             // rows this rank's experts received in the last token-sharded forward
  __nv_bfloat16* recv_x = nullptr;     // [recv_cap, d]
  __nv_bfloat16* recv_h = nullptr;     // [recv_cap, F]
  __nv_bfloat16* recv_y = nullptr;     // [recv_cap, d]
  int32_t* d_counts_all = nullptr;     // [world, E] rows per (source rank, expert)
  int32_t* h_counts_all = nullptr;     // pinned host copy
  int32_t* d_group_offsets = nullptr;  // [world * e_local + 1]
  CUtensorMap tm_recv_x{}, tm_recv_h{};
  // direct exchange (atenia_moe_ep_ipc_import): rows are stored straight into the owner's receive
  // buffer and results straight back into the source's y_perm through peer mappings
  bool ep_direct = false;
  __nv_bfloat16** d_peer_recv_x = nullptr;  // device array [world]: every rank's recv_x (own entry: local)
  __nv_bfloat16** d_peer_y_perm = nullptr;  // device array [world]: every rank's y_perm
  std::vector<void*> ipc_opened;            // peer mappings to close
  int32_t* d_dst_base = nullptr;            // [E]
  int32_t* d_src_base = nullptr;            // [e_local * world]
  int32_t* d_gemm_offsets = nullptr;        // [e_local + 1] expert-major group offsets of the receive buffer
  int32_t* d_bar = nullptr;                 // [1] operand of the barrier all-reduce
  // flag synchronisation of the direct exchange (ATENIA_MOE_EP_FLAGS=1): counts and "my stores are done"
  // epochs are stored into the peers' sync buffers instead of travelling through three collectives
  bool ep_flags = false;
  uint32_t* d_sync = nullptr;        // this rank's sync buffer (own 2 MiB allocation): epochs, then counts [world, E]
  uint32_t** d_peer_sync = nullptr;  // device array [world]: every rank's sync buffer
  uint32_t* d_ep_state = nullptr;    // private: [0] epoch of the current forward, [1],[2] finished-block counters, [3] gave up
  uint64_t ep_flag_limit_ns = 20000000000ull;

  // the shared expert needs only the call's tokens: its GEMMs run on a second stream beside the routing
  // phase and, under expert parallelism, the exchanges (fork at the start, join before the combine)
  bool shared_aside = true;
  cudaStream_t aux_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;

  // timing
  cudaEvent_t ev[8] = {};
  bool ev_valid[4] = {false, false, false, false};
  // phase marks of one forward (recorded only while timing is enabled): 0 start, 1 routed and sorted
  // (rows gathered), 2 rows at their experts (after the dispatch exchange), 3 expert GEMMs done,
  // 4 results back (after the return exchange), 5 end
  cudaEvent_t ph[6] = {};
  bool ph_valid = false;
};

namespace atenia {
int ep_forward_exchange(AteniaMoeLayer* L, int T, cudaStream_t s);  // ep.cu
int ep_forward_replicated(AteniaMoeLayer* L, int n_rows, cudaStream_t s);
int ep_direct_send(AteniaMoeLayer* L, const void* x, int x_is_f32, int T, cudaStream_t s);
int ep_direct_finish(AteniaMoeLayer* L, cudaStream_t s);
bool ep_ready(const AteniaMoeLayer* L);
// Wait for `s` with the expert-parallel deadline (ATENIA_MOE_EP_TIMEOUT_S): polls the stream and the
// communicator; on a failed peer or a passed deadline aborts the communicator and returns
// ATENIA_ERR_NCCL, so a collective whose peer never arrives cannot block the host for ever.
int ep_bounded_wait(AteniaMoeLayer* L, cudaStream_t s);
void ep_destroy(AteniaMoeLayer* L);
int run_expert_gemms(AteniaMoeLayer* L, const CUtensorMap& tm_a, const CUtensorMap& tm_mid,
                     const __nv_bfloat16* a_ptr, __nv_bfloat16* mid, __nv_bfloat16* out,
                     const int32_t* group_offsets, int num_groups, int max_rows, cudaStream_t s);
}  // namespace atenia
