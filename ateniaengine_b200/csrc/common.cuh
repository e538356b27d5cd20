// Shared declarations of the MoE library's translation units (sm_100a only).
#pragma once
#include <vector>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/atenia_moe.h"

namespace atenia {

// Error word written by kernels (first error wins).  Values are the negative status codes of the
// public header; a second word keeps a site id for diagnosis.
struct DeviceError {
  int32_t code;
  int32_t site;
};

__device__ __forceinline__ void report_error(DeviceError* err, int code, int site) {
  if (err && atomicCAS(&err->code, 0, code) == 0) err->site = site;
}

// ---- bf16 helpers ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ float bf16lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ---- launch bookkeeping ---------------------------------------------------------------------
void count_launch(int n = 1);
void count_tcgen05_launch();
void count_bytes(int which, uint64_t n);

// One-time kernel attributes are per device: `flags` is a per-kernel array indexed by device ordinal.
// Returns true exactly once per (kernel, device); a benign double set under a race is harmless.
constexpr int kMaxDevices = 64;
inline bool first_use_on_current_device(bool (&flags)[kMaxDevices]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return true;
  if (flags[dev]) return false;
  flags[dev] = true;
  return true;
}

#define ATENIA_CUDA_TRY(expr)                \
  do {                                       \
    cudaError_t e__ = (expr);                \
    if (e__ != cudaSuccess) return (int)e__; \
  } while (0)

// ---- router / routing ------------------------------------------------------------------------
struct RouterArgs {
  const void* x;          // [T, d] bf16 or f32
  int x_is_f32;
  const float* w_router;  // [E, d] f32
  const float* bias;      // [E] or null
  const float* gate_vec;  // [d] or null
  int T, d, E, k, renormalize;
  int32_t* topk_idx;   // [T, k]
  float* topk_w;       // [T, k]
  float* gate_scale;   // [T] or null
  float* logits;       // [T, E] or null
  DeviceError* err;
  int variant;         // -1: by size; 0: CUDA-core f64 kernel (router.cu); 1: f64 tensor-core kernel
                       // (router_dmma.cu); 2: split-k kernel (router_splitk.cu) when T <= sk_tokens
  double* sk_part;     // variant 2 workspace (router_splitk_workspace), else null
  double* sk_gate;
  unsigned int* sk_counters;
  int sk_tokens;       // largest batch the workspace serves
};
int launch_router(const RouterArgs& a, cudaStream_t s);
int launch_router_dmma(const RouterArgs& a, cudaStream_t s);  // same contract, E <= 128, k <= 8
int launch_router_splitk(const RouterArgs& a, cudaStream_t s);  // same contract, T <= a.sk_tokens
void router_splitk_workspace(int tokens, int d, int E, size_t* part_doubles, size_t* gate_doubles, size_t* counters);
int launch_route_from_logits(const float* logits, int T, int E, int k, int renormalize,
                             int32_t* topk_idx, float* topk_w, DeviceError* err, cudaStream_t s);

// DeepSeek-V3 routing from logits (one thread per token runs v3_route_one of v3_route.cuh).
int launch_v3_route(const float* logits, const float* e_score_bias, int T, int E, int k, int n_group, int topk_group,
                    int norm_topk_prob, float scaling, int32_t* topk_idx, float* topk_w, DeviceError* err,
                    cudaStream_t s);

// ---- dispatch --------------------------------------------------------------------------------
struct DispatchArgs {
  const int32_t* topk_idx;  // [n] flat (t*k + s) -> expert
  int n;                    // T * k
  int E;
  int32_t* block_counts;  // [E, nblk] entries of each expert per block of kDispatchChunk entries
  int32_t* block_base;    // [E, nblk] exclusive scan of block_counts over the blocks
  int32_t* expert_offsets;  // [E + 1]
  int32_t* perm;            // [n]
  int32_t* inv_perm;        // [n]
  int32_t* extra_offsets;   // [2] = {0, T} for the shared-expert group, or null
  int T;
  DeviceError* err;
};
constexpr int kDispatchChunk = 256;  // flat entries per block
int launch_dispatch(const DispatchArgs& a, cudaStream_t s);

// x_perm[r, :] = bf16(x[perm[r] / k, :]) for r < *placed (device: expert_offsets[E], the rows the
// placement wrote); optionally x_bf16 = bf16(x) when x is f32.
int launch_gather_rows(const void* x, int x_is_f32, const int32_t* perm, const int32_t* placed, int n_rows, int k,
                       int d, __nv_bfloat16* x_perm, __nv_bfloat16* x_bf16, int T, cudaStream_t s);

// ---- combine ---------------------------------------------------------------------------------
struct CombineArgs {
  const __nv_bfloat16* y_rows;  // [n, d] expert outputs in dispatch order
  const int32_t* inv_perm;      // [T*k]
  const float* topk_w;          // [T*k]
  const __nv_bfloat16* y_shared;  // [T, d] or null
  const float* gate_scale;        // [T] or null (null = 1.0)
  const float* residual;          // [T, d] f32 added last, or null (layer stacks)
  void* out;
  int out_is_f32;
  int T, k, d;
};
int launch_combine(const CombineArgs& a, cudaStream_t s);

// ---- grouped GEMM ----------------------------------------------------------------------------
// One "group" is a contiguous block of rows of A multiplied by that group's own weight matrices.
//   kSwiGLU: out[r, n] = silu(A[r,:].B0_g[n,:]) * (A[r,:].B1_g[n,:])      (gate / up, N = d_ff)
//   kPlain:  out[r, n] = A[r,:].B0_g[n,:]                                   (down, N = d_model)
// B matrices are row-major [N, K] (K contiguous): the reference's weight layout.
enum GemmMode { kSwiGLU = 0, kPlain = 1 };

struct GroupedGemmArgs {
  CUtensorMap tmap_a;              // A [rows_cap, K] bf16, box {64, 128}, 128B swizzle
  const CUtensorMap* tmap_b0;      // device array [num_groups]
  const CUtensorMap* tmap_b1;      // device array [num_groups] (kSwiGLU only)
  const int32_t* group_offsets;    // device [num_groups + 1] row offsets into A / out
  int num_groups;
  int N, K;
  int mode;
  __nv_bfloat16* out;  // [rows_cap, N]
  // INT8 weights: per-group device pointers to f32 per-row scales (null for bf16)
  const float* const* scale0;  // device array [num_groups] of device pointers
  const float* const* scale1;
  DeviceError* err;
  int max_rows;  // upper bound on total rows (sizes nothing; used by the checking kernel's grid)
  int w8;        // B matrices are int8 (tensor maps of bytes), widened to bf16 inside the kernel
  float* splitk_ws;  // W8 tensor-memory kernel: workspace for stream-K partial sums (null: whole tiles only)
  // stream-K decode kernels: zeroed counters [kSplitKMaxTiles * 8] with which the kernel finishes the split
  // tiles itself (null: a second kernel adds the pieces)
  unsigned int* splitk_cnt;
  // integer-MMA decode kernel only: 2^(e - 26) per token row and the row count of one digit plane
  const float* tok_scale;
  int plane_rows;
};
int launch_grouped_gemm_tcgen05(const GroupedGemmArgs& a, int num_sms, cudaStream_t s);

// Plain CUDA-core version of the same contraction, reading the same buffers through ordinary
// pointers.  Used by the test-suite to localise a fault; never selected by the forward path.
struct GroupedGemmCheckArgs {
  const __nv_bfloat16* a;  // [rows, K]
  const void* const* b0;   // device array [num_groups] of device pointers to [N, K]
  const void* const* b1;
  int b_is_int8;
  const float* const* scale0;
  const float* const* scale1;
  const int32_t* group_offsets;
  int num_groups, N, K, mode;
  __nv_bfloat16* out;
  int max_rows;
};
int launch_grouped_gemm_check(const GroupedGemmCheckArgs& a, cudaStream_t s);
// The same contraction for calls of at most two rows in all (decode at batch 1): a CUDA-core
// matrix-vector kernel that streams the touched experts' weights once (decode_gemv.cu; it handles up to
// four rows per group, but from three rows on the tensor-core kernels are as fast).
int launch_grouped_gemv(const GroupedGemmCheckArgs& a, cudaStream_t s);
constexpr int kGemvMaxRows = 2;

int launch_f32_to_bf16(const float* src, __nv_bfloat16* dst, int64_t n, cudaStream_t s);
// p[0] = a, p[1] = b on the stream (the one-group offsets of the shared expert's GEMMs)
int launch_set_pair(int32_t* p, int32_t a, int32_t b, cudaStream_t s);
// y = (x * inv_rms(x)) * gamma per row (stack.cu); gamma may be null (unit gain)
int launch_rmsnorm_rows(const float* x, const float* gamma, float eps, float* y, int T, int d, cudaStream_t s);

// Tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
int encode_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                        uint32_t box_rows, uint32_t box_cols);
// int8 matrix [rows, cols]; unswizzled box, or 64-byte swizzle for the row-per-thread reads of the
// TMEM-operand kernel
int encode_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                      uint32_t box_cols, int swizzle64);  // swizzle64: 0 none, 1 64-byte, 2 128-byte
// W8A16 grouped GEMM with the weights as the tensor-memory operand (w8_gemm.cu).  tmap_a is the bf16
// token matrix (box {64, 128}, 128B swizzle); tmap_b0/b1 are int8 maps with the 64-byte swizzle.
int launch_grouped_gemm_w8_tmem(const GroupedGemmArgs& a, int num_sms, cudaStream_t s);
constexpr size_t kW8SplitKSlotFloats = 2 * 128 * 128;  // per CTA: two slots of this size
constexpr int kSplitKMaxTiles = 8 * 160;               // tiles a stream-K launch can have (eight rounds of the SMs)
// W8A16 for large groups (w8_gemm_m256.cu): 256-row token tiles, the widened weight tile shared by two
// M128 MMAs.  Tensor maps as for launch_grouped_gemm_tcgen05 with w8 set.
int launch_grouped_gemm_w8_m256(const GroupedGemmArgs& a, int num_sms, cudaStream_t s);
// bf16 weights, groups of at most 128 rows (bf16_decode_gemm.cu): transposed product with stream-K over
// the SMs; tmap_a / tmap_b0 / tmap_b1 are the maps of launch_grouped_gemm_tcgen05, splitk_ws as for
// the INT8 tensor-memory kernel (null: whole tiles only).
int launch_grouped_gemm_bf16_decode(const GroupedGemmArgs& a, int num_sms, cudaStream_t s);
// INT8 weights, calls of at most kI8DecodeMaxRows rows (same file): the codes are multiplied as integers
// (tcgen05 kind::i8) with the token rows split into four planes of base-128 digits by
// launch_quantize_digits.  tmap_a is the digit-plane map (uint8, box {128, 16}, 128B swizzle; plane p of
// row r at row p * plane_rows + r), tmap_b0 / tmap_b1 int8 maps with box {128, 128} and the 128B swizzle.
constexpr int kI8DecodeMaxRows = 512;      // largest call (rows of one digit plane) a layer may be set up for
constexpr int kI8DecodeDefaultRows = 128;  // ... and what a layer takes unless told otherwise
int launch_grouped_gemm_w8_i8_decode(const GroupedGemmArgs& a, int num_sms, cudaStream_t s);
// planes [4][plane_rows][K] int8 and tok_scale [plane_rows] of n_rows rows; n_rows_dev (device, may be null)
// bounds the rows that hold data.  Row r comes from row r of src.x, or -- with src.perm, the dispatch
// permutation -- from token row perm[r] / k of the caller's batch (the row gather and the digits in one pass).
struct DigitSource {
  const void* x;        // [n_src_rows, K], bf16 or f32
  int x_is_f32;
  const int32_t* perm;  // null: no gather
  int k;
  int n_src_rows;
};
int launch_quantize_digits(const DigitSource& src, const int32_t* n_rows_dev, int n_rows, int K, int plane_rows,
                           int8_t* planes, float* tok_scale, cudaStream_t s);
// bf16 weights, CTA pairs (tcgen05 cta_group::2): 256-row tiles, each CTA stages half of the weight tile
int launch_grouped_gemm_2cta(const GroupedGemmArgs& a, int num_sms, cudaStream_t s);

// Sub-batch sizes for the host-buffer operator (planner.cu): n tokens in pieces of at most cap tokens,
// chosen with a cost model of the copies and the forward; one piece means "do not overlap".  `fit`
// (optional) carries what the operator measured in its earlier calls: forward(T) = a + b T milliseconds
// and the copy time of a token.
struct ExecFit {
  double a_ms = 0.0, b_ms = 0.0, copy_token_ms = 0.0;
  bool valid = false;
};
std::vector<uint64_t> plan_exec_pieces(const AteniaMoeConfig& c, uint64_t n, uint64_t cap, const ExecFit* fit);
double model_exec_ms(const AteniaMoeConfig& c, const std::vector<uint64_t>& pieces, const ExecFit* fit);
void update_exec_fit(const AteniaMoeConfig& c, const uint64_t* tokens, const float* forward_ms, int n_pieces,
                     uint64_t copy_tokens, float copy_ms, ExecFit* fit);

}  // namespace atenia
