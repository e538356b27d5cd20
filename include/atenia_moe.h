/*
 * atenia_moe.h -- C ABI of the B200 (sm_100a) mixture-of-experts block.
 *
 * This is the boundary a Rust `unsafe extern "C"` block (or any FFI) binds.  It replaces, for the
 * MoE block only, the CPU path of the reference engine:
 *
 *   reference (paths relative to the reference project root)      this library
 *   ------------------------------------------------------------  ---------------------------------
 *   RealMoeLayer / MoeLayerConfig        src/moe/layer.rs:185-212  AteniaMoeConfig + atenia_moe_create
 *   RealMoeLayer::assemble (weights)     src/moe/layer.rs:276-351  atenia_moe_set_weights
 *   RealMoeLayer::forward_with           src/moe/layer.rs:405-431  atenia_moe_forward
 *   MoeDenseLayer::route + top_k_routing src/moe/dense.rs:325-337,
 *                                        src/moe/sparse.rs:142-191 atenia_moe_route_from_logits
 *   register_real_moe_layer              src/moe/graph_op.rs:228   atenia_register_real_moe_layer
 *   register_resident_moe_layer          src/moe/graph_op.rs:237   atenia_register_resident_moe_layer
 *   execute_real_moe_layer               src/moe/graph_op.rs:327   atenia_execute_real_moe_layer
 *   quantize_per_row_i8                  src/tensor/disk_tier.rs:231-245  atenia_quantize_per_row_i8
 *   absmax_per_channel_symmetric,        src/tensor/quantizer.rs:67-118,
 *   absmax_per_group_symmetric           :176-246                  atenia_quantize_per_group_i8
 *   int8_to_bf16_per_{channel,group}_launch_device
 *                                        src/cuda/int8_to_bf16.cu:42-73, :119-150
 *                                                                  atenia_int8_to_bf16_per_group
 *   RealMoeStack::forward                src/moe/stack.rs:197-210  atenia_moe_stack_forward
 *   RealMoeLayer::forward_with           src/moe/layer.rs:405-431  atenia_moe_forward_with
 *   execute_real_moe_layer_with          src/moe/graph_op.rs:352-364  atenia_execute_real_moe_layer_with
 *   NumericPolicy, numeric_policy()      src/moe/numeric_policy.rs:37-127  atenia_numeric_policy*
 *   auto_expert_cache_capacity           src/moe/residency.rs:201-211  atenia_moe_plan_residency
 *
 * Conventions follow the reference's existing CUDA FFI (the .cu files under src/cuda): plain `extern "C"` functions,
 * `int` status (0 = ok, > 0 = a cudaError_t value, < 0 = argument / shape / state errors listed
 * below), raw pointers and integer sizes, and the caller owns every buffer it passes.  Nothing here
 * falls back to the CPU: an error is returned as a status.
 *
 * Pointer kinds are stated per argument: "device" pointers must be valid on the layer's CUDA device,
 * "host" pointers are ordinary process memory.
 */
#ifndef ATENIA_MOE_H_
#define ATENIA_MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ATENIA_API __attribute__((visibility("default")))
#else
#define ATENIA_API
#endif

/* ---- status codes ------------------------------------------------------------------------- */
#define ATENIA_OK 0
#define ATENIA_ERR_NULL (-1)            /* a required pointer is NULL */
#define ATENIA_ERR_SHAPE (-2)           /* sizes violate a stated constraint */
#define ATENIA_ERR_CAPACITY (-3)        /* more tokens than the layer's max_tokens */
#define ATENIA_ERR_STATE (-4)           /* e.g. forward before set_weights */
#define ATENIA_ERR_LAYER_NOT_FOUND (-5) /* unknown registry id (MoeBindingError::LayerNotFound) */
#define ATENIA_ERR_DIM_MISMATCH (-6)    /* input length not a multiple of d_model (MoeDenseError::DimMismatch) */
#define ATENIA_ERR_UNSUPPORTED (-7)     /* valid in the reference, not built here */
#define ATENIA_ERR_DEVICE_TIMEOUT (-8)  /* a bounded wait inside a kernel gave up */
#define ATENIA_ERR_ROUTING (-9)         /* non-finite routing weight or selected sum <= 0 (MoeSparseError) */
#define ATENIA_ERR_NCCL (-10)           /* an NCCL call failed */
#define ATENIA_ERR_DRIVER (-11)         /* tensor-map encode or driver entry point unavailable */
#define ATENIA_ERR_IO (-13)             /* a tier file is missing or could not be read */
#define ATENIA_ERR_TIER_FORMAT (-14)    /* a tier file's length matches none of its encodings (or not the one asked for) */
#define ATENIA_ERR_SCRATCH_LIMIT (-12)  /* request larger than the fixed scratch of atenia_moe_dispatch_noalloc */
#define ATENIA_ERR_POLICY (-15)         /* the numeric policy the host selected keeps the block on its CPU arms */

/* ---- enums -------------------------------------------------------------------------------- */
#define ATENIA_IO_BF16 0 /* activations as bf16 (high half of an f32, src/tensor/tensor.rs:294-308) */
#define ATENIA_IO_F32 1  /* activations as f32 (what execute_real_moe_layer passes) */

#define ATENIA_W_BF16 0     /* expert weights bf16 */
#define ATENIA_W_INT8_ROW 1 /* expert weights int8, one f32 scale per output row (disk_tier.rs:231-259) */

/* ---- layer description (mirrors MoeLayerConfig + MoeExecutionConvention) ------------------- */
typedef struct AteniaMoeConfig {
  int32_t num_experts;       /* routed experts E (global count under expert parallelism), 1..128 */
  int32_t experts_per_token; /* top-k, 1..min(E, 8) */
  int32_t d_model;           /* multiple of 16 */
  int32_t d_ff;              /* routed expert width F, multiple of 16 */
  int32_t shared_d_ff;       /* shared expert width Fs (0 = no shared expert), multiple of 16 */
  int32_t renormalize;       /* 1: selected weights divided by their sum (Atenia / Mixtral) */
  int32_t shared_gated;      /* 1: shared output scaled by sigmoid(g . x) (HuggingFaceQwen) */
  int32_t weight_dtype;      /* ATENIA_W_* for routed and shared expert matrices */
  int32_t max_tokens;        /* capacity of the layer's device workspace, tokens per forward call */
  int32_t ep_rank;           /* expert-parallel rank of this process (0 when ep_world == 1) */
  int32_t ep_world;          /* expert-parallel world size: 1, 2, 4 or 8; must divide num_experts */
  /* Router family.  ATENIA_ROUTER_SOFTMAX (0): softmax + top-k as above.  ATENIA_ROUTER_V3 (1): DeepSeek-V3
   * routing (src/moe/v3_router.rs:206-309): sigmoid scores, e_score_correction_bias for selection only,
   * groups ranked by the sum of their two best, top-k inside the topk_group best groups, weights =
   * original scores, normalised when `renormalize` (norm_topk_prob), times routed_scaling_factor.
   * Invalid combinations (V3RouterConfig::validate) are ATENIA_ERR_SHAPE at create. */
  int32_t router_mode;
  int32_t n_group;               /* V3 only */
  int32_t topk_group;            /* V3 only */
  float routed_scaling_factor;   /* V3 only */
} AteniaMoeConfig;
#define ATENIA_ROUTER_SOFTMAX 0
#define ATENIA_ROUTER_V3 1

/* Device pointers to the weights.  Expert matrices keep the reference's row-major layouts
 * (src/moe/dense.rs:203-216): gate, up [F, d]; down [d, F].  The per-expert pointer arrays are HOST
 * arrays of `num_experts / ep_world` DEVICE pointers (the experts this rank owns, ascending id).
 * The library borrows the matrices: they must stay alive and unchanged while the layer is used.
 * The router matrix, the bias and the shared gate vector are copied at the call.
 * Scale arrays (f32, one per output row: F for gate/up, d for down) are required for INT8 and
 * ignored for bf16. */
typedef struct AteniaMoeWeights {
  const float* w_router;         /* device [E, d] f32; the router is never quantised (residency.rs:621-622) */
  const float* router_bias;      /* device [E] f32 or NULL; extra logit term for synthetic load skew */
  const void* const* w_gate;     /* host array of device pointers */
  const void* const* w_up;
  const void* const* w_down;
  const float* const* s_gate;    /* host array of device pointers, INT8 only */
  const float* const* s_up;
  const float* const* s_down;
  const void* shared_w_gate;     /* device [Fs, d] */
  const void* shared_w_up;       /* device [Fs, d] */
  const void* shared_w_down;     /* device [d, Fs] */
  const float* shared_s_gate;    /* device [Fs], INT8 only */
  const float* shared_s_up;      /* device [Fs], INT8 only */
  const float* shared_s_down;    /* device [d], INT8 only */
  const float* shared_gate_vec;  /* device [d] f32 or NULL (shared_expert_gate, layer.rs:208-211) */
  const float* e_score_bias;     /* device [E] f32 or NULL (= zeros): V3 e_score_correction_bias */
} AteniaMoeWeights;

/* Optional per-call outputs (device pointers, any may be NULL). */
typedef struct AteniaMoeAux {
  int32_t* topk_idx;       /* [T, k] selected experts, ascending per token */
  float* topk_w;           /* [T, k] combine weights */
  float* logits;           /* [T, E] router logits (f32) */
  int32_t* perm;           /* [T*k] dispatch order: row r holds flat entry t*k+s */
  int32_t* expert_offsets; /* [E+1] first row of each expert in dispatch order */
} AteniaMoeAux;

typedef struct AteniaMoeLayer AteniaMoeLayer;

/* Create a layer on the current CUDA device and allocate its workspace (sized by max_tokens). */
ATENIA_API int atenia_moe_create(const AteniaMoeConfig* cfg, AteniaMoeLayer** out);
ATENIA_API int atenia_moe_destroy(AteniaMoeLayer* layer);

/* Bind weights (see AteniaMoeWeights).  Builds the TMA descriptors of the expert matrices. */
ATENIA_API int atenia_moe_set_weights(AteniaMoeLayer* layer, const AteniaMoeWeights* w);

/* out[T, d] = MoE(x[T, d]).  x and out are device pointers of the stated io dtype; the call is
 * asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the default stream).
 * Follows RealMoeLayer::forward_with row by row; the convention is the one in the config. */
ATENIA_API int atenia_moe_forward(AteniaMoeLayer* layer, const void* x, int x_dtype, int T, void* out,
                                  int out_dtype, const AteniaMoeAux* aux, void* stream);

/* Execution conventions (MoeExecutionConvention, src/moe/layer.rs:37-43) for the calls that take one:
 *   ATENIA_CONVENTION_LAYER    the convention in the layer's config (renormalize, shared_gated)
 *   ATENIA_CONVENTION_ATENIA   selected weights renormalised, shared expert added ungated
 *   ATENIA_CONVENTION_HF_QWEN  raw selected weights, shared expert scaled by sigmoid(g . x) when a
 *                              gate vector was bound with the weights, by 1 otherwise */
#define ATENIA_CONVENTION_LAYER (-1)
#define ATENIA_CONVENTION_ATENIA 0
#define ATENIA_CONVENTION_HF_QWEN 1

/* atenia_moe_forward under an explicit convention for this call only (RealMoeLayer::forward_with,
 * src/moe/layer.rs:405-431).  The gate vector is kept by atenia_moe_set_weights whenever one is given,
 * whatever config.shared_gated says, so both conventions can be asked of one layer.  Softmax routers
 * only (ATENIA_ERR_UNSUPPORTED for ATENIA_ROUTER_V3, whose normalisation flag is part of its config). */
ATENIA_API int atenia_moe_forward_with(AteniaMoeLayer* layer, const void* x, int x_dtype, int T, void* out,
                                       int out_dtype, const AteniaMoeAux* aux, void* stream, int convention);

/* The step either side of the block in a decoder layer (src/moe/full_forward.rs:239-252):
 *   h = rms_norm(x, eps) * gamma;  out = x + MoE(h)
 * x, out: device f32 [T, d]; gamma: device f32 [d] (NULL = unit gain).  rms_norm follows
 * src/nn/normalization.rs:8-37 in f32 (x * (1 / sqrt(mean(x^2) + eps)), then the gain); the residual
 * is added in the combine kernel's epilogue, after the shared expert, as one f32 add per element.
 * The normalised rows pass through an f32 buffer of the layer ([max_tokens, d]) that the FIRST call
 * allocates (make that call outside any stream capture).  With T == 0 under token-sharded expert
 * parallelism x and out may be NULL. */
ATENIA_API int atenia_moe_block_forward(AteniaMoeLayer* layer, const float* x, const float* gamma, float eps, int T,
                                        float* out, void* stream);

/* The block with the selection supplied by the caller instead of the router: topk_idx [T, k] (device,
 * int32, expert ids in [0, E), need not be sorted) and topk_w [T, k] (device, f32) are used as they
 * are; everything after routing is unchanged (out = sum_s w[t,s] * expert_{idx[t,s]}(x_t), slots in
 * the given order, + the shared expert).  This is the batched form of the reference's decomposed
 * graph primitives MoeDynamicDispatch / ConditionalExpert / MoeSparseCombine
 * (src/moe/graph_op.rs:84-188, src/amg/graph.rs:5406-5566), whose selection tensor is the flat
 * [idx0, w0, idx1, w1, ...] list; the router primitives MoeRouterSoftmax / MoeTopK are
 * atenia_moe_route_from_logits.  An id outside [0, E) records ATENIA_ERR_ROUTING (returned by the next
 * atenia_moe_check); such an entry gets no row and contributes nothing, and no read leaves the
 * caller's buffers. */
ATENIA_API int atenia_moe_forward_selected(AteniaMoeLayer* layer, const void* x, int x_dtype, int T,
                                           const int32_t* topk_idx, const float* topk_w, void* out,
                                           int out_dtype, void* stream);

/* Same, then waits for the stream and returns any error a kernel recorded (routing errors,
 * bounded-wait timeouts).  Mirrors the reference's synchronous launchers. */
ATENIA_API int atenia_moe_forward_sync(AteniaMoeLayer* layer, const void* x, int x_dtype, int T, void* out,
                                       int out_dtype, const AteniaMoeAux* aux, void* stream);

/* Wait for `stream` and return the error word kernels of this layer recorded since the last check
 * (ATENIA_OK if none); the word is cleared. */
ATENIA_API int atenia_moe_check(AteniaMoeLayer* layer, void* stream);

/* Routing only, from caller-provided f32 logits [T, E] (device): softmax (dense.rs:172-187), top-k
 * with lowest-index tie-break and optional renormalisation (sparse.rs:142-191), and the dispatch
 * permutation (stable counting sort of the (token, slot) list by expert).  Integer outputs are
 * bit-identical to the CPU algorithm on the same logits.  All outputs are device pointers; perm,
 * inv_perm and expert_offsets may be NULL. */
ATENIA_API int atenia_moe_route_from_logits(AteniaMoeLayer* layer, const float* logits, int T,
                                            int32_t* topk_idx, float* topk_w, int32_t* perm,
                                            int32_t* inv_perm, int32_t* expert_offsets, void* stream);

/* Dispatch order without any allocation.  (No counterpart in the reference: it exists for hosts
 * that cannot call cudaMalloc -- all device memory already belongs to the host runtime's own pool,
 * an allocation's device-wide synchronisation is not acceptable, or the caller is only allowed to
 * touch the buffers it is handed -- and that therefore cannot create an AteniaMoeLayer.)
 * Given topk_idx [T, k] (device, expert ids in [0, E), ascending per token) it writes the same
 * perm [T*k], inv_perm [T*k] and expert_offsets [E+1] (all device, all required) as
 * atenia_moe_route_from_logits.  Scratch is a fixed 256 KiB array inside the library, present on
 * every GPU that loads it; hence the limits T*k <= ATENIA_NOALLOC_MAX_ENTRIES and
 * E <= ATENIA_NOALLOC_MAX_EXPERTS, beyond which the call returns ATENIA_ERR_SCRATCH_LIMIT and does
 * nothing.  Entries whose expert id is out of range get no row: their inv_perm entry is -1 and
 * perm[expert_offsets[E] .. T*k) is left unwritten.  topk_idx, perm, inv_perm and expert_offsets
 * must live on the CURRENT device (the scratch used is the current device's).  Asynchronous on
 * `stream`; the library calls no cudaMalloc / cudaFree / allocating routine here.
 * The first call on each device looks up the array's device address and keeps it for the life of
 * the process; make that first call outside any stream capture, and do not call this entry point
 * on a device after resetting it (cudaDeviceReset): the kept address would be stale.  All calls on
 * one GPU share the array: two calls whose kernels can overlap on that GPU (different streams
 * without ordering, or different host threads) race on it; order them on one stream or with
 * events. */
#define ATENIA_NOALLOC_MAX_ENTRIES 65536
#define ATENIA_NOALLOC_MAX_EXPERTS 128
ATENIA_API int atenia_moe_dispatch_noalloc(const int32_t* topk_idx, int T, int k, int E, int32_t* perm,
                                           int32_t* inv_perm, int32_t* expert_offsets, void* stream);

/* Per-row symmetric int8 quantisation of a row-major [rows, cols] f32 device matrix:
 * scale = max|row| / 127 (1.0 for a zero row), q = clamp(round_half_away(w * (1/scale)), -127, 127).
 * Bit-identical to quantize_per_row_i8 (src/tensor/disk_tier.rs:231-245). */
ATENIA_API int atenia_quantize_per_row_i8(const float* w, int64_t rows, int64_t cols, int8_t* q,
                                          float* scales, void* stream);

/* Dense W8A16 layout (the reference's non-MoE linear weights): row-major [K, N] f32 device matrix,
 * one scale per (group of `group_size` consecutive rows, column): scales is [ceil(K / group_size), N].
 * group_size 0 (or > K) means one group of K rows, i.e. per output channel.
 * scale = max(amax / 127, 1e-12), q = clamp(round_half_away(w / scale), -127, 127), a NaN quotient
 * gives 0.  Bit-identical to absmax_per_channel_symmetric (src/tensor/quantizer.rs:67-118) and
 * absmax_per_group_symmetric (:176-246).  Asynchronous on `stream`; an empty matrix is a no-op. */
ATENIA_API int atenia_quantize_per_group_i8(const float* w, int64_t K, int64_t N, int64_t group_size, int8_t* q,
                                            float* scales, void* stream);

/* The reference's materialising dequant of that layout: out[k, n] = the high 16 bits of
 * (float)q[k, n] * scales[k / group_size, n] (bf16 by truncation).  Bit-identical to
 * int8_to_bf16_per_channel_kernel / int8_to_bf16_per_group_kernel (src/cuda/int8_to_bf16.cu:24-40,
 * :99-117); unlike those launchers it takes a stream and sizes as int64.  The MoE kernels of this
 * library never materialise widened weights; this entry point exists for callers that hand the
 * result to their own bf16 GEMM. */
ATENIA_API int atenia_int8_to_bf16_per_group(const int8_t* q, const float* scales, int64_t K, int64_t N,
                                             int64_t group_size, uint16_t* out_bf16, void* stream);

/* ---- persistent expert tier files (host only) -----------------------------------------------
 * The reference persists each projection of each expert as one file `L{l}.e{i}.{gate,up,down}.bin`
 * (`L{l}.shared.*`, `L{l}.router.bin`, `L{l}.shared_gate.bin`) and recognises the encoding by the
 * byte length (src/moe/residency.rs:511-551; qint8 layout src/tensor/disk_tier.rs:168-224).  These
 * readers return the bytes in the form the GPU path consumes, so a tier written by the reference
 * loads without re-encoding.  All pointers are HOST memory; no CUDA call is made. */
#define ATENIA_TIER_F32 0
#define ATENIA_TIER_BF16 1
#define ATENIA_TIER_QINT8 2
/* The encoding of a [rows, cols] tensor file (ATENIA_TIER_*), ATENIA_ERR_IO if it cannot be opened,
 * ATENIA_ERR_TIER_FORMAT if its length matches none. */
ATENIA_API int atenia_tier_detect_dtype(const char* path, int64_t rows, int64_t cols);
/* qint8: q [rows*cols] int8 and scales [rows] f32 exactly as stored. */
ATENIA_API int atenia_tier_read_qint8(const char* path, int64_t rows, int64_t cols, int8_t* q, float* scales);
/* bf16: the 16-bit words exactly as stored. */
ATENIA_API int atenia_tier_read_bf16(const char* path, int64_t rows, int64_t cols, uint16_t* out);
/* Any encoding materialised as f32 the way the reference does (bf16 bits << 16; (f32)q * scale). */
ATENIA_API int atenia_tier_read_f32(const char* path, int64_t rows, int64_t cols, float* out);

/* ---- operator registry (host-memory interface of the reference's graph op) ---------------- */

/* Host-side description used by the registry: all weights are HOST f32 arrays in the reference's
 * layouts, exactly the fields of RealMoeLayer.  They are rounded to bf16 (nearest even) or quantised
 * per row to int8 and uploaded once; the host arrays are not referenced after the call returns. */
typedef struct AteniaHostMoeLayer {
  AteniaMoeConfig config;       /* weight_dtype selects bf16 or int8 storage on the device */
  const float* w_router;        /* [E, d] */
  const float* const* w_gate;   /* E pointers, each [F, d] */
  const float* const* w_up;     /* E pointers, each [F, d] */
  const float* const* w_down;   /* E pointers, each [d, F] */
  const float* shared_w_gate;   /* [Fs, d] or NULL */
  const float* shared_w_up;     /* [Fs, d] or NULL */
  const float* shared_w_down;   /* [d, Fs] or NULL */
  const float* shared_gate_vec; /* [d] or NULL */
  const float* e_score_bias;    /* [E] or NULL: V3 e_score_correction_bias */
} AteniaHostMoeLayer;

/* register_real_moe_layer: returns the new layer id (>= 0; ids are append-only and stable for the
 * process) or a negative status. */
ATENIA_API int64_t atenia_register_real_moe_layer(const AteniaHostMoeLayer* layer);

/* register_resident_moe_layer (src/moe/graph_op.rs:237): enter an existing device layer, whose
 * weights are already resident in HBM, into the registry.  The registry borrows the layer: the
 * caller keeps ownership and must not destroy it while the id is in use.  Returns the id or a
 * negative status. */
ATENIA_API int64_t atenia_register_resident_moe_layer(AteniaMoeLayer* layer);

/* execute_real_moe_layer: `input` is a flat HOST [n * d_model] f32 batch, `output` receives
 * [n * d_model] f32.  Rows are independent.  Unknown id -> ATENIA_ERR_LAYER_NOT_FOUND; a length that
 * is not a positive multiple of d_model -> ATENIA_ERR_DIM_MISMATCH.  Copies host->device, runs the
 * block, copies back and waits; batches larger than the layer's capacity run in several passes. */
ATENIA_API int atenia_execute_real_moe_layer(int64_t layer_id, const float* input, size_t len,
                                             float* output);

/* execute_real_moe_layer_with (src/moe/graph_op.rs:352-364): the same call under an explicit
 * ATENIA_CONVENTION_* for this call only. */
ATENIA_API int atenia_execute_real_moe_layer_with(int64_t layer_id, const float* input, size_t len, float* output,
                                                  int convention);

/* The device layer behind a registry id (NULL if unknown), for callers that keep activations on the
 * device. */
ATENIA_API AteniaMoeLayer* atenia_get_real_moe_layer(int64_t layer_id);

/* ---- numeric policy (src/moe/numeric_policy.rs:37-127) -------------------------------------------
 * The reference picks the arithmetic of its expert matvec from ATENIA_NUMERIC_POLICY =
 * {certified | f64, strict | f32, fast} (read once; default and any unknown value: certified), with
 * an in-process override (set_numeric_policy / clear_numeric_policy_override).  Only `fast` sends the
 * expert contraction to the GPU (ffn_uses_cuda, hook at src/moe/dense.rs:159-168); certified (f64
 * accumulation) and strict (f32) stay on the reference's own CPU arms; the router accumulates in f64
 * under every policy, as it does here.  This library is the `fast` arm and nothing else: it has no
 * CPU code.  These functions restate the switch so that a host binds one source of truth:
 *   atenia_numeric_policy()            the active policy (override, else environment, else certified)
 *   atenia_numeric_policy_is_explicit  1 when an override is set or the variable names a policy
 *   atenia_numeric_policy_gate()       ATENIA_OK when the library may serve the call: the active policy
 *                                      is fast, or the host never selected one (calling the library
 *                                      is then the selection); ATENIA_ERR_POLICY when the host
 *                                      explicitly selected certified or strict
 * The operator entry points atenia_execute_real_moe_layer[_with] apply the gate before anything else
 * (the host then runs its own CPU arm, exactly as matvec_policy does); the device-level calls
 * (atenia_moe_forward and friends) are explicit requests for the GPU and are not gated. */
#define ATENIA_POLICY_CERTIFIED 0
#define ATENIA_POLICY_STRICT 1
#define ATENIA_POLICY_FAST 2
ATENIA_API int atenia_numeric_policy_from_str(const char* name); /* ATENIA_POLICY_* or ATENIA_ERR_SHAPE */
ATENIA_API const char* atenia_numeric_policy_str(int policy);
ATENIA_API int atenia_numeric_policy(void);
ATENIA_API int atenia_numeric_policy_is_explicit(void);
ATENIA_API int atenia_set_numeric_policy(int policy);
ATENIA_API void atenia_clear_numeric_policy_override(void);
ATENIA_API int atenia_numeric_policy_ffn_uses_f32(int policy);
ATENIA_API int atenia_numeric_policy_ffn_uses_cuda(int policy);
ATENIA_API int atenia_numeric_policy_gate(void);

/* ---- expert residency planner ---------------------------------------------------------------------
 * The reference keeps experts in a RAM / NVMe tier behind a per-layer LRU cache whose capacity is
 * clamp(budget / (n_layers * bytes_per_expert), 1, E) (auto_expert_cache_capacity,
 * src/moe/residency.rs:201-211; resolved per model at src/moe/runtime.rs:559-584).  Here the tier is
 * HBM and a layer is either fully resident on its rank or sharded over more ranks, so the planner
 * answers: for `n_layers` layers of this configuration (max_tokens included: the workspace counts)
 * and `hbm_budget_bytes` per GPU (e.g. what cudaMemGetInfo reports free), which is the smallest
 * ep_world in {1, 2, 4, 8} dividing E in which every rank holds its E / ep_world experts of every
 * layer?  Returns ATENIA_OK with the plan, or ATENIA_ERR_CAPACITY when even 8 ranks do not hold the
 * model (the plan then describes the largest world tried; resident_experts_per_layer < experts_per_rank
 * is the reference's capacity rule applied to the budget left after the fixed costs).  Host arithmetic
 * only; cfg.ep_rank / cfg.ep_world are ignored. */
typedef struct AteniaResidencyPlan {
  int32_t min_ep_world;               /* smallest world that fits (or the largest tried on failure) */
  int32_t experts_per_rank;           /* E / min_ep_world */
  int32_t resident_experts_per_layer; /* experts of each layer the budget holds per rank in that world */
  int32_t reserved;
  uint64_t bytes_per_expert;          /* 3*F*d bytes (bf16: x2) plus (2F+d) f32 scales for int8 */
  uint64_t fixed_bytes_per_rank;      /* shared experts + router + workspace, all layers */
  uint64_t bytes_per_rank;            /* fixed + experts_per_rank * bytes_per_expert * n_layers */
} AteniaResidencyPlan;
ATENIA_API int atenia_moe_plan_residency(const AteniaMoeConfig* cfg, int n_layers, uint64_t hbm_budget_bytes,
                                         AteniaResidencyPlan* plan);
/* auto_expert_cache_capacity itself (src/moe/residency.rs:201-211). */
ATENIA_API uint64_t atenia_auto_expert_cache_capacity(uint64_t budget_bytes, uint64_t n_layers,
                                                      uint64_t per_expert_bytes, uint64_t num_experts);
/* Device bytes atenia_moe_create allocates for this configuration (0 for an invalid one). */
ATENIA_API uint64_t atenia_moe_workspace_bytes(const AteniaMoeConfig* cfg);
/* Sub-batches of atenia_execute_real_moe_layer for a batch of n_tokens (no counterpart in the
 * reference, whose operator computes where the data already is: src/moe/graph_op.rs:327-350).  The
 * operator here copies host buffers over PCIe and cuts a large batch into pieces so that the copies
 * of neighbouring pieces overlap a piece's forward; the cut is chosen with a cost model (weights
 * streamed per piece, flops per token, PCIe bytes per token): short end pieces around a large middle
 * one when the layer is slower than the link, equal pieces when it is faster, one piece (no overlap)
 * for a small batch.  Writes the piece sizes (their sum is n_tokens, none above cfg->max_tokens) and
 * returns their number; ATENIA_ERR_CAPACITY if max_pieces is too small.  Host arithmetic only. */
ATENIA_API int atenia_moe_plan_exec_pieces(const AteniaMoeConfig* cfg, uint64_t n_tokens, uint64_t* pieces_out,
                                           int max_pieces);
/* The same plan from measured figures instead of the analytical model (no counterpart in the reference):
 * a forward of T tokens takes forward_base_ms + forward_token_ms * T and a token's copy over the link
 * copy_token_ms, each way.  This is what the operator does after its first pipelined call, with the
 * figures it timed itself; exported so that a host can plan with its own measurements and so that the
 * choice can be tested without a GPU.  All three zero: the analytical model. */
ATENIA_API int atenia_moe_plan_exec_pieces_measured(const AteniaMoeConfig* cfg, uint64_t n_tokens,
                                                    double forward_base_ms, double forward_token_ms,
                                                    double copy_token_ms, uint64_t* pieces_out, int max_pieces);

/* ---- layer stack ------------------------------------------------------------------------------
 * RealMoeStack::forward (src/moe/stack.rs:197-210): x <- layer_l(x) for l = 0..n-1, every layer with
 * its own convention, no norm.  `residual` = 1 computes x <- x + layer_l(x) instead (the reference
 * stack has no residual; the 32-layer decode benchmark does); `residual` = 2 computes the pre-norm
 * block of a transformer with attention left out, x <- x + layer_l(rmsnorm(x) * gamma_l) (unit gain and
 * eps 1e-5 unless atenia_moe_stack_set_norm says otherwise; without a norm, random SwiGLU layers blow
 * the residual stream up within a few layers).
 * Both require f32 input.  The stack
 * borrows the layers (single GPU, or expert-parallel with replicated tokens or the direct exchange;
 * equal d_model, else
 * ATENIA_ERR_DIM_MISMATCH as
 * MoeStackError::DModelMismatch); activations between layers are f32 buffers of the stack.  On a
 * non-default stream the sequence is captured once per (T, x, out) into a CUDA graph and replayed. */
typedef struct AteniaMoeStack AteniaMoeStack;
ATENIA_API int atenia_moe_stack_create(AteniaMoeLayer* const* layers, int n_layers, int residual,
                                       AteniaMoeStack** out);
ATENIA_API int atenia_moe_stack_forward(AteniaMoeStack* stack, const void* x, int x_dtype, int T, void* out,
                                        int out_dtype, void* stream);
/* Gains and epsilon of the pre-norm of a `residual` = 2 stack: `gammas` is a HOST array of n_layers
 * DEVICE pointers to f32 [d] vectors (an entry, or the whole array, may be NULL = unit gain); the
 * vectors are borrowed.  ATENIA_ERR_STATE for a stack without a pre-norm. */
ATENIA_API int atenia_moe_stack_set_norm(AteniaMoeStack* stack, const float* const* gammas, float eps);
/* Waits for the stream and returns the first error any layer's kernels recorded. */
ATENIA_API int atenia_moe_stack_check(AteniaMoeStack* stack, void* stream);
ATENIA_API int atenia_moe_stack_destroy(AteniaMoeStack* stack);

/* ---- expert parallelism ------------------------------------------------------------------- */

/* Size of the opaque NCCL unique id, and a fresh id (rank 0 creates it, the host program
 * broadcasts it to the other ranks by any means). */
ATENIA_API int atenia_moe_ep_unique_id_bytes(void);
ATENIA_API int atenia_moe_ep_get_unique_id(void* id_out);

/* Join the expert-parallel group of `layer` (config.ep_world ranks, one process per GPU).  After
 * this, atenia_moe_forward routes this rank's tokens, exchanges rows with the ranks that own the
 * selected experts, runs the local experts and exchanges the results back. */
ATENIA_API int atenia_moe_ep_init(AteniaMoeLayer* layer, const void* unique_id);

/* Let `layer` use the communicator `owner` joined with atenia_moe_ep_init (same ep_rank, ep_world and
 * device), so that the layers of a model share one NCCL communicator instead of one each.  The
 * communicator lives until the last layer holding it is destroyed.  After ATENIA_ERR_NCCL (a peer
 * failed, the communicator was aborted) every layer that shares it returns ATENIA_ERR_STATE. */
ATENIA_API int atenia_moe_ep_attach(AteniaMoeLayer* layer, AteniaMoeLayer* owner);

/* How tokens are laid out over the ranks of an expert-parallel layer (no counterpart in the
 * reference, which has no multi-GPU path):
 *   ATENIA_EP_TOKENS_SHARDED     (default) every rank brings its own tokens; rows travel to the ranks
 *                                that own the selected experts and back (two all-to-alls and one
 *                                host read of the row counts per forward)
 *   ATENIA_EP_TOKENS_REPLICATED  every rank passes the SAME [T, d] batch (decode); each rank runs its
 *                                own experts over it and the expert outputs are assembled with one
 *                                all-reduce in which every element has a single non-zero
 *                                contributor, so every rank returns the bytes of the single-GPU
 *                                result.  No host read: the forward can be captured in a CUDA graph
 *                                and such layers can be put in an atenia_moe_stack. */
#define ATENIA_EP_TOKENS_SHARDED 0
#define ATENIA_EP_TOKENS_REPLICATED 1
ATENIA_API int atenia_moe_ep_set_token_layout(AteniaMoeLayer* layer, int layout);

/* Direct exchange for token-sharded expert parallelism (no counterpart in the reference).  After
 * atenia_moe_ep_init every rank exports handles to its receive and result buffers, the host program
 * gathers the blobs of all ranks (rank order) and every rank imports them.  From then on
 * atenia_moe_forward stores each routed row straight into the receive buffer of the rank that owns
 * its expert and each expert output straight back into the source rank's buffer over NVLink; row
 * positions are derived on the device from all-gathered counts, two one-word all-reduces order the
 * stores, nothing is read on the host and the results are those of the NCCL send/receive path.
 * All ranks must be processes on one node whose GPUs have peer access, and their layers must have
 * been created with the same max_tokens (else ATENIA_ERR_SHAPE at import).  Destroy the layers of all
 * ranks only after every rank has finished its last forward. */
ATENIA_API int atenia_moe_ep_ipc_bytes(void);
ATENIA_API int atenia_moe_ep_ipc_export(AteniaMoeLayer* layer, void* blob_out);
ATENIA_API int atenia_moe_ep_ipc_import(AteniaMoeLayer* layer, const void* blobs_of_all_ranks);

/* Row placement of the direct exchange for one rank (pure host arithmetic, the same function the
 * device runs).  The receive buffer is laid out [local expert][source rank][rows].  dst_base[E] =
 * first row, in the owner's receive buffer, of the rows this rank holds for each expert;
 * gemm_offsets[E / world + 1] = first row of each local expert in this rank's receive buffer;
 * sub_offsets[E + 1] = first row of each (local expert, source rank) slice of it; src_base[E] = first
 * row of that slice in its source rank's dispatch order. */
ATENIA_API int atenia_moe_ep_plan_direct(const int32_t* counts_all, int world, int num_experts, int rank,
                                         int32_t* dst_base, int32_t* src_base, int32_t* sub_offsets,
                                         int32_t* gemm_offsets);

/* The exchange plan one rank derives from the all-gathered count matrix counts_all[world][E]
 * (rows rank p holds for expert e, in p's dispatch order).  Experts are owned contiguously:
 * expert e lives on rank e / (E / world).  Pure host arithmetic (no CUDA, no NCCL); exported so the
 * partition can be tested without GPUs.  Outputs (host arrays of `world` entries; rows, not bytes):
 *   send_off/send_cnt[p]  slice of this rank's dispatch-ordered rows bound for rank p
 *   recv_off/recv_cnt[p]  where rank p's rows land in this rank's receive buffer
 *   group_offsets[world * E/world + 1] (may be NULL) first receive-buffer row of each
 *                         (source rank, local expert) group, in buffer order; total_recv may be NULL */
ATENIA_API int atenia_moe_ep_plan(const int32_t* counts_all, int world, int num_experts, int rank,
                                  int64_t* send_off, int64_t* send_cnt, int64_t* recv_off, int64_t* recv_cnt,
                                  int64_t* group_offsets, int64_t* total_recv);

/* ---- diagnostics -------------------------------------------------------------------------- */
ATENIA_API const char* atenia_moe_status_str(int status);

#define ATENIA_COUNTER_FORWARD_CALLS 0   /* forwards issued */
#define ATENIA_COUNTER_KERNEL_LAUNCHES 1 /* kernels of this library launched */
#define ATENIA_COUNTER_TCGEN05_LAUNCHES 2 /* tensor-core grouped-GEMM launches among them */
#define ATENIA_COUNTER_H2D_BYTES 3       /* bytes copied host->device by the registry path */
#define ATENIA_COUNTER_D2H_BYTES 4       /* bytes copied device->host by the registry path */
ATENIA_API uint64_t atenia_moe_counter(int which);

/* Time of the most recent grouped-GEMM launches of this layer, measured with CUDA events on the
 * launching stream while timing is enabled (enable != 0).  `which`: 0 = routed gate/up + SwiGLU,
 * 1 = routed down, 2 = shared gate/up, 3 = shared down.  Returns milliseconds, or a negative value
 * if nothing was recorded.  Enabling timing adds event records to every forward. */
ATENIA_API int atenia_moe_enable_timing(AteniaMoeLayer* layer, int enable);
ATENIA_API float atenia_moe_last_gemm_ms(AteniaMoeLayer* layer, int which);
/* Phases of the most recent forward, from the same events: 0 = routing, permutation and row gather,
 * 1 = rows to the ranks of their experts (expert parallelism; 0 on one GPU), 2 = routed expert GEMMs,
 * 3 = results back to their source ranks (expert parallelism), 4 = shared expert and combine,
 * 5 = the whole forward.  Milliseconds, negative if nothing was recorded. */
ATENIA_API float atenia_moe_last_phase_ms(AteniaMoeLayer* layer, int which);
/* Rows the experts of this rank received in the most recent token-sharded expert-parallel forward; -1 if
 * none.  Under the direct exchange the count lives on the device and this call copies it back
 * (synchronous: call it outside timed regions, after the forward has completed). */
ATENIA_API int atenia_moe_last_recv_rows(AteniaMoeLayer* layer);

#ifdef __cplusplus
}
#endif
#endif /* ATENIA_MOE_H_ */
