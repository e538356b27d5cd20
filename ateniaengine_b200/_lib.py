"""ctypes loader for libatenia_moe.so (the C ABI declared in include/atenia_moe.h).

There is no fallback: if the shared library is missing the import of any op raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libatenia_moe.so")

IO_BF16, IO_F32 = 0, 1
CONVENTION_LAYER, CONVENTION_ATENIA, CONVENTION_HF_QWEN = -1, 0, 1
POLICY_CERTIFIED, POLICY_STRICT, POLICY_FAST = 0, 1, 2
ERR_POLICY = -15
W_BF16, W_INT8_ROW = 0, 1

ERR_LAYER_NOT_FOUND = -5
ERR_DIM_MISMATCH = -6


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_experts", "experts_per_token", "d_model", "d_ff", "shared_d_ff", "renormalize",
        "shared_gated", "weight_dtype", "max_tokens", "ep_rank", "ep_world", "router_mode", "n_group",
        "topk_group")] + [("routed_scaling_factor", C.c_float)]


class MoeWeights(C.Structure):
    _fields_ = [
        ("w_router", C.c_void_p), ("router_bias", C.c_void_p),
        ("w_gate", C.POINTER(C.c_void_p)), ("w_up", C.POINTER(C.c_void_p)), ("w_down", C.POINTER(C.c_void_p)),
        ("s_gate", C.POINTER(C.c_void_p)), ("s_up", C.POINTER(C.c_void_p)), ("s_down", C.POINTER(C.c_void_p)),
        ("shared_w_gate", C.c_void_p), ("shared_w_up", C.c_void_p), ("shared_w_down", C.c_void_p),
        ("shared_s_gate", C.c_void_p), ("shared_s_up", C.c_void_p), ("shared_s_down", C.c_void_p),
        ("shared_gate_vec", C.c_void_p), ("e_score_bias", C.c_void_p),
    ]


class MoeAux(C.Structure):
    _fields_ = [("topk_idx", C.c_void_p), ("topk_w", C.c_void_p), ("logits", C.c_void_p),
                ("perm", C.c_void_p), ("expert_offsets", C.c_void_p)]


class ResidencyPlan(C.Structure):
    _fields_ = [("min_ep_world", C.c_int32), ("experts_per_rank", C.c_int32),
                ("resident_experts_per_layer", C.c_int32), ("reserved", C.c_int32),
                ("bytes_per_expert", C.c_uint64), ("fixed_bytes_per_rank", C.c_uint64),
                ("bytes_per_rank", C.c_uint64)]


class HostMoeLayer(C.Structure):
    _fields_ = [
        ("config", MoeConfig), ("w_router", C.c_void_p),
        ("w_gate", C.POINTER(C.c_void_p)), ("w_up", C.POINTER(C.c_void_p)), ("w_down", C.POINTER(C.c_void_p)),
        ("shared_w_gate", C.c_void_p), ("shared_w_up", C.c_void_p), ("shared_w_down", C.c_void_p),
        ("shared_gate_vec", C.c_void_p), ("e_score_bias", C.c_void_p),
    ]


EXPORTS = [
    "atenia_moe_create", "atenia_moe_destroy", "atenia_moe_set_weights", "atenia_moe_forward",
    "atenia_moe_forward_sync", "atenia_moe_check", "atenia_moe_route_from_logits",
    "atenia_quantize_per_row_i8", "atenia_register_real_moe_layer", "atenia_register_resident_moe_layer", "atenia_execute_real_moe_layer",
    "atenia_get_real_moe_layer", "atenia_moe_ep_unique_id_bytes", "atenia_moe_ep_get_unique_id",
    "atenia_moe_ep_init", "atenia_moe_status_str", "atenia_moe_counter", "atenia_moe_enable_timing",
    "atenia_moe_last_gemm_ms", "atenia_moe_dispatch_noalloc", "atenia_moe_ep_plan", "atenia_moe_stack_create",
    "atenia_moe_stack_forward", "atenia_moe_stack_check", "atenia_moe_stack_destroy",
    "atenia_moe_forward_selected", "atenia_tier_detect_dtype", "atenia_tier_read_qint8", "atenia_tier_read_bf16",
    "atenia_tier_read_f32", "atenia_quantize_per_group_i8", "atenia_int8_to_bf16_per_group",
    "atenia_moe_ep_attach", "atenia_moe_ep_set_token_layout",
    "atenia_moe_ep_ipc_bytes", "atenia_moe_ep_ipc_export", "atenia_moe_ep_ipc_import", "atenia_moe_ep_plan_direct",
    "atenia_moe_forward_with", "atenia_execute_real_moe_layer_with",
    "atenia_numeric_policy_from_str", "atenia_numeric_policy_str", "atenia_numeric_policy",
    "atenia_numeric_policy_is_explicit", "atenia_set_numeric_policy", "atenia_clear_numeric_policy_override",
    "atenia_numeric_policy_ffn_uses_f32", "atenia_numeric_policy_ffn_uses_cuda", "atenia_numeric_policy_gate",
    "atenia_moe_block_forward", "atenia_moe_stack_set_norm", "atenia_moe_last_phase_ms", "atenia_moe_last_recv_rows", "atenia_moe_plan_residency", "atenia_auto_expert_cache_capacity", "atenia_moe_workspace_bytes",
    "atenia_moe_plan_exec_pieces", "atenia_moe_plan_exec_pieces_measured",
]

_lib = None


class AteniaError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        msg = lib().atenia_moe_status_str(C.c_int(status)).decode()
        super().__init__(f"{where}: status {status}: {msg}")


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for the MoE block.")
        l = C.CDLL(LIB_PATH)
        l.atenia_moe_status_str.restype = C.c_char_p
        l.atenia_moe_counter.restype = C.c_uint64
        l.atenia_register_real_moe_layer.restype = C.c_int64
        l.atenia_get_real_moe_layer.restype = C.c_void_p
        l.atenia_register_resident_moe_layer.restype = C.c_int64
        l.atenia_register_resident_moe_layer.argtypes = [C.c_void_p]
        l.atenia_get_real_moe_layer.argtypes = [C.c_int64]
        l.atenia_moe_last_gemm_ms.restype = C.c_float
        l.atenia_moe_last_gemm_ms.argtypes = [C.c_void_p, C.c_int]
        l.atenia_moe_enable_timing.argtypes = [C.c_void_p, C.c_int]
        l.atenia_moe_create.argtypes = [C.POINTER(MoeConfig), C.POINTER(C.c_void_p)]
        l.atenia_moe_destroy.argtypes = [C.c_void_p]
        l.atenia_moe_set_weights.argtypes = [C.c_void_p, C.POINTER(MoeWeights)]
        fwd = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.POINTER(MoeAux), C.c_void_p]
        l.atenia_moe_forward.argtypes = fwd
        l.atenia_moe_forward_sync.argtypes = fwd
        l.atenia_moe_check.argtypes = [C.c_void_p, C.c_void_p]
        l.atenia_moe_forward_selected.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                                  C.c_void_p, C.c_int, C.c_void_p]
        l.atenia_moe_route_from_logits.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        l.atenia_quantize_per_row_i8.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                                 C.c_void_p]
        l.atenia_quantize_per_group_i8.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                                                   C.c_void_p]
        l.atenia_int8_to_bf16_per_group.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                                    C.c_void_p, C.c_void_p]
        l.atenia_register_real_moe_layer.argtypes = [C.POINTER(HostMoeLayer)]
        l.atenia_execute_real_moe_layer.argtypes = [C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]
        l.atenia_moe_ep_get_unique_id.argtypes = [C.c_void_p]
        l.atenia_moe_ep_plan.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6
        l.atenia_moe_counter.argtypes = [C.c_int]
        l.atenia_moe_status_str.argtypes = [C.c_int]
        l.atenia_moe_ep_attach.argtypes = [C.c_void_p, C.c_void_p]
        l.atenia_moe_ep_ipc_export.argtypes = [C.c_void_p, C.c_void_p]
        l.atenia_moe_ep_ipc_import.argtypes = [C.c_void_p, C.c_void_p]
        l.atenia_moe_ep_plan_direct.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_void_p]
        l.atenia_moe_ep_set_token_layout.argtypes = [C.c_void_p, C.c_int]
        for fn in (l.atenia_tier_detect_dtype,):
            fn.argtypes = [C.c_char_p, C.c_int64, C.c_int64]
        l.atenia_tier_read_qint8.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        l.atenia_tier_read_bf16.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.c_void_p]
        l.atenia_tier_read_f32.argtypes = [C.c_char_p, C.c_int64, C.c_int64, C.c_void_p]
        l.atenia_moe_stack_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.POINTER(C.c_void_p)]
        l.atenia_moe_stack_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                               C.c_void_p]
        l.atenia_moe_stack_check.argtypes = [C.c_void_p, C.c_void_p]
        l.atenia_moe_stack_destroy.argtypes = [C.c_void_p]
        l.atenia_moe_dispatch_noalloc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                                  C.c_void_p, C.c_void_p]
        l.atenia_moe_ep_init.argtypes = [C.c_void_p, C.c_void_p]
        l.atenia_moe_block_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p,
                                               C.c_void_p]
        l.atenia_moe_stack_set_norm.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_float]
        l.atenia_moe_last_phase_ms.restype = C.c_float
        l.atenia_moe_last_phase_ms.argtypes = [C.c_void_p, C.c_int]
        l.atenia_moe_last_recv_rows.argtypes = [C.c_void_p]
        l.atenia_moe_forward_with.argtypes = fwd + [C.c_int]
        l.atenia_execute_real_moe_layer_with.argtypes = [C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]
        l.atenia_numeric_policy_from_str.argtypes = [C.c_char_p]
        l.atenia_numeric_policy_str.argtypes = [C.c_int]
        l.atenia_numeric_policy_str.restype = C.c_char_p
        l.atenia_numeric_policy.argtypes = []
        l.atenia_numeric_policy_is_explicit.argtypes = []
        l.atenia_set_numeric_policy.argtypes = [C.c_int]
        l.atenia_clear_numeric_policy_override.argtypes = []
        l.atenia_clear_numeric_policy_override.restype = None
        l.atenia_numeric_policy_ffn_uses_f32.argtypes = [C.c_int]
        l.atenia_numeric_policy_ffn_uses_cuda.argtypes = [C.c_int]
        l.atenia_numeric_policy_gate.argtypes = []
        l.atenia_moe_plan_residency.argtypes = [C.POINTER(MoeConfig), C.c_int, C.c_uint64, C.POINTER(ResidencyPlan)]
        l.atenia_auto_expert_cache_capacity.argtypes = [C.c_uint64] * 4
        l.atenia_auto_expert_cache_capacity.restype = C.c_uint64
        l.atenia_moe_workspace_bytes.argtypes = [C.POINTER(MoeConfig)]
        l.atenia_moe_workspace_bytes.restype = C.c_uint64
        l.atenia_moe_plan_exec_pieces.argtypes = [C.POINTER(MoeConfig), C.c_uint64, C.POINTER(C.c_uint64), C.c_int]
        l.atenia_moe_plan_exec_pieces_measured.argtypes = [C.POINTER(MoeConfig), C.c_uint64, C.c_double, C.c_double,
                                                            C.c_double, C.POINTER(C.c_uint64), C.c_int]
        _lib = l
    return _lib


def check(status, where=""):
    if status != 0:
        raise AteniaError(status, where)
