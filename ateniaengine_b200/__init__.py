"""B200-native (sm_100a) implementation of the Atenia engine's mixture-of-experts block.

The product is the C-ABI library under `csrc/` (declared in `include/atenia_moe.h`); this package is
the thin host-side mirror of the reference's MoE operator interface on top of it.
"""
from .moe import (  # noqa: F401
    MoeExecutionConvention,
    MoeLayerConfig,
    RealMoeLayer,
    MoeLayerError,
    execute_real_moe_layer,
    register_real_moe_layer,
    register_resident_moe_layer,
    quantize_per_row_i8,
    quantize_per_group_i8,
    int8_to_bf16_per_group,
    execute_real_moe_layer_with,
    NumericPolicy,
    numeric_policy,
    set_numeric_policy,
    clear_numeric_policy_override,
    auto_expert_cache_capacity,
    plan_exec_pieces,
    plan_residency,
    workspace_bytes,
)
