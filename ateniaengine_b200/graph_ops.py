"""The reference's decomposed MoE graph primitives as thin views over the fused operator.

The reference also exposes the block in pieces for its graph executor (src/amg/nodes.rs:124-181,
src/amg/graph.rs:5406-5566, src/moe/graph_op.rs:62-188): MoeRouterSoftmax + MoeTopK produce a flat f32
selection tensor `[idx0, w0, idx1, w1, ...]` (indices stored as f32, weights renormalised),
MoeDynamicDispatch / ConditionalExpert / MoeSparseCombine consume it.  Here a selection is a
[T, 2k] f32 tensor with the same interleaving, one row per token, and every function is a view over
`RealMoeLayer.route_from_logits` / `forward_selected`: no arithmetic happens in Python beyond the
encoding of the selection.
"""
import torch


def encode_selection(topk_idx, topk_w):
    """[T, k] int32 indices + [T, k] f32 weights -> [T, 2k] f32 `[idx0, w0, idx1, w1, ...]`."""
    T, k = topk_idx.shape
    sel = torch.empty((T, 2 * k), dtype=torch.float32, device=topk_idx.device)
    sel[:, 0::2] = topk_idx.to(torch.float32)
    sel[:, 1::2] = topk_w
    return sel


def decode_selection(selection):
    """Inverse of encode_selection.  Follows execute_dynamic_dispatch's validation
    (src/moe/graph_op.rs:104-121): an odd length, a negative or non-finite index is an error."""
    if selection.dim() != 2 or selection.shape[1] % 2 != 0:
        raise ValueError("dispatch selection must be [T, 2k]: [idx, w, ...] per token")
    idx_f = selection[:, 0::2]
    if not bool(torch.isfinite(idx_f).all()) or bool((idx_f < 0).any()):
        raise ValueError("dispatch selection holds a negative or non-finite expert index")
    return idx_f.to(torch.int32).contiguous(), selection[:, 1::2].contiguous()


def expert_weight_in_selection(selection_row, expert_id):
    """Weight of `expert_id` in one token's selection, or None (src/moe/graph_op.rs:142-150)."""
    pairs = selection_row.numel() // 2
    for p in range(pairs):
        if int(selection_row[2 * p]) == int(expert_id):
            return float(selection_row[2 * p + 1])
    return None


def moe_router_top_k(layer, logits):
    """MoeRouterSoftmax followed by MoeTopK{k} on router logits [T, E] (CUDA f32): the layer's softmax
    + top-k (lowest index wins ties, ascending indices).  The reference's MoeTopK always renormalises;
    this follows the layer's `renormalize` setting."""
    idx, w, _, _, _ = layer.route_from_logits(logits, want_perm=False)
    return encode_selection(idx, w)


def execute_dynamic_dispatch(layer, x, selection, out_dtype=torch.float32):
    """MoeDynamicDispatch (src/moe/graph_op.rs:92-139): run exactly the listed experts on each token and
    combine their outputs with the listed weights, in the listed order.  Returns (output [T, d],
    executed expert ids [T, k]).  The selection must list k = experts_per_token experts per token; a
    layer with a shared expert adds it as its forward does."""
    idx, w = decode_selection(selection)
    if idx.shape[1] != layer.config.experts_per_token:
        raise ValueError("selection must list experts_per_token experts per token")
    if bool((idx >= layer.config.num_experts).any()):
        raise ValueError("selection names an expert the layer does not have")
    return layer.forward_selected(x, idx, w, out_dtype=out_dtype), idx


def execute_sparse_reference(layer, x, out_dtype=torch.float32):
    """MoeSparseReference (src/moe/graph_op.rs:62-73): the fused sparse forward."""
    return layer.forward(x, out_dtype=out_dtype, sync=True)
