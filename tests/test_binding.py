"""Checkpoint binding: tensor-name classification and expert assembly, against the naming of the
model families the reference supports and against its golden layer-0 fixtures."""
import os

import numpy as np
import pytest

from ateniaengine_b200 import binding as b
from oracle import oracle as orc


def test_classification_follows_reference_rules():
    c = b.classify_tensor_name
    assert c("model.layers.3.block_sparse_moe.experts.5.w1.weight") == (b.ROLE_GATE, 3, 5)
    assert c("model.layers.3.block_sparse_moe.experts.5.w3.weight") == (b.ROLE_UP, 3, 5)
    assert c("model.layers.3.block_sparse_moe.experts.5.w2.weight") == (b.ROLE_DOWN, 3, 5)
    assert c("model.layers.3.block_sparse_moe.gate.weight") == (b.ROLE_ROUTER, 3, None)
    assert c("model.layers.0.mlp.experts.11.gate_proj.weight") == (b.ROLE_GATE, 0, 11)
    assert c("model.layers.0.mlp.gate.weight") == (b.ROLE_ROUTER, 0, None)
    assert c("model.layers.0.mlp.router.weight") == (b.ROLE_ROUTER, 0, None)
    assert c("model.layers.0.mlp.gate_proj.weight")[0] == b.ROLE_OTHER  # a dense SwiGLU gate is not a router
    assert c("model.layers.0.mlp.shared_expert.up_proj.weight")[0] == b.ROLE_SHARED
    assert c("model.layers.0.mlp.shared_experts.down_proj.weight")[0] == b.ROLE_SHARED
    assert c("model.layers.0.mlp.shared_expert_gate.weight")[0] == b.ROLE_SHARED
    assert c("model.layers.0.mlp.experts.gate_up_proj") == (b.ROLE_PACKED_GATE_UP, 0, None)
    assert c("model.layers.0.mlp.experts.down_proj") == (b.ROLE_PACKED_DOWN, 0, None)
    assert c("model.layers.0.self_attn.q_proj.weight")[0] == b.ROLE_OTHER


def _golden(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: z[k] for k in z.files}


@pytest.mark.parametrize("name,family", [("mixtral_layer0", "mixtral"), ("qwen15_moe_layer0", "qwen"),
                                         ("deepseek_block", "deepseek")])
def test_binding_reproduces_golden_block(golden_dir, name, family):
    """Re-create a checkpoint dict in each family's naming (classic per-expert and packed), bind it,
    and run the bound arrays through the oracle: the fixture's expected output must come back."""
    g = _golden(golden_dir, name)
    E = g["gate"].shape[0]
    pre = "model.layers.0.block_sparse_moe" if family == "mixtral" else "model.layers.0.mlp"
    names = ("w1", "w3", "w2") if family == "mixtral" else ("gate_proj", "up_proj", "down_proj")
    classic = {f"{pre}.gate.weight": g["router"]}
    for e in range(E):
        for role, n in zip(("gate", "up", "down"), names):
            classic[f"{pre}.experts.{e}.{n}.weight"] = g[role][e]
    packed = {f"{pre}.gate.weight": g["router"],
              f"{pre}.experts.gate_up_proj": np.concatenate([g["gate"], g["up"]], axis=1),
              f"{pre}.experts.down_proj": g["down"]}
    extra = {}
    if "shared_gate_proj" in g:
        sh = "shared_experts" if family == "deepseek" else "shared_expert"
        for role in ("gate_proj", "up_proj", "down_proj"):
            extra[f"{pre}.{sh}.{role}.weight"] = g["shared_" + role]
        if "shared_gate_vec" in g:
            extra[f"{pre}.shared_expert_gate.weight"] = g["shared_gate_vec"][None, :]
    extra["model.layers.0.self_attn.q_proj.weight"] = np.zeros((4, 4), np.float32)
    extra["model.layers.1.mlp.gate.weight"] = g["router"] * 2  # another layer must not leak in
    key = "mlp_output" if family == "deepseek" else "atenia_ref"
    renorm = family != "deepseek"
    for ckpt in (classic, packed):
        bound = b.bind_layer({**ckpt, **extra}, 0)
        assert len(bound["gate"]) == E
        lay = orc.OracleLayer(bound["router"], bound["gate"], bound["up"], bound["down"], int(g["top_k"]), renorm,
                              shared=bound["shared"], shared_gated=False)
        out = lay.forward(g["input"].astype(np.float32))
        assert np.max(np.abs(out - g[key])) < 1e-8
        if "shared_gate_vec" in g:
            np.testing.assert_array_equal(bound["shared_gate"], g["shared_gate_vec"])


def test_binding_errors():
    r = np.zeros((2, 4), np.float32)
    w = np.zeros((6, 4), np.float32)
    d = np.zeros((4, 6), np.float32)
    pre = "model.layers.0.mlp"
    ok = {f"{pre}.gate.weight": r}
    for e in range(2):
        ok.update({f"{pre}.experts.{e}.gate_proj.weight": w, f"{pre}.experts.{e}.up_proj.weight": w,
                   f"{pre}.experts.{e}.down_proj.weight": d})
    assert len(b.bind_layer(ok, 0)["down"]) == 2
    with pytest.raises(b.MoeBindingError) as ei:
        b.bind_layer(ok, 7)
    assert ei.value.kind == "LayerNotFound"
    miss = dict(ok)
    del miss[f"{pre}.experts.1.up_proj.weight"]
    with pytest.raises(b.MoeBindingError) as ei:
        b.bind_layer(miss, 0)
    assert ei.value.kind == "MissingExpertTensor"
    mixed = dict(ok)
    mixed[f"{pre}.experts.gate_up_proj"] = np.zeros((2, 12, 4), np.float32)
    with pytest.raises(b.MoeBindingError) as ei:
        b.bind_layer(mixed, 0)
    assert ei.value.kind == "MixedExpertFormat"
    with pytest.raises(b.MoeBindingError) as ei:
        b.bind_layer({f"{pre}.gate.weight": r}, 0)
    assert ei.value.kind == "NoExperts"
    bad = dict(ok)
    bad[f"{pre}.experts.0.down_proj.weight"] = np.zeros((4, 5), np.float32)
    with pytest.raises(b.MoeBindingError) as ei:
        b.bind_layer(bad, 0)
    assert ei.value.kind == "ShapeMismatch"
    sh = dict(ok)
    sh[f"{pre}.shared_expert.gate_proj.weight"] = w
    with pytest.raises(b.MoeBindingError) as ei:
        b.bind_layer(sh, 0)
    assert ei.value.kind == "SharedExpertIncomplete"
