"""Checkpoint binding: from HuggingFace tensor names to the arrays of one MoE layer.

Mirrors the reference's name classification and expert binding
(src/moe/detect.rs:120-192 `classify_tensor_name`, src/moe/data_plane.rs:100-145 `MoeWeightMap`,
src/moe/binding.rs:254-315 classic per-expert tensors, :381-447 packed `gate_up_proj [E, 2F, d]` whose
first half on dim 1 is gate, src/moe/layer.rs:214-268 shared expert and its sigmoid gate).  Host-side
only: the result feeds `RealMoeLayer` (device) or the CPU oracle (tests).
"""
import re
from dataclasses import dataclass, field

import numpy as np

ROLE_ROUTER = "MoeRouter"
ROLE_GATE, ROLE_UP, ROLE_DOWN = "MoeExpertGate", "MoeExpertUp", "MoeExpertDown"
ROLE_PACKED_GATE_UP, ROLE_PACKED_DOWN = "MoePackedGateUp", "MoePackedDown"
ROLE_SHARED = "MoeSharedExpert"
ROLE_OTHER = "Other"


class MoeBindingError(ValueError):
    """kind: LayerNotFound | NoExperts | MissingExpertTensor | MissingPackedTensor | MixedExpertFormat |
    SharedExpertIncomplete | ShapeMismatch | RouterMissing"""

    def __init__(self, kind, detail=""):
        super().__init__(f"moe-binding: {kind}: {detail}")
        self.kind = kind


def _id_after(name, marker):
    i = name.find(marker)
    if i < 0:
        return None
    m = re.match(r"\d+", name[i + len(marker):])
    return int(m.group(0)) if m else None


def is_moe_router_tensor(name):
    return ("block_sparse_moe.gate." in name or (".mlp.gate." in name and "gate_proj" not in name)
            or ".mlp.router." in name)


def classify_tensor_name(name):
    """(role, layer_id, expert_id), in the reference's order of tests."""
    layer_id = _id_after(name, ".layers.")
    expert_id = _id_after(name, ".experts.")
    if "shared_expert" in name:
        role = ROLE_SHARED
    elif "experts.gate_up_proj" in name:
        role = ROLE_PACKED_GATE_UP
    elif "experts." in name and expert_id is None and "down_proj" in name:
        role = ROLE_PACKED_DOWN
    elif ".experts." in name or "block_sparse_moe.experts." in name:
        if ".w1." in name or ".gate_proj." in name:
            role = ROLE_GATE
        elif ".w3." in name or ".up_proj." in name:
            role = ROLE_UP
        elif ".w2." in name or ".down_proj." in name:
            role = ROLE_DOWN
        else:
            role = ROLE_OTHER
    elif is_moe_router_tensor(name):
        role = ROLE_ROUTER
    else:
        role = ROLE_OTHER
    return role, layer_id, expert_id


@dataclass
class LayerEntries:
    router: str = None
    experts: dict = field(default_factory=dict)  # expert id -> {"gate": name, "up": name, "down": name}
    packed_gate_up: str = None
    packed_down: str = None
    shared: list = field(default_factory=list)   # names

    def has_classic_experts(self):
        return bool(self.experts)

    def has_packed_experts(self):
        return self.packed_gate_up is not None or self.packed_down is not None


class MoeWeightMap:
    """Tensor names of a checkpoint grouped by layer and role (MoeWeightMap::from_tensors)."""

    def __init__(self):
        self.layers = {}

    @classmethod
    def from_tensors(cls, names):
        m = cls()
        for name in names:
            role, layer_id, expert_id = classify_tensor_name(name)
            if role == ROLE_OTHER or layer_id is None:
                continue
            le = m.layers.setdefault(layer_id, LayerEntries())
            if role == ROLE_ROUTER:
                le.router = name
            elif role == ROLE_SHARED:
                le.shared.append(name)
            elif role == ROLE_PACKED_GATE_UP:
                le.packed_gate_up = name
            elif role == ROLE_PACKED_DOWN:
                le.packed_down = name
            elif expert_id is not None:
                slot = {ROLE_GATE: "gate", ROLE_UP: "up", ROLE_DOWN: "down"}[role]
                le.experts.setdefault(expert_id, {})[slot] = name
        return m

    def layer(self, layer_id):
        return self.layers.get(layer_id)


def bind_layer(tensors, layer_id, names=None):
    """tensors: mapping name -> 2-D / 3-D array.  Returns
    {"router" [E,d], "gate"/"up"/"down": per-expert lists, "shared": [g,u,d] or None, "shared_gate" [d] or None}."""
    wm = MoeWeightMap.from_tensors(names if names is not None else tensors.keys())
    le = wm.layer(layer_id)
    if le is None:
        raise MoeBindingError("LayerNotFound", f"layer {layer_id}")
    if le.router is None:
        raise MoeBindingError("RouterMissing", f"layer {layer_id}")
    router = np.asarray(tensors[le.router], dtype=np.float32)
    if le.has_classic_experts() and le.has_packed_experts():
        raise MoeBindingError("MixedExpertFormat", f"layer {layer_id}")
    gate, up, down = [], [], []
    if le.has_classic_experts():
        n = router.shape[0]
        for e in range(n):
            slots = le.experts.get(e)
            if slots is None or any(k not in slots for k in ("gate", "up", "down")):
                raise MoeBindingError("MissingExpertTensor", f"layer {layer_id} expert {e}")
            g, u, dn = (np.asarray(tensors[slots[k]], dtype=np.float32) for k in ("gate", "up", "down"))
            if g.shape != u.shape or dn.shape != g.shape[::-1] or g.shape[1] != router.shape[1]:
                raise MoeBindingError("ShapeMismatch", f"layer {layer_id} expert {e}: {g.shape} {u.shape} {dn.shape}")
            gate.append(g)
            up.append(u)
            down.append(dn)
    elif le.has_packed_experts():
        if le.packed_gate_up is None:
            raise MoeBindingError("MissingPackedTensor", "gate_up_proj")
        if le.packed_down is None:
            raise MoeBindingError("MissingPackedTensor", "down_proj")
        gu = np.asarray(tensors[le.packed_gate_up], dtype=np.float32)
        dn = np.asarray(tensors[le.packed_down], dtype=np.float32)
        if gu.ndim != 3 or dn.ndim != 3 or gu.shape[1] % 2:
            raise MoeBindingError("ShapeMismatch", f"packed {gu.shape} {dn.shape}")
        F = gu.shape[1] // 2
        if dn.shape != (gu.shape[0], gu.shape[2], F) or gu.shape[0] != router.shape[0]:
            raise MoeBindingError("ShapeMismatch", f"down_proj {dn.shape} inconsistent with gate_up_proj {gu.shape}")
        for e in range(gu.shape[0]):
            gate.append(np.ascontiguousarray(gu[e, :F]))  # first half of the fused dim is gate
            up.append(np.ascontiguousarray(gu[e, F:]))
            down.append(np.ascontiguousarray(dn[e]))
    else:
        raise MoeBindingError("NoExperts", f"layer {layer_id}")
    shared = shared_gate = None
    if le.shared:
        find = lambda needle: next((n for n in le.shared if needle in n), None)
        g, u, dn = find(".gate_proj."), find(".up_proj."), find(".down_proj.")
        if g is not None or u is not None or dn is not None:
            if g is None or u is None or dn is None:
                raise MoeBindingError("SharedExpertIncomplete", f"layer {layer_id}")
            shared = [np.asarray(tensors[n], dtype=np.float32) for n in (g, u, dn)]
        sg = find("shared_expert_gate")
        if sg is not None:
            shared_gate = np.asarray(tensors[sg], dtype=np.float32).reshape(-1)
    return {"router": router, "gate": gate, "up": up, "down": down, "shared": shared, "shared_gate": shared_gate}


def to_device_layer(bound, top_k, device, convention=None, renormalize=None, max_tokens=4096, int8=False):
    """Upload a layer bound by `bind_layer` and create the device layer: matrices rounded to bf16 (or
    quantised per row to int8 on the GPU, the reference's tier quantiser), router and gate vector kept
    f32.  The kernels need d_ff and the shared width to be multiples of 16: narrower experts are
    zero-padded, which changes nothing (a zero gate/up row gives h = 0 and the matching zero column of
    the down projection ignores it)."""
    import torch

    from .moe import MoeLayerConfig, RealMoeLayer, quantize_per_row_i8

    def pad16(a, axis):
        n = a.shape[axis]
        m = (n + 15) // 16 * 16
        if m == n:
            return a
        pad = [(0, 0)] * a.ndim
        pad[axis] = (0, m - n)
        return np.pad(a, pad)

    def up(a):
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)
        if int8:
            return quantize_per_row_i8(t)
        return t.to(torch.bfloat16), None

    E, d = bound["router"].shape
    mats = {k: [up(pad16(a, 0 if k != "down" else 1)) for a in bound[k]] for k in ("gate", "up", "down")}
    shared = shared_scales = None
    if bound["shared"] is not None:
        sh = [up(pad16(bound["shared"][0], 0)), up(pad16(bound["shared"][1], 0)), up(pad16(bound["shared"][2], 1))]
        shared = [m for m, _ in sh]
        shared_scales = [s for _, s in sh] if int8 else None
    f32 = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)
    cfg = MoeLayerConfig(E, int(top_k), shared is not None, d, mats["gate"][0][0].shape[0])
    scales = {k: [s for _, s in mats[k]] for k in mats} if int8 else None
    return RealMoeLayer(cfg, f32(bound["router"]), [m for m, _ in mats["gate"]], [m for m, _ in mats["up"]],
                        [m for m, _ in mats["down"]], shared=shared, shared_gate=f32(bound["shared_gate"]),
                        scales=scales, shared_scales=shared_scales, convention=convention, renormalize=renormalize,
                        max_tokens=max_tokens)

