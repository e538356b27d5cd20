"""Builds an OracleLayer from the seeded device tensors of a synthetic layer.  TEST INFRASTRUCTURE ONLY
(used by the tests, the smoke check and the benchmark's CPU legs; never by the product package)."""
import numpy as np
import torch

from . import oracle as orc


def to_np_weight(t):
    """Device bf16 / int8 / f32 tensor -> numpy array in the oracle's storage convention."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def oracle_layer(shape, w):
    """The CPU oracle over the very bytes the GPU layer was given (`w` from synth.make_weights)."""
    sc = None
    ssc = None
    if shape.int8:
        sc = {k: [s.cpu().numpy() for s in w["scales"][k]] for k in ("gate", "up", "down")}
        if w["shared"] is not None:
            ssc = [s.cpu().numpy() for s in w["shared_scales"]]
    return orc.OracleLayer(
        w["router"].cpu().numpy(), [to_np_weight(t) for t in w["gate"]], [to_np_weight(t) for t in w["up"]],
        [to_np_weight(t) for t in w["down"]], shape.top_k, shape.renormalize,
        shared=None if w["shared"] is None else [to_np_weight(t) for t in w["shared"]],
        shared_gate_vec=None if w["shared_gate"] is None else w["shared_gate"].cpu().numpy(),
        shared_gated=shape.shared_gated,
        router_bias=None if w["router_bias"] is None else w["router_bias"].cpu().numpy(),
        scales=sc, shared_scales=ssc)


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))
