"""Decomposed graph primitives over the fused operator, on the GPU."""
import os

import numpy as np
import pytest
import torch

from tests.helpers import oracle_layer, rel_l2
from tests.test_gpu_parity import TOL_BF16, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


def test_router_topk_then_dispatch_equals_the_fused_forward(dev):
    from ateniaengine_b200 import graph_ops as go
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=512, d_ff=512)
    w = synth.make_weights(shape, 17, dev)
    x = synth.make_activations(shape, 17, dev, tokens=200)
    layer = synth.build_layer(shape, w, max_tokens=200)
    fused, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    sel = go.moe_router_top_k(layer, aux["logits"])
    assert sel.shape == (200, 2 * shape.top_k)
    assert torch.equal(sel[:, 0::2].to(torch.int32), aux["topk_idx"])
    out, executed = go.execute_dynamic_dispatch(layer, x, sel)
    assert torch.equal(executed, aux["topk_idx"])
    assert torch.equal(out, fused)
    ref = oracle_layer(shape, w).forward(x.float().cpu().numpy())
    assert rel_l2(out.cpu().numpy(), ref) <= TOL_BF16
    # a selection in a different order of the same experts gives the same rows up to f32 addition order
    flipped = torch.cat([sel[:, 2:4], sel[:, 0:2]], dim=1).contiguous()
    out2, _ = go.execute_dynamic_dispatch(layer, x, flipped)
    assert rel_l2(out2.cpu().numpy(), out.cpu().numpy()) < 1e-6
    with pytest.raises(ValueError):
        go.execute_dynamic_dispatch(layer, x, sel[:, :2].contiguous())
