"""ATENIA_MOE_ROUTER=splitk: the split-k router for small batches against the oracle and the default
router, repeated calls (its counters reset themselves) and the hand-over to the default router above
1024 tokens."""
import os

import numpy as np
import pytest
import torch

from tests.test_gpu_parity import TOL_BF16, _run_parity, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,d_model,T", [("mixtral", 512, 1), ("mixtral", 528, 13), ("qwen_moe", 512, 64),
                                             ("deepseek_v2_lite", 1024, 200), ("mixtral", 512, 1500)])
def test_layer_parity_with_the_splitk_router(dev, monkeypatch, name, d_model, T):
    monkeypatch.setenv("ATENIA_MOE_ROUTER", "splitk")
    synth = _synth()
    base = synth.SHAPES[name]
    shape = synth.small(base, d_model=d_model, d_ff=384, shared_d_ff=256 if base.shared_d_ff else 0)
    _run_parity(dev, shape, T, TOL_BF16, seed=T, sample=256)


@pytest.mark.parametrize("E,k", [(8, 2), (60, 4), (64, 6), (128, 8)])
def test_same_routing_as_the_default_router_and_repeatable(dev, monkeypatch, E, k):
    synth = _synth()
    shape = synth.MoeShape("r", 4096, 64, E, k, True)
    w = synth.make_weights(shape, 3, dev)
    x = synth.make_activations(shape, 3, dev, tokens=37)
    monkeypatch.setenv("ATENIA_MOE_ROUTER", "scalar")
    _, a = synth.build_layer(shape, w, max_tokens=64).forward(x, out_dtype=torch.float32, aux=True, sync=True)
    monkeypatch.setenv("ATENIA_MOE_ROUTER", "splitk")
    layer = synth.build_layer(shape, w, max_tokens=64)
    outs = [layer.forward(x, out_dtype=torch.float32, aux=True, sync=True) for _ in range(3)]
    for _, b in outs:
        la, lb = a["logits"].cpu().numpy(), b["logits"].cpu().numpy()
        assert np.abs(la - lb).max() <= 1e-6 and (la != lb).mean() < 1e-2
        assert (a["topk_idx"].cpu().numpy() == b["topk_idx"].cpu().numpy()).all(axis=1).mean() >= 0.97
    assert torch.equal(outs[0][1]["logits"], outs[2][1]["logits"]) and torch.equal(outs[0][0], outs[2][0])
    # fewer tokens than the last call: only the counters of the first token blocks are touched
    y1, a1 = layer.forward(x[:3], out_dtype=torch.float32, aux=True, sync=True)
    assert torch.equal(a1["logits"], outs[0][1]["logits"][:3]) and torch.equal(a1["topk_idx"], outs[0][1]["topk_idx"][:3])
    # (three tokens take the decode GEMM kernel, thirty-seven the tile kernels: outputs agree to rounding)
    assert (y1 - outs[0][0][:3]).abs().max() <= 1e-2 * outs[0][0].abs().max()
