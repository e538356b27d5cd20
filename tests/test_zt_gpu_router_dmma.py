"""ATENIA_MOE_ROUTER=dmma: router logits on the f64 tensor cores against the oracle and against the
default router."""
import os

import numpy as np
import pytest
import torch

from tests.test_gpu_parity import TOL_BF16, _run_parity, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,d_model,T", [("mixtral", 512, 1), ("mixtral", 528, 77), ("qwen_moe", 512, 300),
                                             ("deepseek_v2_lite", 512, 515), ("deepseek_v2_lite", 512, 1500),
                                             ("mixtral", 1024, 4096)])
def test_layer_parity_with_the_dmma_router(dev, monkeypatch, name, d_model, T):
    monkeypatch.setenv("ATENIA_MOE_ROUTER", "dmma")
    synth = _synth()
    base = synth.SHAPES[name]
    shape = synth.small(base, d_model=d_model, d_ff=384, shared_d_ff=256 if base.shared_d_ff else 0)
    _run_parity(dev, shape, T, TOL_BF16, seed=T, sample=256)


@pytest.mark.parametrize("E,k", [(8, 2), (16, 4), (32, 4), (60, 4), (64, 6), (128, 8)])
def test_same_routing_as_the_default_router(dev, monkeypatch, E, k):
    synth = _synth()
    shape = synth.MoeShape("r", 256, 64, E, k, True)
    w = synth.make_weights(shape, 3, dev)
    x = synth.make_activations(shape, 3, dev, tokens=999)
    monkeypatch.setenv("ATENIA_MOE_ROUTER", "scalar")
    _, a = synth.build_layer(shape, w, max_tokens=999).forward(x, out_dtype=torch.float32, aux=True, sync=True)
    monkeypatch.setenv("ATENIA_MOE_ROUTER", "dmma")
    _, b = synth.build_layer(shape, w, max_tokens=999).forward(x, out_dtype=torch.float32, aux=True, sync=True)
    # f64 sums in a different order: the f32 logits agree except for rare last-bit roundings
    la, lb = a["logits"].cpu().numpy(), b["logits"].cpu().numpy()
    assert np.abs(la - lb).max() <= 1e-6 and (la != lb).mean() < 1e-3
    same = (a["topk_idx"].cpu().numpy() == b["topk_idx"].cpu().numpy()).all(axis=1)
    assert same.mean() >= 0.999
