"""ATENIA_MOE_W8_MODE=3: the wide tensor-memory INT8 kernel (one widened weight tile per k-block for
up to 192 tokens) against the oracle and against the default INT8 kernels."""
import numpy as np
import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_W8A16, _run_parity, _synth, dev  # noqa: F401

import os

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d_model,d_ff,T", [(512, 768, 700), (512, 768, 2600), (528, 400, 1500), (1024, 2048, 4096)])
def test_wide_kernel_matches_oracle(dev, monkeypatch, d_model, d_ff, T):
    """Groups of ~175 to ~1000 rows (ragged last tiles, one to three token boxes), a feature count that
    is not a multiple of the 64-feature tile and a K that is not a multiple of the k-block."""
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "3")
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=d_model, d_ff=d_ff)
    _run_parity(dev, shape, T, TOL_W8A16, seed=T, sample=256)


def test_wide_kernel_agrees_with_default_kernels(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=512, d_ff=768)
    w = synth.make_weights(shape, 21, dev)
    x = synth.make_activations(shape, 21, dev, tokens=3000)
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "2")  # the shared-memory widening kernel as the other side
    a = synth.build_layer(shape, w, max_tokens=3000).forward(x, out_dtype=torch.float32, sync=True)
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "3")
    layer = synth.build_layer(shape, w, max_tokens=3000)
    b = layer.forward(x, out_dtype=torch.float32, sync=True)
    b2 = layer.forward(x, out_dtype=torch.float32, sync=True)
    assert torch.equal(b, b2)
    # same exact integer weights, same bf16 activations: only the f32 accumulation order differs
    assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 2e-3
    # small batches of the same layer still go to the decode kernel
    xs = x[:5]
    c = layer.forward(xs, out_dtype=torch.float32, sync=True)
    assert rel_l2(c.cpu().numpy(), a[:5].cpu().numpy()) < 2e-3
