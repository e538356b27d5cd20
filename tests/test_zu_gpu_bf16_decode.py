"""ATENIA_MOE_BF16_DECODE=1: the stream-K bf16 decode kernel (calls of at most 128 rows) against the
oracle and against the default bf16 kernels."""
import os

import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_BF16, _run_parity, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,d_model,d_ff,shared,T", [
    ("mixtral", 1024, 2048, 0, 1), ("mixtral", 1024, 2048, 0, 2), ("mixtral", 1024, 2048, 0, 16),
    ("mixtral", 1024, 2048, 0, 64), ("mixtral", 528, 400, 0, 7), ("deepseek_v2_lite", 512, 384, 256, 21),
    ("qwen_moe", 512, 384, 768, 3)])
def test_decode_kernel_matches_oracle(dev, monkeypatch, name, d_model, d_ff, shared, T):
    """Stream-K (few tiles) and whole-tile (64 experts) walks, ragged N and K, with and without a shared expert."""
    monkeypatch.setenv("ATENIA_MOE_BF16_DECODE", "1")
    synth = _synth()
    shape = synth.small(synth.SHAPES[name], d_model=d_model, d_ff=d_ff, shared_d_ff=shared)
    _run_parity(dev, shape, T, TOL_BF16, seed=T)


def test_decode_kernel_agrees_with_default_kernels(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=1024, d_ff=2048)
    w = synth.make_weights(shape, 23, dev)
    x = synth.make_activations(shape, 23, dev, tokens=64)
    monkeypatch.setenv("ATENIA_MOE_BF16_DECODE", "0")  # the 128-row-tile kernels as the other side
    base = synth.build_layer(shape, w, max_tokens=200)
    monkeypatch.setenv("ATENIA_MOE_BF16_DECODE", "1")
    layer = synth.build_layer(shape, w, max_tokens=200)
    for T in (1, 5, 64):
        a = base.forward(x[:T], out_dtype=torch.float32, sync=True)
        b = layer.forward(x[:T], out_dtype=torch.float32, sync=True)
        b2 = layer.forward(x[:T], out_dtype=torch.float32, sync=True)
        assert torch.equal(b, b2)  # the reduction order of stream-K is fixed
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 2e-3
    # a larger batch of the same layer leaves the decode kernel
    xl = synth.make_activations(shape, 24, dev, tokens=200)
    assert rel_l2(base.forward(xl, out_dtype=torch.float32, sync=True).cpu().numpy(),
                  layer.forward(xl, out_dtype=torch.float32, sync=True).cpu().numpy()) == 0.0
