"""ATENIA_MOE_W8_MODE=5: the INT8 decode kernel that widens into shared memory (w8_decode_gemm.cu) against
the oracle and against the tensor-memory decode kernel it may replace."""
import os
from dataclasses import replace

import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_W8A16, _run_parity, _synth, dev  # noqa: F401

# Opt-in here until the kernel has run on hardware once: ATENIA_TEST_W8_DECODE=1.
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("ATENIA_TEST_W8_DECODE", "0") != "1",
                                 reason="opt-in kernel: set ATENIA_TEST_W8_DECODE=1")]


@pytest.mark.parametrize("name,d_model,d_ff,shared,T", [
    ("mixtral", 1024, 2048, 0, 1), ("mixtral", 1024, 2048, 0, 8), ("mixtral", 1024, 2048, 0, 64),
    ("mixtral", 528, 400, 0, 7), ("deepseek_v2_lite", 512, 384, 256, 21), ("qwen_moe", 512, 384, 768, 3),
    ("mixtral", 512, 768, 0, 300)])
def test_w8_decode_kernel_matches_oracle(dev, monkeypatch, name, d_model, d_ff, shared, T):
    """Stream-K (few tiles) and whole-tile walks, ragged N and K, with and without a shared expert, and groups
    above 128 rows (more than one token tile per expert)."""
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "5")
    monkeypatch.setenv("ATENIA_MOE_GEMV", "0")
    synth = _synth()
    shape = replace(synth.small(synth.SHAPES[name], d_model=d_model, d_ff=d_ff, shared_d_ff=shared), int8=True)
    _run_parity(dev, shape, T, TOL_W8A16, seed=T)


def test_w8_decode_kernel_agrees_with_tensor_memory_kernel(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=1024, d_ff=2048)
    w = synth.make_weights(shape, 23, dev)
    x = synth.make_activations(shape, 23, dev, tokens=64)
    monkeypatch.setenv("ATENIA_MOE_GEMV", "0")
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "1")
    base = synth.build_layer(shape, w, max_tokens=64)
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "5")
    layer = synth.build_layer(shape, w, max_tokens=64)
    for T in (1, 5, 64):
        a = base.forward(x[:T], out_dtype=torch.float32, sync=True)
        b = layer.forward(x[:T], out_dtype=torch.float32, sync=True)
        assert torch.equal(b, layer.forward(x[:T], out_dtype=torch.float32, sync=True))  # fixed reduction order
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 2e-3
