"""ATENIA_MOE_W8_MODE=4: the INT8 decode kernel whose widening groups take alternate k-blocks must give
the bytes of the default INT8 decode kernel (same tiles, same MMA order, same stream-K pieces)."""
import os

import pytest
import torch

from tests.test_gpu_parity import TOL_W8A16, _run_parity, _synth, dev  # noqa: F401

# Opt-in in the library and here until it has run on hardware: ATENIA_TEST_W8_ALT=1.
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("ATENIA_TEST_W8_ALT", "0") != "1",
                                 reason="opt-in kernel: set ATENIA_TEST_W8_ALT=1")]


@pytest.mark.parametrize("T", [1, 8, 64, 200])
def test_alt_kernel_equals_default_kernel(dev, monkeypatch, T):
    from dataclasses import replace
    synth = _synth()
    for shape in (synth.small(synth.SHAPES["mixtral_int8"], d_model=1024, d_ff=2048),
                  replace(synth.small(synth.SHAPES["qwen_moe"], d_model=528, d_ff=400, shared_d_ff=768), int8=True)):
        w = synth.make_weights(shape, 29, dev)
        x = synth.make_activations(shape, 29, dev, tokens=T)
        monkeypatch.delenv("ATENIA_MOE_W8_MODE", raising=False)
        a = synth.build_layer(shape, w, max_tokens=T).forward(x, out_dtype=torch.float32, sync=True)
        monkeypatch.setenv("ATENIA_MOE_W8_MODE", "4")
        b = synth.build_layer(shape, w, max_tokens=T).forward(x, out_dtype=torch.float32, sync=True)
        assert torch.equal(a, b)


def test_alt_kernel_matches_oracle(dev, monkeypatch):
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "4")
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=1024, d_ff=2048)
    for T in (1, 64):
        _run_parity(dev, shape, T, TOL_W8A16, seed=T)
