"""The INT8 kernel with 256-row token tiles (w8_gemm_m256.cu) against the oracle and
against the shared-memory widening kernel of grouped_gemm.cu."""
import os

import numpy as np
import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_W8A16, _run_parity, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d_model,d_ff,T", [(512, 768, 1100), (512, 768, 2600), (528, 400, 1500), (1024, 2048, 4096)])
def test_m256_kernel_matches_oracle(dev, monkeypatch, d_model, d_ff, T):
    """Groups of ~270 to ~1000 rows (ragged last tiles, second half-tile empty or partly filled), a
    feature count that is not a multiple of the tile and a K that is not a multiple of the k-block."""
    monkeypatch.delenv("ATENIA_MOE_W8_MODE", raising=False)  # the default for groups of 256 rows and more
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=d_model, d_ff=d_ff)
    _run_parity(dev, shape, T, TOL_W8A16, seed=T, sample=256)


def test_m256_kernel_agrees_with_shared_memory_widening_kernel(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=512, d_ff=768)
    w = synth.make_weights(shape, 21, dev)
    x = synth.make_activations(shape, 21, dev, tokens=3000)
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", "2")
    a = synth.build_layer(shape, w, max_tokens=3000).forward(x, out_dtype=torch.float32, sync=True)
    monkeypatch.delenv("ATENIA_MOE_W8_MODE")
    layer = synth.build_layer(shape, w, max_tokens=3000)
    b = layer.forward(x, out_dtype=torch.float32, sync=True)
    assert torch.equal(b, layer.forward(x, out_dtype=torch.float32, sync=True))
    # same integer codes, same bf16 activations, the same order of k: identical products
    assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 1e-6
