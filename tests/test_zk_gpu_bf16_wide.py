"""ATENIA_MOE_BF16_WIDE=1: the transposed bf16 product with token tiles of up to 256 rows (the WIDE form of
bf16_decode_gemm.cu) against the oracle and against the 128-row-tile kernel it may replace."""
import os

import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_BF16, _run_parity, _synth, dev  # noqa: F401

# Opt-in here until the kernel has run on hardware once: ATENIA_TEST_BF16_WIDE=1.
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("ATENIA_TEST_BF16_WIDE", "0") != "1",
                                 reason="opt-in kernel: set ATENIA_TEST_BF16_WIDE=1")]


@pytest.mark.parametrize("name,d_model,d_ff,shared,T", [
    ("qwen_moe", 512, 384, 768, 600), ("qwen_moe", 512, 384, 768, 2048), ("deepseek_v2_lite", 512, 384, 256, 300),
    ("mixtral", 1024, 2048, 0, 64), ("mixtral", 1024, 2048, 0, 700), ("mixtral", 528, 400, 0, 1300),
    ("mixtral", 512, 768, 0, 20)])
def test_wide_kernel_matches_oracle(dev, monkeypatch, name, d_model, d_ff, shared, T):
    """Groups below 64 rows (one copy of token rows), between 64 and 256 (several copies, one tile), above 256
    (several tiles per expert), N and K that are not multiples of the tile, with and without a shared expert."""
    monkeypatch.setenv("ATENIA_MOE_BF16_WIDE", "1")
    monkeypatch.setenv("ATENIA_MOE_PAIR_MODE", "2")  # (never the CTA-pair kernel: every size takes this one)
    synth = _synth()
    shape = synth.small(synth.SHAPES[name], d_model=d_model, d_ff=d_ff, shared_d_ff=shared)
    _run_parity(dev, shape, T, TOL_BF16, seed=T)


def test_wide_kernel_agrees_with_tile_kernel(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["qwen_moe"], d_model=512, d_ff=384, shared_d_ff=0)
    w = synth.make_weights(shape, 23, dev)
    x = synth.make_activations(shape, 23, dev, tokens=1500)
    monkeypatch.setenv("ATENIA_MOE_PAIR_MODE", "2")
    monkeypatch.setenv("ATENIA_MOE_BF16_WIDE", "0")
    base = synth.build_layer(shape, w, max_tokens=1500)
    monkeypatch.setenv("ATENIA_MOE_BF16_WIDE", "1")
    layer = synth.build_layer(shape, w, max_tokens=1500)
    for T in (40, 500, 1500):
        a = base.forward(x[:T], out_dtype=torch.float32, sync=True)
        b = layer.forward(x[:T], out_dtype=torch.float32, sync=True)
        assert torch.equal(b, layer.forward(x[:T], out_dtype=torch.float32, sync=True))
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 3e-3
