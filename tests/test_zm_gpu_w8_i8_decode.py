"""The INT8 decode kernel that multiplies the codes as integers (tcgen05 kind::i8, the token rows as four
planes of base-128 digits; the default for INT8 calls of at most 128 rows) against the oracle and against the
tensor-memory decode kernel it replaced (ATENIA_MOE_W8_I8=0)."""
from dataclasses import replace

import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_W8A16, _run_parity, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,d_model,d_ff,shared,T", [
    ("mixtral", 1024, 2048, 0, 1), ("mixtral", 1024, 2048, 0, 8), ("mixtral", 1024, 2048, 0, 64),
    ("mixtral", 528, 400, 0, 7), ("mixtral", 528, 400, 0, 33), ("deepseek_v2_lite", 512, 384, 256, 21),
    ("qwen_moe", 512, 384, 768, 3), ("mixtral", 512, 768, 0, 200)])
def test_w8_i8_kernel_matches_oracle(dev, monkeypatch, name, d_model, d_ff, shared, T):
    """Stream-K (few tiles) and whole-tile walks, N and K that are not multiples of the tile (K tails are
    zero-filled by the copies on both operands), one and several 32-token tiles per expert, with and without
    a shared expert (which keeps its own kernels)."""
    monkeypatch.setenv("ATENIA_MOE_W8_I8", "1")
    monkeypatch.setenv("ATENIA_MOE_W8_I8_ROWS", "512")  # (the 200-token case: 400 rows, many tiles per expert)
    synth = _synth()
    shape = replace(synth.small(synth.SHAPES[name], d_model=d_model, d_ff=d_ff, shared_d_ff=shared), int8=True)
    if shape.top_k * T > 512:
        pytest.skip("more than 512 rows: not a call of this kernel")
    _run_parity(dev, shape, T, TOL_W8A16, seed=T)


def test_w8_i8_kernel_agrees_with_tensor_memory_kernel(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=1024, d_ff=2048)
    w = synth.make_weights(shape, 23, dev)
    x = synth.make_activations(shape, 23, dev, tokens=64)
    monkeypatch.setenv("ATENIA_MOE_GEMV", "0")  # (the baseline's one-token call: tensor-memory kernel too)
    monkeypatch.setenv("ATENIA_MOE_W8_I8", "0")
    base = synth.build_layer(shape, w, max_tokens=64)
    monkeypatch.setenv("ATENIA_MOE_W8_I8", "1")
    layer = synth.build_layer(shape, w, max_tokens=64)
    for T in (1, 5, 64):
        a = base.forward(x[:T], out_dtype=torch.float32, sync=True)
        b = layer.forward(x[:T], out_dtype=torch.float32, sync=True)
        assert torch.equal(b, layer.forward(x[:T], out_dtype=torch.float32, sync=True))  # fixed reduction order
        # both round the intermediate rows to bf16; the integer product itself is the more exact one
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 3e-3


def test_rows_with_very_different_magnitudes(dev, monkeypatch):
    """Digit planes are scaled per token row: rows a factor 2^20 apart in one call must both come out right."""
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=512, d_ff=512)
    w = synth.make_weights(shape, 5, dev)
    x = synth.make_activations(shape, 5, dev, tokens=6).float()
    x[1] *= 2.0 ** -10
    x[4] *= 2.0 ** 10
    x = x.to(torch.bfloat16)
    monkeypatch.setenv("ATENIA_MOE_W8_I8", "0")
    base = synth.build_layer(shape, w, max_tokens=6)
    monkeypatch.setenv("ATENIA_MOE_W8_I8", "1")
    layer = synth.build_layer(shape, w, max_tokens=6)
    a = base.forward(x, out_dtype=torch.float32, sync=True).cpu().numpy()
    b = layer.forward(x, out_dtype=torch.float32, sync=True).cpu().numpy()
    for t in range(6):
        assert rel_l2(a[t], b[t]) < 5e-3, t
