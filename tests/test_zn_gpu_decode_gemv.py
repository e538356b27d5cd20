"""The CUDA-core matrix-vector kernel for calls of at most two rows (decode at batch 1) against the
oracle and against the tensor-core kernels, bf16 and INT8, with and without a shared expert, including a K that is not a multiple of the 512 elements a warp covers per step."""
import os
from dataclasses import replace

import pytest
import torch

from tests.helpers import rel_l2
from tests.test_gpu_parity import TOL_BF16, TOL_W8A16, _run_parity, _synth, dev  # noqa: F401

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,int8,d_model,d_ff,shared,T", [
    ("mixtral", False, 1024, 2048, 0, 1), ("mixtral", False, 1024, 2048, 0, 2), ("mixtral", True, 1024, 2048, 0, 1),
    ("mixtral", True, 528, 400, 0, 2), ("mixtral", False, 528, 400, 0, 2), ("qwen_moe", False, 512, 384, 768, 1),
    ("qwen_moe", True, 512, 384, 768, 1), ("deepseek_v2_lite", False, 512, 384, 256, 1)])
def test_gemv_matches_oracle(dev, monkeypatch, name, int8, d_model, d_ff, shared, T):
    monkeypatch.setenv("ATENIA_MOE_GEMV", "1")
    synth = _synth()
    shape = replace(synth.small(synth.SHAPES[name], d_model=d_model, d_ff=d_ff, shared_d_ff=shared), int8=int8)
    # (routed calls of more than two rows take the tensor-core kernels; the shared expert still takes
    # this kernel while the batch is at most two tokens)
    _run_parity(dev, shape, T, TOL_W8A16 if int8 else TOL_BF16, seed=T + d_model)


@pytest.mark.parametrize("int8", [False, True])
def test_gemv_agrees_with_tensor_core_kernels(dev, monkeypatch, int8):
    synth = _synth()
    shape = replace(synth.small(synth.SHAPES["mixtral"], d_model=1024, d_ff=2048), int8=int8)
    w = synth.make_weights(shape, 23, dev)
    x = synth.make_activations(shape, 23, dev, tokens=8)
    monkeypatch.setenv("ATENIA_MOE_GEMV", "0")
    base = synth.build_layer(shape, w, max_tokens=8)
    monkeypatch.setenv("ATENIA_MOE_GEMV", "1")
    layer = synth.build_layer(shape, w, max_tokens=8)
    for T in (1, 2):
        a = base.forward(x[:T], out_dtype=torch.float32, sync=True)
        b = layer.forward(x[:T], out_dtype=torch.float32, sync=True)
        assert torch.equal(b, layer.forward(x[:T], out_dtype=torch.float32, sync=True))
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 3e-3
    # eight tokens are sixteen rows: both layers take the tensor-core kernels
    assert torch.equal(base.forward(x, out_dtype=torch.float32, sync=True), layer.forward(x, out_dtype=torch.float32, sync=True))
