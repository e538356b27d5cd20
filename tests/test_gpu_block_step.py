"""The decoder-layer step around the MoE block on the GPU: post-attention RMSNorm with its gain before
the block and the residual add after it (src/moe/full_forward.rs:239-252; rms_norm
src/nn/normalization.rs:8-37), against the CPU oracle.  Tolerance: rel-L2 <= 1e-2 on the block's
contribution (bf16 weights), as for the block alone."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import oracle_layer, rel_l2

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


@pytest.mark.parametrize("name,T,with_gamma", [("mixtral", 70, True), ("qwen_moe", 129, True), ("deepseek_v2_lite", 33, False)])
def test_block_step_matches_oracle(name, T, with_gamma):
    from ateniaengine_b200 import synth
    dev = _dev()
    base = synth.SHAPES[name]
    shape = synth.small(base, d_model=512, d_ff=384, shared_d_ff=256 if base.shared_d_ff else 0)
    w = synth.make_weights(shape, 61, dev)
    # a residual stream that is far from unit scale, so that the norm matters
    x = synth.make_activations(shape, 61, dev, tokens=T, dtype=torch.float32) * 7.5 + 0.3
    g = torch.Generator(device=dev).manual_seed(3)
    gamma = (1.0 + 0.2 * torch.randn(shape.d_model, generator=g, device=dev)) if with_gamma else None
    eps = 1e-6
    layer = synth.build_layer(shape, w, max_tokens=T)
    out = layer.block_forward(x, gamma, eps, sync=True)
    assert torch.equal(out, layer.block_forward(x, gamma, eps, sync=True))
    xs = x.cpu().numpy()
    h = orc.rms_norm_gamma(xs, None if gamma is None else gamma.cpu().numpy(), eps)
    moe = oracle_layer(shape, w).forward(h)
    # the block's contribution, with the residual taken out on both sides
    assert rel_l2(out.cpu().numpy() - xs, moe) <= 1e-2
    # and the residual itself is exact: out - MoE part reproduces x to f32 rounding of one add
    np.testing.assert_allclose(out.cpu().numpy(), xs + moe, rtol=0, atol=1e-2 * np.abs(moe).max() + 1e-6)
    # the same through the plain forward on the oracle's normalised rows (isolates the norm kernel)
    h_dev = torch.from_numpy(h).to(dev)
    plain = layer.forward(h_dev, out_dtype=torch.float32, sync=True)
    assert rel_l2((out - x).cpu().numpy(), plain.cpu().numpy()) <= 2e-3


def test_stack_with_gains_matches_layerwise_oracle():
    from ateniaengine_b200 import synth
    from ateniaengine_b200.moe import RealMoeStack
    dev = _dev()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=512, d_ff=768)
    ws = [synth.make_weights(shape, 200 + l, dev) for l in range(3)]
    layers = [synth.build_layer(shape, w, max_tokens=16) for w in ws]
    g = torch.Generator(device=dev).manual_seed(11)
    gammas = [1.0 + 0.3 * torch.randn(shape.d_model, generator=g, device=dev) for _ in range(3)]
    gammas[1] = None
    x = synth.make_activations(shape, 9, dev, tokens=9, dtype=torch.float32)
    stack = RealMoeStack(layers, residual=2)
    stack.set_norm(gammas, eps=1e-6)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        outs = [stack.forward(x, sync=True) for _ in range(3)]  # eager, captured, replayed
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    cur = x.cpu().numpy()
    for l in range(3):
        h = orc.rms_norm_gamma(cur, None if gammas[l] is None else gammas[l].cpu().numpy(), 1e-6)
        cur = cur + oracle_layer(shape, ws[l]).forward(h)
    assert rel_l2(outs[0].cpu().numpy(), cur) <= 1e-2
    # changing the gains takes effect (the captured graph is dropped)
    stack.set_norm(None, eps=1e-6)
    with torch.cuda.stream(side):
        other = stack.forward(x, sync=True)
    assert (other - outs[0]).abs().max() > 1e-3


def test_argument_errors():
    from ateniaengine_b200 import _lib, synth
    dev = _dev()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=256, d_ff=256)
    layer = synth.build_layer(shape, synth.make_weights(shape, 1, dev), max_tokens=4)
    lib = _lib.lib()
    x = torch.zeros((5, 256), device=dev)
    assert lib.atenia_moe_block_forward(layer.handle, x.data_ptr(), None, 1e-5, 5, x.data_ptr(), None) == -3
    assert lib.atenia_moe_block_forward(layer.handle, None, None, 1e-5, 2, x.data_ptr(), None) == -1
    assert lib.atenia_moe_block_forward(layer.handle, x.data_ptr(), None, -1.0, 2, x.data_ptr(), None) == -2
    assert lib.atenia_moe_block_forward(None, x.data_ptr(), None, 1e-5, 2, x.data_ptr(), None) == -1
