"""Parity at the benchmark configurations' full sizes.

The oracle runs one token at a time in f64, so at these sizes it checks a seeded sample of the tokens
(the block is position-wise: a sampled token's expected output does not depend on the others), while
the integer results (routing given the kernel's own logits, permutation, offsets) are checked for the
whole batch.  Tolerances: rel-L2 <= 1e-2 (bf16), <= 2e-2 (W8A16).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import oracle_layer, rel_l2, routing_agreement

pytestmark = pytest.mark.gpu


def _check(name, T, tol, sample, seed=2):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ateniaengine_b200 import synth
    dev = torch.device("cuda:0")
    shape = synth.SHAPES[name]
    w = synth.make_weights(shape, seed, dev)
    x = synth.make_activations(shape, seed, dev, tokens=T)
    layer = synth.build_layer(shape, w, max_tokens=T)
    out, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    assert torch.isfinite(out).all()
    # whole batch: integer results follow from the kernel's logits exactly as on the CPU
    g_logits = aux["logits"].cpu().numpy()
    idx_ref, w_ref = orc.route_from_logits(g_logits, shape.top_k, shape.renormalize)
    np.testing.assert_array_equal(aux["topk_idx"].cpu().numpy(), idx_ref)
    np.testing.assert_allclose(aux["topk_w"].cpu().numpy(), w_ref, rtol=2e-7, atol=0)
    off_ref, perm_ref, _ = orc.dispatch_permutation(idx_ref, shape.num_experts)
    np.testing.assert_array_equal(aux["expert_offsets"].cpu().numpy(), off_ref)
    np.testing.assert_array_equal(aux["perm"].cpu().numpy(), perm_ref)
    # sampled tokens against the f64 oracle
    rows = np.sort(np.random.default_rng(seed).choice(T, size=min(sample, T), replace=False))
    ol = oracle_layer(shape, w)
    ref, raux = ol.forward(x.float().cpu().numpy()[rows], want_aux=True)
    np.testing.assert_allclose(g_logits[rows], raux["logits"], rtol=0, atol=4e-6)
    same = routing_agreement(idx_ref[rows], raux["topk_idx"], raux["logits"], shape.top_k, f"{name} T={T}", 0.97)
    err = rel_l2(out.cpu().numpy()[rows][same], ref[same])
    assert err <= tol, f"{name} T={T}: rel-L2 {err:.3e} > {tol}"
    # determinism of the whole batch
    assert torch.equal(layer.forward(x, out_dtype=torch.float32, sync=True), out)
    layer.close()


def test_mixtral_8x7b_layer_4096_tokens():
    _check("mixtral", 4096, 1e-2, sample=32)


@pytest.mark.parametrize("T", [1, 16, 256])
def test_mixtral_8x7b_layer_small_batches(T):
    _check("mixtral", T, 1e-2, sample=32)


def test_qwen15_moe_layer_2048_tokens():
    _check("qwen_moe", 2048, 1e-2, sample=64)


def test_deepseek_v2_lite_layer_8192_tokens():
    _check("deepseek_v2_lite", 8192, 1e-2, sample=64)


@pytest.mark.parametrize("T", [1, 8, 64])
def test_mixtral_w8a16_layer_decode_batches(T):
    _check("mixtral_int8", T, 2e-2, sample=64)


def test_mixtral_w8a16_layer_4096_tokens():
    _check("mixtral_int8", 4096, 2e-2, sample=24)
