"""GPU parity tests: the CUDA library (called through its C ABI) against the CPU oracle.

Bars: integer results (top-k indices, permutation, offsets, int8 codes) bit-exact; layer outputs
relative L2 <= 1e-2 for bf16 weights and <= 2e-2 for W8A16, against the f64-accumulating oracle fed
the same bf16-rounded (or int8 + scale) values.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import oracle_layer, reference_metrics, rel_l2, routing_agreement

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
TOL_W8A16 = 2e-2


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _synth():
    from ateniaengine_b200 import synth
    return synth


# ---- integer paths: bit-exact -----------------------------------------------------------------

def test_quantizer_is_bit_identical_to_cpu(dev):
    from ateniaengine_b200 import quantize_per_row_i8
    g = torch.Generator(device=dev).manual_seed(11)
    w = torch.randn((257, 1408), generator=g, device=dev) * 0.02
    w[5] = 0.0
    w[7, 3] = w[7].abs().max() * 2  # a clear row maximum
    q, s = quantize_per_row_i8(w)
    q_ref, s_ref = orc.quantize_per_row_i8(w.cpu().numpy())
    np.testing.assert_array_equal(s.cpu().numpy(), s_ref)
    np.testing.assert_array_equal(q.cpu().numpy(), q_ref)
    assert s_ref[5] == 1.0


@pytest.mark.parametrize("E,k,renorm", [(8, 2, True), (60, 4, False), (64, 6, False), (4, 2, True), (128, 8, True)])
def test_route_from_logits_bit_exact(dev, E, k, renorm):
    synth = _synth()
    shape = synth.MoeShape("r", 64, 64, E, k, renorm)
    w = synth.make_weights(shape, 1, dev)
    T = 1537
    layer = synth.build_layer(shape, w, max_tokens=T)
    g = torch.Generator(device=dev).manual_seed(E * 100 + k)
    logits = torch.randn((T, E), generator=g, device=dev) * 2.0
    # ties: identical logits in whole rows, pairs, and near-ties one ulp apart
    logits[0] = 1.25
    logits[1, : E // 2] = 0.5
    logits[2] = logits[2].round()
    logits[3, 1] = logits[3, 0]
    logits[4, E - 1] = torch.nextafter(logits[4, 0], torch.tensor(10.0, device=dev))
    # saturated softmax: huge spread rounds most weights to 0 -> ties at zero resolved by index
    logits[5] = torch.linspace(-200.0, 200.0, E, device=dev)
    idx, tw, perm, inv, off = layer.route_from_logits(logits)
    idx_ref, tw_ref = orc.route_from_logits(logits.cpu().numpy(), k, renorm)
    np.testing.assert_array_equal(idx.cpu().numpy(), idx_ref)
    # weights: same algorithm; exp() may differ in the last bit between libm and CUDA
    np.testing.assert_allclose(tw.cpu().numpy(), tw_ref, rtol=2e-7, atol=0)
    off_ref, perm_ref, inv_ref = orc.dispatch_permutation(idx_ref, E)
    np.testing.assert_array_equal(off.cpu().numpy(), off_ref)
    np.testing.assert_array_equal(perm.cpu().numpy(), perm_ref)
    np.testing.assert_array_equal(inv.cpu().numpy(), inv_ref)


def test_route_from_logits_rejects_non_finite(dev):
    from ateniaengine_b200._lib import AteniaError
    synth = _synth()
    shape = synth.MoeShape("r", 64, 64, 8, 2, True)
    layer = synth.build_layer(shape, synth.make_weights(shape, 1, dev), max_tokens=16)
    logits = torch.zeros((4, 8), device=dev)
    logits[2, 3] = float("nan")
    with pytest.raises(AteniaError) as ei:
        layer.route_from_logits(logits)
    assert ei.value.status == -9


# ---- layer parity ------------------------------------------------------------------------------

def _run_parity(dev, shape, T, tol, seed=3, x_dtype=torch.bfloat16, sample=None):
    synth = _synth()
    w = synth.make_weights(shape, seed, dev)
    x = synth.make_activations(shape, seed, dev, tokens=T, dtype=x_dtype)
    layer = synth.build_layer(shape, w, max_tokens=max(T, 1))
    out, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    out = out.cpu().numpy()
    ol = oracle_layer(shape, w)
    rows = np.arange(T) if sample is None or sample >= T else np.sort(
        np.random.default_rng(seed).choice(T, size=sample, replace=False))
    xs = x.float().cpu().numpy()[rows]
    ref, raux = ol.forward(xs, want_aux=True)
    # routing: identical selection given the GPU's own logits, and (nearly always) the oracle's
    g_logits = aux["logits"].cpu().numpy()
    idx_from_gpu_logits, _ = orc.route_from_logits(g_logits, shape.top_k, shape.renormalize)
    np.testing.assert_array_equal(aux["topk_idx"].cpu().numpy(), idx_from_gpu_logits)
    off_ref, perm_ref, _ = orc.dispatch_permutation(idx_from_gpu_logits, shape.num_experts)
    np.testing.assert_array_equal(aux["perm"].cpu().numpy(), perm_ref)
    np.testing.assert_array_equal(aux["expert_offsets"].cpu().numpy(), off_ref)
    np.testing.assert_allclose(g_logits[rows], raux["logits"], rtol=0, atol=2e-6)
    same = routing_agreement(aux["topk_idx"].cpu().numpy()[rows], raux["topk_idx"], raux["logits"], shape.top_k,
                             f"{shape.name} T={T}", 0.995)
    err = rel_l2(out[rows][same], ref[same])
    assert err <= tol, f"{shape.name}: rel-L2 {err:.3e} > {tol}"
    return err, reference_metrics(out[rows][same], ref[same])


def test_tiny_config_matches_oracle(dev):
    """The reference's CPU-runnable case: d512, F1408, 8 experts top-2, 64 tokens."""
    synth = _synth()
    _run_parity(dev, synth.SHAPES["tiny"], 64, TOL_BF16, seed=0)


def test_tiny_config_f32_io(dev):
    synth = _synth()
    _run_parity(dev, synth.SHAPES["tiny"], 64, TOL_BF16, seed=0, x_dtype=torch.float32)


@pytest.mark.parametrize("T", [1, 2, 16, 127, 129, 300])
def test_mixtral_structure_ragged_token_counts(dev, T):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=1024, d_ff=2048)
    _run_parity(dev, shape, T, TOL_BF16, seed=T)


def test_qwen_structure_shared_gated(dev):
    synth = _synth()
    shape = synth.small(synth.SHAPES["qwen_moe"], d_model=512, d_ff=384, shared_d_ff=768)
    _run_parity(dev, shape, 333, TOL_BF16)


def test_deepseek_structure_shared_ungated(dev):
    synth = _synth()
    shape = synth.small(synth.SHAPES["deepseek_v2_lite"], d_model=512, d_ff=384, shared_d_ff=768)
    _run_parity(dev, shape, 515, TOL_BF16)


def test_w8a16_structure(dev):
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=1024, d_ff=2048)
    for T in (1, 8, 64):
        _run_parity(dev, shape, T, TOL_W8A16, seed=T)


@pytest.mark.parametrize("mode", ["0", "1", "2"])
def test_w8a16_every_kernel(dev, monkeypatch, mode):
    """ATENIA_MOE_W8_MODE pins the INT8 kernel family (0: by size -- the integer-MMA decode kernel up to
    128 rows, weights widened into tensor memory for small groups, 256-row tiles widened into shared memory
    for large ones; 1: always the tensor-memory kernel; 2: 128-row tiles widened into shared memory); each
    must meet the bar at small and large group sizes."""
    monkeypatch.setenv("ATENIA_MOE_W8_MODE", mode)
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral_int8"], d_model=512, d_ff=768)
    for T in (3, 700):
        _run_parity(dev, shape, T, TOL_W8A16, seed=T)


@pytest.mark.parametrize("T", [200, 700])
def test_w8a16_with_shared_expert(dev, T):
    """Below 256 tokens the shared expert takes the small-group INT8 kernel, above it the 256-row-tile one."""
    synth = _synth()
    from dataclasses import replace
    shape = replace(synth.small(synth.SHAPES["qwen_moe"], d_model=512, d_ff=384, shared_d_ff=768), int8=True)
    _run_parity(dev, shape, T, TOL_W8A16)


def test_all_tokens_on_one_expert_and_empty_experts(dev):
    """A bias that dominates the logits sends every token to experts 2 and 5; the rest get no rows."""
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=512, d_ff=512)
    w = synth.make_weights(shape, 5, dev)
    bias = torch.full((8,), -50.0, device=dev)
    bias[2] = 50.0
    bias[5] = 49.0
    w["router_bias"] = bias
    x = synth.make_activations(shape, 5, dev, tokens=200)
    layer = synth.build_layer(shape, w, max_tokens=200)
    out, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    assert (aux["topk_idx"].cpu().numpy() == np.array([2, 5])).all()
    off = aux["expert_offsets"].cpu().numpy()
    assert off.tolist() == [0, 0, 0, 200, 200, 200, 400, 400, 400]
    ref = oracle_layer(shape, w).forward(x.float().cpu().numpy())
    assert rel_l2(out.cpu().numpy(), ref) <= TOL_BF16


def test_tensor_core_kernel_agrees_with_cuda_core_check(dev, monkeypatch):
    synth = _synth()
    shape = synth.small(synth.SHAPES["deepseek_v2_lite"], d_model=256, d_ff=384, shared_d_ff=256)
    w = synth.make_weights(shape, 9, dev)
    x = synth.make_activations(shape, 9, dev, tokens=300)
    a = synth.build_layer(shape, w, max_tokens=300).forward(x, out_dtype=torch.float32, sync=True)
    monkeypatch.setenv("ATENIA_MOE_CHECK_GEMM", "1")
    b = synth.build_layer(shape, w, max_tokens=300).forward(x, out_dtype=torch.float32, sync=True)
    assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) < 2e-3


@pytest.mark.parametrize("T", [5, 300, 1100])
def test_cta_pair_kernel_matches_single_cta_kernel(dev, monkeypatch, T):
    """ATENIA_MOE_PAIR_MODE pins the bf16 kernel (1: CTA pairs with 256-row tiles, 2: single CTA).
    Both see the same rows and accumulate over k in the same order."""
    synth = _synth()
    shape = synth.small(synth.SHAPES["deepseek_v2_lite"], d_model=512, d_ff=384, shared_d_ff=256)
    w = synth.make_weights(shape, 21, dev)
    x = synth.make_activations(shape, 21, dev, tokens=T)
    monkeypatch.setenv("ATENIA_MOE_PAIR_MODE", "2")
    a = synth.build_layer(shape, w, max_tokens=T).forward(x, out_dtype=torch.float32, sync=True)
    monkeypatch.setenv("ATENIA_MOE_PAIR_MODE", "1")
    b = synth.build_layer(shape, w, max_tokens=T).forward(x, out_dtype=torch.float32, sync=True)
    assert rel_l2(b.cpu().numpy(), a.cpu().numpy()) < 1e-3
    ref = oracle_layer(shape, w).forward(x.float().cpu().numpy())
    assert rel_l2(b.cpu().numpy(), ref) <= TOL_BF16


def test_forward_with_caller_selection(dev):
    """The decomposed form: route, then run the experts on a selection given from outside."""
    synth = _synth()
    shape = synth.small(synth.SHAPES["qwen_moe"], d_model=256, d_ff=128, shared_d_ff=0)
    w = synth.make_weights(shape, 31, dev)
    x = synth.make_activations(shape, 31, dev, tokens=90)
    layer = synth.build_layer(shape, w, max_tokens=90)
    out, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    # the router's own selection reproduces the fused result bit for bit
    again = layer.forward_selected(x, aux["topk_idx"], aux["topk_w"], out_dtype=torch.float32)
    assert torch.equal(again, out)
    # single-expert selections are the expert outputs; a weighted pair is their f32 combination
    k = shape.top_k
    e1 = torch.full((90, k), 3, dtype=torch.int32, device=dev)
    e2 = torch.full((90, k), 41, dtype=torch.int32, device=dev)
    one = torch.zeros((90, k), device=dev)
    one[:, 0] = 1.0
    y1 = layer.forward_selected(x, e1, one, out_dtype=torch.float32)
    y2 = layer.forward_selected(x, e2, one, out_dtype=torch.float32)
    mix_idx = e1.clone()
    mix_idx[:, 1] = 41
    mix_w = torch.zeros((90, k), device=dev)
    mix_w[:, 0] = 0.25
    mix_w[:, 1] = 0.5
    y = layer.forward_selected(x, mix_idx, mix_w, out_dtype=torch.float32)
    torch.testing.assert_close(y, 0.25 * y1 + 0.5 * y2, rtol=1e-6, atol=1e-9)
    # expert 3 alone with weight 1 is the expert's own output: against the oracle's expert on the same
    # bf16-rounded weights (MoeDenseExpert::forward, src/moe/dense.rs:253-270)
    up16 = lambda t: t.float().cpu().numpy()
    xs = x.float().cpu().numpy()
    for e, ye in ((3, y1), (41, y2)):
        ref = np.stack([orc.expert_forward(up16(w["gate"][e]), up16(w["up"][e]), up16(w["down"][e]), xs[t])
                        for t in range(90)])
        assert rel_l2(ye.cpu().numpy(), ref) <= TOL_BF16
    # and the weighted pair against combine_selected over the concatenated expert outputs
    # (src/moe/sparse.rs:87-116)
    e3 = np.stack([orc.expert_forward(up16(w["gate"][3]), up16(w["up"][3]), up16(w["down"][3]), xs[t]) for t in range(8)])
    e41 = np.stack([orc.expert_forward(up16(w["gate"][41]), up16(w["up"][41]), up16(w["down"][41]), xs[t]) for t in range(8)])
    for t in range(8):
        rc, ref = orc.combine_selected(np.array([0, 1], dtype=np.int32), np.array([0.25, 0.5], dtype=np.float32),
                                       np.concatenate([e3[t], e41[t]]), shape.d_model)
        assert rc == 0
        assert rel_l2(y[t].cpu().numpy(), ref) <= TOL_BF16


def test_invalid_expert_id_after_a_larger_batch_stays_in_bounds(dev):
    """A selection with an id outside [0, E) is reported as a routing error; its entry gets no row, so
    nothing left over from an earlier, larger forward is followed and the valid entries still count."""
    from ateniaengine_b200._lib import AteniaError
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=256, d_ff=256)
    w = synth.make_weights(shape, 17, dev)
    layer = synth.build_layer(shape, w, max_tokens=2048)
    big = synth.make_activations(shape, 17, dev, tokens=2048)
    layer.forward(big, sync=True)                       # leaves 4096 permutation entries behind
    x = synth.make_activations(shape, 18, dev, tokens=8)
    idx = torch.tensor([[0, 1]] * 8, dtype=torch.int32, device=dev)
    wts = torch.full((8, 2), 0.5, device=dev)
    good = layer.forward_selected(x, idx, wts, out_dtype=torch.float32)
    bad = idx.clone()
    bad[5, 1] = 99
    with pytest.raises(AteniaError) as ei:
        layer.forward_selected(x, bad, wts, out_dtype=torch.float32)
    assert ei.value.status == -9
    # the layer is usable afterwards and gives the same result as before
    again = layer.forward_selected(x, idx, wts, out_dtype=torch.float32)
    assert torch.equal(again, good)


def test_empty_batch_and_capacity(dev):
    from ateniaengine_b200._lib import AteniaError
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=256, d_ff=256)
    layer = synth.build_layer(shape, synth.make_weights(shape, 1, dev), max_tokens=8)
    out = layer.forward(torch.empty((0, 256), dtype=torch.bfloat16, device=dev), sync=True)
    assert out.shape == (0, 256)
    with pytest.raises(AteniaError) as ei:
        layer.forward(torch.zeros((9, 256), dtype=torch.bfloat16, device=dev))
    assert ei.value.status == -3  # more tokens than max_tokens


def test_token_order_does_not_change_rows(dev):
    """The block is position-wise: shuffling the tokens shuffles the outputs, bit for bit."""
    synth = _synth()
    shape = synth.small(synth.SHAPES["mixtral"], d_model=512, d_ff=1024)
    w = synth.make_weights(shape, 13, dev)
    x = synth.make_activations(shape, 13, dev, tokens=777)
    layer = synth.build_layer(shape, w, max_tokens=777)
    a = layer.forward(x, sync=True)
    p = torch.randperm(777, device=dev)
    b = layer.forward(x[p].contiguous(), sync=True)
    assert torch.equal(a[p], b)
    # and repeated calls are deterministic
    assert torch.equal(layer.forward(x, sync=True), a)


# ---- the reference's golden vectors, through the operator registry ------------------------------

def _golden(golden_dir, name):
    import os
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: z[k] for k in z.files}


def _pad16(a, axis):
    n = a.shape[axis]
    m = (n + 15) // 16 * 16
    if m == n:
        return a
    pad = [(0, 0)] * a.ndim
    pad[axis] = (0, m - n)
    return np.pad(a, pad)


@pytest.mark.parametrize("name,key,conv,renorm", [
    ("mixtral_layer0", "atenia_ref", "Atenia", True),
    ("qwen2_moe_layer0", "atenia_hf_ref", "HuggingFaceQwen", False),
    ("qwen2_moe_layer0", "atenia_ref", "Atenia", True),
    ("qwen3_moe_layer0", "atenia_ref", "Atenia", True),
    ("qwen15_moe_layer0", "atenia_hf_ref", "HuggingFaceQwen", False),
    ("deepseek_block", "mlp_output", "Atenia", False),
])
def test_reference_golden_vectors_through_registry(dev, golden_dir, name, key, conv, renorm):
    """register_real_moe_layer + execute_real_moe_layer on the reference's own fixtures.  d_ff that is
    not a multiple of 16 is zero-padded (zero gate/up rows give h = 0, zero down columns ignore it)."""
    import ateniaengine_b200 as ae
    g = _golden(golden_dir, name)
    E, F, d = g["gate"].shape
    gate = [_pad16(g["gate"][e], 0) for e in range(E)]
    up = [_pad16(g["up"][e], 0) for e in range(E)]
    down = [_pad16(g["down"][e], 1) for e in range(E)]
    shared = None
    if "shared_gate_proj" in g:
        shared = [_pad16(g["shared_gate_proj"], 0), _pad16(g["shared_up_proj"], 0), _pad16(g["shared_down_proj"], 1)]
    convention = ae.MoeExecutionConvention[conv]
    gate_vec = g.get("shared_gate_vec") if convention == ae.MoeExecutionConvention.HuggingFaceQwen else None
    cfg = ae.MoeLayerConfig(E, int(g["top_k"]), shared is not None, d, gate[0].shape[0])
    lid = ae.register_real_moe_layer(cfg, g["router"], gate, up, down, shared=shared, shared_gate=gate_vec,
                                     convention=convention, renormalize=renorm, max_tokens=64)
    out = ae.execute_real_moe_layer(lid, g["input"].astype(np.float32).ravel())
    assert rel_l2(out, g[key]) <= TOL_BF16


@pytest.mark.parametrize("name", ["qwen2_moe_layer0", "qwen15_moe_layer0"])
def test_execute_with_pins_the_convention_per_call(dev, golden_dir, name):
    """execute_real_moe_layer_with (src/moe/graph_op.rs:352-364) as the reference's convention tests use
    it (tests/moe_hf_convention_test.rs:124-156): ONE registered layer, with its gate vector, gives the
    Atenia result and the HuggingFace-Qwen result depending on the convention of the call."""
    import ateniaengine_b200 as ae
    g = _golden(golden_dir, name)
    E, F, d = g["gate"].shape
    gate = [_pad16(g["gate"][e], 0) for e in range(E)]
    up = [_pad16(g["up"][e], 0) for e in range(E)]
    down = [_pad16(g["down"][e], 1) for e in range(E)]
    shared = [_pad16(g["shared_gate_proj"], 0), _pad16(g["shared_up_proj"], 0), _pad16(g["shared_down_proj"], 1)]
    cfg = ae.MoeLayerConfig(E, int(g["top_k"]), True, d, gate[0].shape[0])
    # registered under the Atenia convention, gate vector supplied all the same
    lid = ae.register_real_moe_layer(cfg, g["router"], gate, up, down, shared=shared, shared_gate=g["shared_gate_vec"],
                                     convention=ae.MoeExecutionConvention.Atenia, max_tokens=64)
    x = g["input"].astype(np.float32).ravel()
    a = ae.execute_real_moe_layer_with(lid, x, ae.MoeExecutionConvention.Atenia)
    h = ae.execute_real_moe_layer_with(lid, x, ae.MoeExecutionConvention.HuggingFaceQwen)
    assert rel_l2(a, g["atenia_ref"]) <= TOL_BF16
    assert rel_l2(h, g["atenia_hf_ref"]) <= TOL_BF16
    assert np.max(np.abs(a - h)) > 1e-4          # the conventions do differ on these layers
    np.testing.assert_array_equal(ae.execute_real_moe_layer(lid, x), a)   # the layer's own convention


def test_forward_with_ignores_the_gate_under_the_atenia_convention(dev):
    """RealMoeLayer::forward_with on a device layer: two layers that differ in the gate vector only agree
    under Atenia and differ under HuggingFaceQwen (tests/moe_hf_convention_test.rs:110-121); without a
    shared expert the conventions differ by the renormalisation alone (:100-107)."""
    import ateniaengine_b200 as ae
    synth = _synth()
    shape = synth.small(synth.SHAPES["qwen_moe"], d_model=256, d_ff=128, shared_d_ff=256)
    w1 = synth.make_weights(shape, 41, dev)
    w2 = dict(w1)
    w2["shared_gate"] = (torch.randn(shape.d_model, device=dev) * 0.5).to(torch.bfloat16).float()
    x = synth.make_activations(shape, 41, dev, tokens=70)
    l1 = synth.build_layer(shape, w1, max_tokens=70)
    l2 = synth.build_layer(shape, w2, max_tokens=70)
    A, H = ae.MoeExecutionConvention.Atenia, ae.MoeExecutionConvention.HuggingFaceQwen
    a1 = l1.forward_with(x, A, out_dtype=torch.float32, sync=True)
    a2 = l2.forward_with(x, A, out_dtype=torch.float32, sync=True)
    h1 = l1.forward_with(x, H, out_dtype=torch.float32, sync=True)
    h2 = l2.forward_with(x, H, out_dtype=torch.float32, sync=True)
    assert torch.equal(a1, a2)
    assert (h1 - h2).abs().max() > 1e-4
    assert torch.equal(h1, l1.forward(x, out_dtype=torch.float32, sync=True))   # the layer's own convention
    # against the oracle under both conventions
    ol = oracle_layer(shape, w1)
    xs = x.float().cpu().numpy()
    assert rel_l2(h1.cpu().numpy(), ol.forward(xs)) <= TOL_BF16
    ol.renormalize, ol.shared_gated = True, False
    assert rel_l2(a1.cpu().numpy(), ol.forward(xs)) <= TOL_BF16


def test_registry_error_behaviour(dev, golden_dir):
    import ateniaengine_b200 as ae
    with pytest.raises(ae.MoeLayerError) as ei:
        ae.execute_real_moe_layer(10 ** 6, np.zeros(64, dtype=np.float32))
    assert ei.value.kind == "LayerNotFound"
    g = _golden(golden_dir, "mixtral_layer0")
    E, F, d = g["gate"].shape
    cfg = ae.MoeLayerConfig(E, 2, False, d, F)
    lid = ae.register_real_moe_layer(cfg, g["router"], list(g["gate"]), list(g["up"]), list(g["down"]), max_tokens=8)
    with pytest.raises(ae.MoeLayerError) as ei:
        ae.execute_real_moe_layer(lid, np.zeros(d + 1, dtype=np.float32))
    assert ei.value.kind == "DimMismatch"
    # a batch larger than the layer's capacity runs in passes; rows stay independent
    x = np.random.default_rng(0).normal(size=(19, d)).astype(np.float32)
    full = ae.execute_real_moe_layer(lid, x.ravel()).reshape(19, d)
    one = ae.execute_real_moe_layer(lid, x[11]).reshape(d)
    np.testing.assert_array_equal(full[11], one)
