"""The seeded synthetic layers that stand in for checkpoints: shapes, value distributions and
determinism (CPU generator; the GPU generator draws different numbers from the same distributions)."""
import numpy as np
import torch

from ateniaengine_b200 import synth


def test_shapes_of_the_benchmark_configurations():
    s = synth.SHAPES
    assert (s["tiny"].d_model, s["tiny"].d_ff, s["tiny"].num_experts, s["tiny"].top_k, s["tiny"].tokens) == (512, 1408, 8, 2, 64)
    assert (s["mixtral"].d_model, s["mixtral"].d_ff, s["mixtral"].num_experts, s["mixtral"].top_k) == (4096, 14336, 8, 2)
    assert s["mixtral"].renormalize and s["mixtral"].bias == "normal"
    q = s["qwen_moe"]
    assert (q.d_model, q.d_ff, q.num_experts, q.top_k, q.shared_d_ff, q.shared_gated, q.renormalize) == (
        2048, 1408, 60, 4, 5632, True, False)
    d = s["deepseek_v2_lite"]
    assert (d.d_model, d.d_ff, d.num_experts, d.top_k, d.shared_d_ff, d.shared_gated, d.renormalize, d.tokens) == (
        2048, 1408, 64, 6, 2816, False, False, 8192)
    assert s["mixtral_int8"].int8 and s["mixtral_int8"].bias == "zipf"


def test_distributions_and_determinism():
    shape = synth.small(synth.SHAPES["qwen_moe"], d_model=256, d_ff=128, shared_d_ff=64)
    a = synth.make_weights(shape, 3, "cpu")
    b = synth.make_weights(shape, 3, "cpu")
    c = synth.make_weights(shape, 4, "cpu")
    assert torch.equal(a["gate"][7], b["gate"][7]) and not torch.equal(a["gate"][7], c["gate"][7])
    w = torch.cat([m.float().flatten() for m in a["gate"]])
    assert abs(float(w.std()) - 0.02) < 5e-4 and abs(float(w.mean())) < 2e-4
    assert a["gate"][0].dtype == torch.bfloat16 and a["gate"][0].shape == (128, 256) and a["down"][0].shape == (256, 128)
    assert a["router"].dtype == torch.float32
    assert torch.equal(a["router"], a["router"].to(torch.bfloat16).float())  # representable in bf16
    assert a["shared"][0].shape == (64, 256) and a["shared_gate"].shape == (256,)
    x = synth.make_activations(shape, 3, "cpu", tokens=4096)
    assert abs(float(x.float().std()) - 1.0) < 0.02
    # expert slices for expert parallelism see the same layer
    part = synth.make_weights(shape, 3, "cpu", experts=(20, 10))
    assert len(part["gate"]) == 10 and torch.equal(part["gate"][0], a["gate"][20]) and torch.equal(part["down"][9], a["down"][29])
    assert torch.equal(part["shared"][2], a["shared"][2])


def test_routing_skew_inputs():
    n = synth.make_weights(synth.small(synth.SHAPES["mixtral"], d_model=64, d_ff=64), 1, "cpu")
    assert n["router_bias"].shape == (8,) and 0.1 < float(n["router_bias"].std()) < 1.2
    from dataclasses import replace
    z = synth.make_weights(replace(synth.small(synth.SHAPES["mixtral_int8"], d_model=64, d_ff=64), int8=False), 1, "cpu")
    got = np.sort(z["router_bias"].numpy())[::-1]
    np.testing.assert_allclose(got, -1.1 * np.log(np.arange(1, 9)), rtol=1e-6)
