"""DeepSeek-V3 routing on the GPU (router_mode = 1): the reference's v3_route_ref golden block, a
larger synthetic layer against the oracle, and routing from given logits (integer results bit-exact)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.helpers import rel_l2

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _pad16(a, axis):
    n = a.shape[axis]
    m = (n + 15) // 16 * 16
    if m == n:
        return a
    pad = [(0, 0)] * a.ndim
    pad[axis] = (0, m - n)
    return np.pad(a, pad)


def test_v3_golden_block_on_gpu(golden_dir):
    import ateniaengine_b200 as ae
    dev = _dev()
    z = np.load(os.path.join(golden_dir, "v3_route_ref.npz"))
    E, F, d = z["gate"].shape
    bf = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev).to(torch.bfloat16)
    gate = [bf(_pad16(z["gate"][e], 0)) for e in range(E)]
    up = [bf(_pad16(z["up"][e], 0)) for e in range(E)]
    down = [bf(_pad16(z["down"][e], 1)) for e in range(E)]
    shared = [bf(_pad16(z["shared_gate_proj"], 0)), bf(_pad16(z["shared_up_proj"], 0)), bf(_pad16(z["shared_down_proj"], 1))]
    cfg = ae.MoeLayerConfig(E, int(z["top_k"]), True, d, gate[0].shape[0])
    v3 = {"n_group": int(z["n_group"]), "topk_group": int(z["topk_group"]),
          "scaling": float(z["routed_scaling_factor"]), "e_score_bias": torch.from_numpy(z["router_bias"]).to(dev)}
    layer = ae.RealMoeLayer(cfg, torch.from_numpy(z["router"]).to(dev), gate, up, down, shared=shared,
                            convention=ae.MoeExecutionConvention.Atenia, renormalize=bool(z["norm_topk_prob"]),
                            max_tokens=16, v3=v3)
    x = torch.from_numpy(z["hidden"]).to(dev)
    out, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    np.testing.assert_array_equal(aux["topk_idx"].cpu().numpy(), z["selected_experts"])
    dense = np.zeros((x.shape[0], E))
    np.put_along_axis(dense, aux["topk_idx"].cpu().numpy().astype(np.int64), aux["topk_w"].cpu().numpy(), axis=1)
    assert np.max(np.abs(dense - z["dense_combine_weights"])) < 1e-5
    assert rel_l2(out.cpu().numpy(), z["block_out"]) <= 1e-2


def test_v3_synthetic_layer_matches_oracle():
    from ateniaengine_b200 import synth
    from tests.helpers import oracle_layer
    dev = _dev()
    shape = synth.small(synth.SHAPES["deepseek_v2_lite"], d_model=512, d_ff=384, shared_d_ff=256)
    w = synth.make_weights(shape, 77, dev)
    g = torch.Generator(device=dev).manual_seed(5)
    bias = torch.randn((shape.num_experts,), generator=g, device=dev) * 0.05
    v3 = {"n_group": 8, "topk_group": 3, "scaling": 2.5, "e_score_bias": bias}
    from ateniaengine_b200 import MoeExecutionConvention, MoeLayerConfig, RealMoeLayer
    cfg = MoeLayerConfig(shape.num_experts, shape.top_k, True, shape.d_model, shape.d_ff)
    layer = RealMoeLayer(cfg, w["router"], w["gate"], w["up"], w["down"], shared=w["shared"],
                         convention=MoeExecutionConvention.Atenia, renormalize=True, max_tokens=300, v3=v3)
    x = synth.make_activations(shape, 77, dev, tokens=300)
    out, aux = layer.forward(x, out_dtype=torch.float32, aux=True, sync=True)
    ol = oracle_layer(shape, w)
    ol.renormalize = True
    ol.v3 = {"n_group": 8, "topk_group": 3, "scaling": 2.5}
    ol.e_score_bias = bias.cpu().numpy()
    ref, raux = ol.forward(x.float().cpu().numpy(), want_aux=True)
    # selection follows from the kernel's own logits exactly as on the CPU
    lg = aux["logits"].cpu().numpy()
    for t in range(300):
        rc, idx, wts, _ = orc.v3_route(lg[t], ol.e_score_bias, shape.top_k, 8, 3, 2.5, True)
        assert rc == 0
        assert idx.tolist() == aux["topk_idx"][t].cpu().numpy().tolist()
        np.testing.assert_allclose(aux["topk_w"][t].cpu().numpy(), wts, rtol=2e-7, atol=0)
    same = (aux["topk_idx"].cpu().numpy() == raux["topk_idx"]).all(axis=1)
    assert same.mean() >= 0.99
    assert rel_l2(out.cpu().numpy()[same], ref[same]) <= 1e-2
    # routing only, from given logits
    idx2, w2, perm, inv, off = layer.route_from_logits(aux["logits"])
    assert torch.equal(idx2, aux["topk_idx"])
    off_ref, perm_ref, _ = orc.dispatch_permutation(idx2.cpu().numpy(), shape.num_experts)
    np.testing.assert_array_equal(perm.cpu().numpy(), perm_ref)
    np.testing.assert_array_equal(off.cpu().numpy(), off_ref)
