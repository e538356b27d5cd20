"""The expert-residency planner: the reference's capacity rule
(auto_expert_cache_capacity, src/moe/residency.rs:201-211; its unit tests :1450-1480 give the
known answers used here) and the placement it drives on B200 (smallest expert-parallel world in which
every rank's experts are resident in HBM).  Host arithmetic only."""
import pytest


def test_capacity_rule_known_answers():
    from ateniaengine_b200 import auto_expert_cache_capacity as cap
    # budget / (layers * bytes) clamped to [1, E]
    assert cap(1000, 2, 100, 8) == 5
    assert cap(10 ** 12, 2, 100, 8) == 8      # never more than the experts there are
    assert cap(1, 32, 10 ** 9, 8) == 1        # never less than one
    assert cap(0, 0, 0, 0) == 1               # degenerate inputs: max(.., 1) everywhere
    assert cap(2 ** 63, 2 ** 40, 2 ** 40, 64) == 1  # the product saturates instead of wrapping


def _cfg(name):
    from ateniaengine_b200 import MoeLayerConfig, synth
    s = synth.SHAPES[name]
    return s, MoeLayerConfig(s.num_experts, s.top_k, s.shared_d_ff > 0, s.d_model, s.d_ff)


def test_mixtral_8x7b_bf16_needs_sharding_and_int8_fits_one_gpu():
    from ateniaengine_b200 import plan_residency
    s, cfg = _cfg("mixtral")
    hbm = 180 * 10 ** 9
    rc, p = plan_residency(cfg, 32, hbm, max_tokens=4096)
    # 32 layers x 8 experts x 352 MB = 90 GB of experts: one B200 holds them
    assert rc == 0 and p["min_ep_world"] == 1 and p["resident_experts_per_layer"] == 8
    assert p["bytes_per_expert"] == 3 * s.d_model * s.d_ff * 2
    assert p["bytes_per_rank"] <= hbm
    # on a 80 GB budget the same model needs two ranks; on 40 GB four (decode-sized workspaces: every
    # layer owns one, and under expert parallelism it includes the receive buffers)
    rc, p = plan_residency(cfg, 32, 80 * 10 ** 9, max_tokens=256)
    assert rc == 0 and p["min_ep_world"] == 2 and p["experts_per_rank"] == 4
    rc, p = plan_residency(cfg, 32, 40 * 10 ** 9, max_tokens=256)
    assert rc == 0 and p["min_ep_world"] == 4
    assert p["fixed_bytes_per_rank"] + 2 * 32 * p["bytes_per_expert"] == p["bytes_per_rank"]
    # int8 halves the expert bytes: 80 GB hold all of it again
    rc, p8 = plan_residency(cfg, 32, 80 * 10 ** 9, int8=True, max_tokens=256)
    assert rc == 0 and p8["min_ep_world"] == 1
    assert p8["bytes_per_expert"] < p["bytes_per_expert"] * 0.51


def test_a_model_that_does_not_fit_eight_ranks_is_refused():
    from ateniaengine_b200 import auto_expert_cache_capacity, plan_residency
    _, cfg = _cfg("mixtral")
    budget = 5 * 10 ** 9
    rc, p = plan_residency(cfg, 32, budget, max_tokens=4096)
    assert rc == -3
    assert p["min_ep_world"] == 8 and p["experts_per_rank"] == 1
    assert p["resident_experts_per_layer"] < p["experts_per_rank"]
    assert p["bytes_per_rank"] > budget
    # what is reported is the reference's rule on the budget left after the fixed costs
    left = budget - p["fixed_bytes_per_rank"]
    if left > 0:
        assert auto_expert_cache_capacity(left, 32, p["bytes_per_expert"], 1) == 1


def test_expert_count_must_divide():
    from ateniaengine_b200 import plan_residency
    _, cfg = _cfg("qwen_moe")   # 60 experts: worlds 1, 2, 4 only
    s, _ = _cfg("qwen_moe")
    rc, p = plan_residency(cfg, 24, 10 ** 9, shared_d_ff=s.shared_d_ff, max_tokens=256)
    assert p["min_ep_world"] in (1, 2, 4)
    rc2, p2 = plan_residency(cfg, 24, 180 * 10 ** 9, shared_d_ff=s.shared_d_ff, max_tokens=2048)
    assert rc2 == 0 and p2["min_ep_world"] == 1 and p2["resident_experts_per_layer"] == 60


def test_argument_errors():
    import ctypes as C
    from ateniaengine_b200 import MoeLayerConfig, _lib, plan_residency
    lib = _lib.lib()
    assert lib.atenia_moe_plan_residency(None, 1, 1, None) == -1
    rc, _ = plan_residency(MoeLayerConfig(8, 2, False, 4096, 14336), 0, 10 ** 9)
    assert rc == -2
    rc, _ = plan_residency(MoeLayerConfig(8, 2, False, 4090, 14336), 1, 10 ** 9)
    assert rc == -2


@pytest.mark.gpu
def test_workspace_bytes_match_what_create_allocates():
    """The planner's workspace figure against the free-memory delta of a real atenia_moe_create."""
    import torch
    from ateniaengine_b200 import synth, workspace_bytes, MoeLayerConfig
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    dev = torch.device("cuda:0")
    shape = synth.small(synth.SHAPES["deepseek_v2_lite"], d_model=1024, d_ff=512, shared_d_ff=1024)
    w = synth.make_weights(shape, 3, dev)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    free0, _ = torch.cuda.mem_get_info()
    layer = synth.build_layer(shape, w, max_tokens=8192)
    free1, _ = torch.cuda.mem_get_info()
    cfg = MoeLayerConfig(shape.num_experts, shape.top_k, True, shape.d_model, shape.d_ff)
    want = workspace_bytes(cfg, shared_d_ff=shape.shared_d_ff, max_tokens=8192)
    got = free0 - free1
    # the driver allocates in 2 MiB granules; small buffers share them
    assert abs(got - want) <= 0.05 * want + 64 * 2 ** 20, (got, want)
    layer.close()
