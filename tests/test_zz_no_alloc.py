"""The entry point that allocates nothing (atenia_moe_dispatch_noalloc), against the existing one.

Some hosts cannot call cudaMalloc -- the host runtime owns all device memory in its own pool, or an
allocation's device-wide synchronisation is not acceptable where they run -- so they cannot hold an
AteniaMoeLayer.  For them the library computes the dispatch order with scratch that is compiled into
it.  This file checks, through the C ABI, that two calls in a row give exactly what
atenia_moe_route_from_logits gives for the same routing (integer results: bit-exact), that stale
scratch from a larger call does not leak into a smaller one, and that requests beyond the fixed
scratch are refused.  It is collected last so that a run that stops at the first failure has already
run every other test; it also passes when run alone in a fresh process.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_noalloc_dispatch_matches_layer_dispatch_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ateniaengine_b200 import synth
    from ateniaengine_b200.moe import dispatch_noalloc

    dev = torch.device("cuda:0")
    E, k = 64, 6
    shape = synth.MoeShape("noalloc", 64, 64, E, k, False)
    layer = synth.build_layer(shape, synth.make_weights(shape, 1, dev), max_tokens=4096)
    gen = torch.Generator(device=dev).manual_seed(5)
    # first a large batch, then a small one: the second call sees the first call's leftovers
    for T in (4096, 301):
        logits = torch.randn((T, E), generator=gen, device=dev)
        idx, _, perm_ref, inv_ref, off_ref = layer.route_from_logits(logits)
        perm = torch.full((T * k,), -1, dtype=torch.int32, device=dev)
        inv = torch.full((T * k,), -1, dtype=torch.int32, device=dev)
        off = torch.full((E + 1,), -1, dtype=torch.int32, device=dev)
        assert dispatch_noalloc(idx, E, perm, inv, off) == 0
        torch.cuda.synchronize()
        assert torch.equal(off, off_ref)
        assert torch.equal(perm, perm_ref)
        assert torch.equal(inv, inv_ref)
        # and against the CPU statement of the same order, which shares no code with the library
        o_off, o_perm, o_inv = orc.dispatch_permutation(idx.cpu().numpy(), E)
        np.testing.assert_array_equal(off.cpu().numpy(), o_off)
        np.testing.assert_array_equal(perm.cpu().numpy(), o_perm)
        np.testing.assert_array_equal(inv.cpu().numpy(), o_inv)


def test_noalloc_dispatch_refuses_requests_beyond_its_scratch():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ateniaengine_b200.moe import dispatch_noalloc

    dev = torch.device("cuda:0")
    idx = torch.zeros((65536 // 8 + 1, 8), dtype=torch.int32, device=dev)
    out = torch.zeros((idx.numel(),), dtype=torch.int32, device=dev)
    off = torch.zeros((130,), dtype=torch.int32, device=dev)
    assert dispatch_noalloc(idx, 8, out, out.clone(), off) == -12     # T*k = 65544 > 65536
    assert dispatch_noalloc(idx[:16], 129, out, out.clone(), off) == -12  # E > 128
    assert dispatch_noalloc(idx[:16], 8, out, out.clone(), off) == 0
    torch.cuda.synchronize()
    assert off[:9].tolist() == [0] + [128] * 8
