"""Sub-batch plan of the host-buffer operator (atenia_moe_plan_exec_pieces): host arithmetic only."""
import ctypes as C

import pytest


def _cfg(name):
    from ateniaengine_b200 import MoeLayerConfig, synth
    s = synth.SHAPES[name]
    return s, MoeLayerConfig(s.num_experts, s.top_k, s.shared_d_ff > 0, s.d_model, s.d_ff)


@pytest.mark.parametrize("name,n,cap", [("mixtral", 4096, 4096), ("mixtral", 1, 4096), ("mixtral", 300, 4096),
                                        ("mixtral", 10000, 4096), ("deepseek_v2_lite", 8192, 8192),
                                        ("qwen_moe", 2048, 2048), ("mixtral_int8", 4096, 4096), ("tiny", 64, 64),
                                        ("tiny", 5000, 512)])
def test_pieces_cover_the_batch_and_respect_max_tokens(name, n, cap):
    from ateniaengine_b200 import plan_exec_pieces
    s, cfg = _cfg(name)
    pieces = plan_exec_pieces(cfg, n, shared_d_ff=s.shared_d_ff, int8=s.int8, max_tokens=cap)
    assert sum(pieces) == n
    assert all(0 < p <= cap for p in pieces)
    assert len(pieces) >= -(-n // cap)


def test_small_batches_stay_whole_and_large_ones_get_short_ends():
    from ateniaengine_b200 import plan_exec_pieces
    s, cfg = _cfg("mixtral")
    assert plan_exec_pieces(cfg, 256, max_tokens=4096) == [256]
    assert plan_exec_pieces(cfg, 1024, max_tokens=4096) == [1024]
    # a layer slower than the link: the exposed copies (first in, last out) belong to short pieces
    pieces = plan_exec_pieces(cfg, 4096, max_tokens=4096)
    assert len(pieces) == 3 and pieces[0] == pieces[2] and pieces[0] * 2 < pieces[1]
    # a layer faster than the link: pieces of similar size, more than two of them
    s2, cfg2 = _cfg("deepseek_v2_lite")
    p2 = plan_exec_pieces(cfg2, 8192, shared_d_ff=s2.shared_d_ff, max_tokens=8192)
    assert len(p2) >= 3 and max(p2) <= 2 * min(p2)


def test_argument_checks():
    from ateniaengine_b200 import _lib
    from ateniaengine_b200.moe import _plan_config
    s, cfg = _cfg("mixtral")
    c = _plan_config(cfg, 0, False, 4096)
    buf = (C.c_uint64 * 2)()
    lib = _lib.lib()
    assert lib.atenia_moe_plan_exec_pieces(None, 4096, buf, 2) == -1          # ATENIA_ERR_NULL
    assert lib.atenia_moe_plan_exec_pieces(C.byref(c), 4096, None, 2) == -1
    assert lib.atenia_moe_plan_exec_pieces(C.byref(c), 4096, buf, 0) == -2    # ATENIA_ERR_SHAPE
    assert lib.atenia_moe_plan_exec_pieces(C.byref(c), 4096, buf, 2) == -3    # three pieces do not fit two slots
    assert lib.atenia_moe_plan_exec_pieces(C.byref(c), 0, buf, 2) == 0


def test_plan_follows_measured_figures():
    """The cut from timings: the forward of an end piece should last about as long as the copy of the
    middle one when the layer is slower than the link; a link slower than the layer wants similar pieces;
    a forward that is nearly all fixed cost is not cut at all."""
    from ateniaengine_b200 import plan_exec_pieces
    s, cfg = _cfg("mixtral")
    # Mixtral shape as measured on B200: forward(T) = 0.49 + 0.00041 T ms, 0.00031 ms per token and copy
    p = plan_exec_pieces(cfg, 4096, max_tokens=4096, measured=(0.49, 0.00041, 0.00031))
    assert len(p) == 3 and p[0] == p[2] and 512 <= p[0] <= 1024
    end_forward = 0.49 + 0.00041 * p[0]
    middle_copy = 0.00031 * p[1]
    assert abs(end_forward - middle_copy) < 0.15
    # the same layer behind a link ten times slower: copies dominate, pieces of similar size
    q = plan_exec_pieces(cfg, 4096, max_tokens=4096, measured=(0.49, 0.00041, 0.0031))
    assert len(q) >= 3 and max(q) <= 3 * min(q)
    # a forward that costs 5 ms whatever the batch: every extra piece costs more than its overlap gains
    assert plan_exec_pieces(cfg, 4096, max_tokens=4096, measured=(5.0, 0.00001, 0.00031)) == [4096]
    # negative figures are refused
    from ateniaengine_b200 import _lib
    with pytest.raises(_lib.AteniaError):
        plan_exec_pieces(cfg, 4096, max_tokens=4096, measured=(-1.0, 0.1, 0.1))
