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
