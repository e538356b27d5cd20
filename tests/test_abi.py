"""CPU-only checks of the C ABI: the library loads, exports every symbol the header declares, and
rejects bad arguments before touching a device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    from ateniaengine_b200 import _lib
    return _lib.lib()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "atenia_moe.h")).read()
    return sorted(set(re.findall(r"ATENIA_API\s+[\w\s\*]+?\b(atenia_\w+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    names = _declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/atenia_moe.h but not exported"


def test_python_binding_lists_every_symbol():
    from ateniaengine_b200 import _lib
    assert sorted(_lib.EXPORTS) == _declared_symbols()


def test_status_strings(lib):
    assert lib.atenia_moe_status_str(0) == b"ok"
    assert b"not found" in lib.atenia_moe_status_str(-5)
    assert b"d_model" in lib.atenia_moe_status_str(-6)
    assert lib.atenia_moe_status_str(-12345) == b"unknown status"


def test_create_rejects_bad_arguments_without_a_device(lib):
    from ateniaengine_b200 import _lib
    h = C.c_void_p()
    assert lib.atenia_moe_create(None, C.byref(h)) == -1
    good = dict(num_experts=8, experts_per_token=2, d_model=512, d_ff=1408, shared_d_ff=0, renormalize=1,
                shared_gated=0, weight_dtype=0, max_tokens=64, ep_rank=0, ep_world=1)
    for bad in (dict(num_experts=0), dict(experts_per_token=9), dict(experts_per_token=0), dict(d_model=100),
                dict(d_ff=8), dict(shared_d_ff=24), dict(weight_dtype=5), dict(max_tokens=0), dict(ep_world=3),
                dict(ep_world=2, ep_rank=2), dict(num_experts=6, ep_world=4), dict(num_experts=129)):
        cfg = _lib.MoeConfig(**{**good, **bad})
        assert lib.atenia_moe_create(C.byref(cfg), C.byref(h)) == -2, bad
        assert not h.value


def test_create_rejects_invalid_v3_router_configs_without_a_device(lib):
    """V3RouterConfig::validate (src/moe/v3_router.rs:150-183) at the ABI."""
    from ateniaengine_b200 import _lib
    h = C.c_void_p()
    base = dict(num_experts=8, experts_per_token=2, d_model=64, d_ff=64, shared_d_ff=0, renormalize=1,
                shared_gated=0, weight_dtype=0, max_tokens=8, ep_rank=0, ep_world=1, router_mode=1, n_group=4,
                topk_group=2, routed_scaling_factor=2.5)
    for bad in (dict(n_group=0), dict(topk_group=0), dict(n_group=3), dict(n_group=8), dict(topk_group=5),
                dict(experts_per_token=5), dict(router_mode=2)):
        cfg = _lib.MoeConfig(**{**base, **bad})
        assert lib.atenia_moe_create(C.byref(cfg), C.byref(h)) == -2, bad
        assert not h.value


def test_registry_rejects_unknown_layer_and_null(lib):
    x = np.zeros(16, dtype=np.float32)
    assert lib.atenia_execute_real_moe_layer(12345, x.ctypes.data, 16, x.ctypes.data) == -5
    assert lib.atenia_execute_real_moe_layer(-1, x.ctypes.data, 16, x.ctypes.data) == -5
    assert lib.atenia_register_real_moe_layer(None) == -1
    assert lib.atenia_get_real_moe_layer(7) is None


def test_null_handles(lib):
    assert lib.atenia_moe_forward(None, None, 0, 1, None, 0, None, None) == -1
    assert lib.atenia_moe_check(None, None) == -1
    assert lib.atenia_moe_set_weights(None, None) == -1
    assert lib.atenia_moe_destroy(None) == 0
    assert lib.atenia_moe_last_gemm_ms(None, 0) < 0
    assert lib.atenia_moe_ep_unique_id_bytes() == 128
    assert lib.atenia_moe_counter(99) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ateniaengine_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.lib()
