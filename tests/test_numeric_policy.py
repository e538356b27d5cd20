"""The numeric-policy switch at the C ABI against the reference's rules
(src/moe/numeric_policy.rs:37-127): names, precedence (override, environment read once, Certified),
which policies use f32 / the GPU, and the gate the operator entry points apply.  No GPU needed: the
gate answers before any CUDA call."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_names_follow_the_reference():
    from ateniaengine_b200 import NumericPolicy
    # from_str: case-insensitive, trimmed, with the f64 / f32 aliases (numeric_policy.rs:56-63)
    assert NumericPolicy.from_str("certified") is NumericPolicy.Certified
    assert NumericPolicy.from_str(" F64 ") is NumericPolicy.Certified
    assert NumericPolicy.from_str("Strict") is NumericPolicy.Strict
    assert NumericPolicy.from_str("f32") is NumericPolicy.Strict
    assert NumericPolicy.from_str("FAST") is NumericPolicy.Fast
    assert NumericPolicy.from_str("tf32") is None
    assert NumericPolicy.from_str("") is None
    assert [p.as_str() for p in NumericPolicy] == ["certified", "strict", "fast"]
    # ffn_uses_f32 / ffn_uses_cuda (numeric_policy.rs:65-77)
    assert [p.ffn_uses_f32() for p in NumericPolicy] == [False, True, True]
    assert [p.ffn_uses_cuda() for p in NumericPolicy] == [False, False, True]


def test_override_wins_and_clears():
    import ateniaengine_b200 as ae
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    try:
        ae.set_numeric_policy(ae.NumericPolicy.Strict)
        assert ae.numeric_policy() is ae.NumericPolicy.Strict
        assert lib.atenia_numeric_policy_is_explicit() == 1
        assert lib.atenia_numeric_policy_gate() == _lib.ERR_POLICY
        ae.set_numeric_policy(ae.NumericPolicy.Fast)
        assert lib.atenia_numeric_policy_gate() == 0
        assert lib.atenia_set_numeric_policy(7) == -2
        assert ae.numeric_policy() is ae.NumericPolicy.Fast
    finally:
        ae.clear_numeric_policy_override()


def test_operator_entry_points_apply_the_gate_before_anything_else():
    """Under an explicit Certified / Strict selection execute_real_moe_layer refuses (the host runs its
    own CPU arm, as matvec_policy does); with Fast or no selection it goes on to its normal checks."""
    import ateniaengine_b200 as ae
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    buf = np.zeros(64, dtype=np.float32)
    call = lambda: lib.atenia_execute_real_moe_layer(10 ** 6, C.c_void_p(buf.ctypes.data), 64, C.c_void_p(buf.ctypes.data))
    try:
        ae.set_numeric_policy(ae.NumericPolicy.Certified)
        assert call() == _lib.ERR_POLICY
        with pytest.raises(ae.MoeLayerError) as ei:
            ae.execute_real_moe_layer(10 ** 6, buf)
        assert ei.value.kind == "NumericPolicy"
        ae.set_numeric_policy(ae.NumericPolicy.Fast)
        assert call() == _lib.ERR_LAYER_NOT_FOUND
    finally:
        ae.clear_numeric_policy_override()
    assert lib.atenia_execute_real_moe_layer_with(10 ** 6, C.c_void_p(buf.ctypes.data), 64, C.c_void_p(buf.ctypes.data), 5) in (
        -2, _lib.ERR_POLICY)


@pytest.mark.parametrize("env,policy,explicit,gate", [
    (None, "certified", 0, 0),         # unset: Certified by the reference's rule, but nothing was selected
    ("fast", "fast", 1, 0),
    ("strict", "strict", 1, -15),
    ("F64", "certified", 1, -15),
    ("bogus", "certified", 0, 0),      # unknown value: as if unset (numeric_policy.rs:100-105)
])
def test_environment_is_read_once_in_a_fresh_process(env, policy, explicit, gate):
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from ateniaengine_b200 import _lib\n"
            "l = _lib.lib()\n"
            "print(l.atenia_numeric_policy_str(l.atenia_numeric_policy()).decode(), "
            "l.atenia_numeric_policy_is_explicit(), l.atenia_numeric_policy_gate())\n") % ROOT
    e = dict(os.environ)
    e.pop("ATENIA_NUMERIC_POLICY", None)
    if env is not None:
        e["ATENIA_NUMERIC_POLICY"] = env
    out = subprocess.run([sys.executable, "-c", code], env=e, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == [policy, str(explicit), str(gate)]
