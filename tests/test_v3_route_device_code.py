"""The library's DeepSeek-V3 routing function (ateniaengine_b200/csrc/v3_route.cuh, the code the CUDA
kernel runs per thread) compiled for the host and compared with the oracle on the reference's golden
vector and on random cases with ties."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    so = tmp_path_factory.mktemp("v3") / "libv3probe.so"
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-shared", "-fPIC",
                           os.path.join(ROOT, "tests", "v3_host_probe.cpp"), "-o", str(so)])
    lib = C.CDLL(str(so))
    lib.v3_probe_route.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double,
                                   C.c_void_p, C.c_void_p]

    def route(logits, bias, top_k, n_group, topk_group, scaling, norm):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        idx = np.zeros(8, dtype=np.int32)
        w = np.zeros(8, dtype=np.float32)
        rc = lib.v3_probe_route(logits.ctypes.data, bias.ctypes.data, logits.size, top_k, n_group, topk_group,
                                int(norm), float(scaling), idx.ctypes.data, w.ctypes.data)
        return rc, idx[:max(top_k, 0)], w[:max(top_k, 0)]
    return route


def test_device_code_matches_golden(probe, golden_dir):
    z = np.load(os.path.join(golden_dir, "v3_route_ref.npz"))
    args = (int(z["top_k"]), int(z["n_group"]), int(z["topk_group"]), float(z["routed_scaling_factor"]),
            bool(z["norm_topk_prob"]))
    for t in range(z["hidden"].shape[0]):
        logits = orc.router_logits(z["router"], z["hidden"][t])
        rc, idx, w = probe(logits, z["router_bias"], *args)
        assert rc == 0 and idx.tolist() == z["selected_experts"][t].tolist()
        dense = np.zeros(z["router"].shape[0])
        dense[idx] = w
        assert np.max(np.abs(dense - z["dense_combine_weights"][t])) < 1e-6


def test_device_code_matches_oracle_on_random_cases(probe):
    rng = np.random.default_rng(0)
    for n, top_k, n_group, topk_group in [(8, 2, 4, 2), (64, 6, 8, 3), (128, 8, 8, 4), (60, 4, 6, 6), (16, 8, 2, 2)]:
        for trial in range(200):
            logits = rng.normal(0, 2, size=n).astype(np.float32)
            bias = rng.normal(0, 0.1, size=n).astype(np.float32)
            if trial % 4 == 0:  # ties: quantised values
                logits = np.round(logits)
                bias = np.zeros(n, dtype=np.float32)
            norm = bool(trial % 2)
            rc, idx, w = probe(logits, bias, top_k, n_group, topk_group, 2.5, norm)
            rc2, idx2, w2, _ = orc.v3_route(logits, bias, top_k, n_group, topk_group, 2.5, norm)
            assert rc == rc2 == 0
            assert idx.tolist() == idx2.tolist()
            np.testing.assert_array_equal(w, w2)


def test_device_code_rejects_what_the_reference_rejects(probe):
    z = np.zeros(8, dtype=np.float32)
    assert probe(z, z, 0, 4, 2, 1.0, True)[0] == -1
    assert probe(z, z, 2, 3, 2, 1.0, True)[0] == -2
    assert probe(z, z, 2, 8, 2, 1.0, True)[0] == -3
    assert probe(z, z, 2, 4, 5, 1.0, True)[0] == -4
    assert probe(z, z, 5, 4, 2, 1.0, True)[0] == -5
    bad = z.copy()
    bad[1] = np.nan
    assert probe(bad, z, 2, 4, 2, 1.0, True)[0] == -6
