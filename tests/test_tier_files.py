"""The reference's persistent expert tier files, read by the library's host-side readers.

The files are written here in the reference's formats (src/tensor/disk_tier.rs:168-197 for qint8,
plain little-endian f32, bf16 high halves; names from src/moe/residency.rs:492-505, :608-651)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc


@pytest.fixture(scope="module")
def tier():
    import __graft_entry__ as ge
    ge.build()
    from ateniaengine_b200 import tier as t
    return t


def _write_qint8(path, w):
    q, s = orc.quantize_per_row_i8(w)
    with open(path, "wb") as f:
        f.write(s.astype("<f4").tobytes())
        f.write(q.tobytes())
    return q, s


def _write_bf16(path, w):
    bits = (w.view(np.uint32) >> 16).astype("<u2")
    bits.tofile(path)
    return bits


def test_encodings_are_recognised_by_length(tier, tmp_path):
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, size=(12, 40)).astype(np.float32)
    pf, pb, pq = (str(tmp_path / n) for n in ("f.bin", "b.bin", "q.bin"))
    w.astype("<f4").tofile(pf)
    bits = _write_bf16(pb, w)
    q, s = _write_qint8(pq, w)
    assert tier.detect(pf, 12, 40) == tier.F32
    assert tier.detect(pb, 12, 40) == tier.BF16
    assert tier.detect(pq, 12, 40) == tier.QINT8
    k, a, sc = tier.read_tensor(pq, 12, 40)
    np.testing.assert_array_equal(a, q)
    np.testing.assert_array_equal(sc, s)
    k, a, _ = tier.read_tensor(pb, 12, 40)
    np.testing.assert_array_equal(a, bits)
    np.testing.assert_array_equal(tier.read_f32(pf, 12, 40), w)
    # materialised the way the reference does
    np.testing.assert_array_equal(tier.read_f32(pb, 12, 40), (bits.astype(np.uint32) << 16).view(np.float32))
    np.testing.assert_array_equal(tier.read_f32(pq, 12, 40), orc.dequantize_per_row_i8(q, s))


def test_bad_files_are_rejected(tier, tmp_path):
    p = str(tmp_path / "x.bin")
    with pytest.raises(tier.TierError) as ei:
        tier.detect(p, 4, 4)
    assert ei.value.status == -13
    np.zeros(17, dtype=np.uint8).tofile(p)
    with pytest.raises(tier.TierError) as ei:
        tier.detect(p, 4, 4)
    assert ei.value.status == -14
    # a 4x4 qint8 file is 32 bytes = a 4x4 bf16 file: the reference checks f32, bf16, then qint8
    np.zeros(32, dtype=np.uint8).tofile(p)
    assert tier.detect(p, 4, 4) == tier.BF16


def test_layer_directory_round_trip(tier, tmp_path):
    rng = np.random.default_rng(1)
    E, d, F, Fs = 3, 32, 48, 16
    d_ = str(tmp_path)
    router = rng.normal(0, 0.02, size=(E, d)).astype(np.float32)
    _write_bf16(os.path.join(d_, "L2.router.bin"), router)
    want = {"gate": [], "up": [], "down": []}
    for e in range(E):
        for role, shape in (("gate", (F, d)), ("up", (F, d)), ("down", (d, F))):
            w = rng.normal(0, 0.02, size=shape).astype(np.float32)
            want[role].append(_write_qint8(os.path.join(d_, f"L2.e{e}.{role}.bin"), w))
    for role, shape in (("gate", (Fs, d)), ("up", (Fs, d)), ("down", (d, Fs))):
        _write_qint8(os.path.join(d_, f"L2.shared.{role}.bin"), rng.normal(0, 0.02, size=shape).astype(np.float32))
    gate_vec = rng.normal(0, 0.02, size=(d,)).astype(np.float32)
    gate_vec.astype("<f4").tofile(os.path.join(d_, "L2.shared_gate.bin"))
    json.dump({"version": 5, "model_id": "0" * 16, "family": "qwen_moe", "num_hidden_layers": 3, "num_experts": E,
               "experts_per_token": 2, "hidden_size": d, "moe_intermediate_size": F, "convention": "hf_qwen",
               "has_shared": True, "attn_has_bias": False, "tensor_count": 0, "total_bytes": 0, "entries": []},
              open(os.path.join(d_, "tier_manifest.json"), "w"))
    m = tier.read_manifest(d_)
    assert m["convention"] == "hf_qwen"
    host = tier.read_layer(d_, 2, E, d, F, shared_d_ff=Fs, shared_gate=True)
    assert host["kind"] == tier.QINT8
    np.testing.assert_array_equal(host["router"], (((router.view(np.uint32) >> 16) << 16)).view(np.float32))
    for role in ("gate", "up", "down"):
        for e in range(E):
            np.testing.assert_array_equal(host[role][e], want[role][e][0])
            np.testing.assert_array_equal(host["scales"][role][e], want[role][e][1])
    np.testing.assert_array_equal(host["shared_gate"], gate_vec)
    assert len(host["shared"]) == 3 and host["shared"][2].shape == (d, Fs)
    # the oracle consumes the same arrays directly
    lay = orc.OracleLayer(host["router"], host["gate"], host["up"], host["down"], 2, False, shared=host["shared"],
                          shared_gate_vec=host["shared_gate"], scales=host["scales"],
                          shared_scales=host["shared_scales"])
    y = lay.forward(rng.normal(size=(2, d)).astype(np.float32))
    assert np.isfinite(y).all()
    # an older manifest is refused
    json.dump({"version": 4}, open(os.path.join(d_, "tier_manifest.json"), "w"))
    with pytest.raises(ValueError):
        tier.read_manifest(d_)
