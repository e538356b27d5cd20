"""Data formats either side of the block, end to end on the GPU: a persistent expert tier written in
the reference's layout is loaded into a device layer WITHOUT re-quantising and matches the oracle run
on the same file contents; a checkpoint dict in each model family's tensor naming (classic and packed
experts) is bound, uploaded and reproduces the reference's golden block outputs.

Formats: src/tensor/disk_tier.rs:168-224 (qint8 = [rows x f32 scales][rows*cols x i8]), names
src/moe/residency.rs:492-505, :608-651, manifest src/moe/runtime.rs:146-206; binding
src/moe/binding.rs:254-315, :381-447.  Bars: rel-L2 <= 2e-2 (W8A16), <= 1e-2 (bf16)."""
import json
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


def _write(path, w, kind):
    if kind == "qint8":
        q, s = orc.quantize_per_row_i8(w)  # the reference's tier quantiser, restated
        with open(path, "wb") as f:
            f.write(s.astype("<f4").tobytes())
            f.write(q.tobytes())
    elif kind == "bf16":
        (w.view(np.uint32) >> 16).astype("<u2").tofile(path)
    else:
        w.astype("<f4").tofile(path)


def _bf16_exact(a):
    """f32 values that survive the bf16 tier unchanged (the reference stores bf16 only when lossless)."""
    return ((a.view(np.uint32) >> 16) << 16).view(np.float32)


@pytest.mark.parametrize("kind", ["qint8", "bf16", "f32"])
def test_tier_directory_to_device_layer(tmp_path, kind):
    from ateniaengine_b200 import MoeExecutionConvention, MoeLayerConfig, tier
    dev = _dev()
    rng = np.random.default_rng(7)
    E, k, d, F, Fs, L = 8, 2, 256, 384, 128, 3
    td = str(tmp_path)
    mk = lambda shape: _bf16_exact(rng.normal(0, 0.02, size=shape).astype(np.float32))
    _write(os.path.join(td, f"L{L}.router.bin"), mk((E, d)), "bf16")
    for e in range(E):
        for role, shape in (("gate", (F, d)), ("up", (F, d)), ("down", (d, F))):
            _write(os.path.join(td, f"L{L}.e{e}.{role}.bin"), mk(shape), kind)
    for role, shape in (("gate", (Fs, d)), ("up", (Fs, d)), ("down", (d, Fs))):
        _write(os.path.join(td, f"L{L}.shared.{role}.bin"), mk(shape), kind)
    _write(os.path.join(td, f"L{L}.shared_gate.bin"), mk((1, d)), "f32")
    json.dump({"version": 5, "model_id": "0" * 16, "family": "qwen_moe", "num_hidden_layers": L + 1, "num_experts": E,
               "experts_per_token": k, "hidden_size": d, "moe_intermediate_size": F, "convention": "hf_qwen",
               "has_shared": True, "attn_has_bias": False, "tensor_count": 0, "total_bytes": 0, "entries": []},
              open(os.path.join(td, "tier_manifest.json"), "w"))
    m = tier.read_manifest(td)
    host = tier.read_layer(td, L, m["num_experts"], m["hidden_size"], m["moe_intermediate_size"], shared_d_ff=Fs,
                           shared_gate=True)
    assert host["kind"] == {"qint8": tier.QINT8, "bf16": tier.BF16, "f32": tier.F32}[kind]
    conv = MoeExecutionConvention.HuggingFaceQwen if m["convention"] == "hf_qwen" else MoeExecutionConvention.Atenia
    layer = tier.to_device_layer(host, MoeLayerConfig(E, k, True, d, F), dev, convention=conv, max_tokens=64)
    x = torch.from_numpy(rng.normal(size=(50, d)).astype(np.float32)).to(dev).to(torch.bfloat16)
    out = layer.forward(x, out_dtype=torch.float32, sync=True).cpu().numpy()
    # the oracle on the very arrays the files hold (int8 codes + scales, bf16 words, or f32)
    ol = orc.OracleLayer(host["router"], host["gate"], host["up"], host["down"], k, False, shared=host["shared"],
                         shared_gate_vec=host["shared_gate"], scales=host["scales"], shared_scales=host["shared_scales"])
    ref = ol.forward(x.float().cpu().numpy())
    assert rel_l2(out, ref) <= (2e-2 if kind == "qint8" else 1e-2)
    if kind == "qint8":
        # nothing was re-encoded on the way: the codes the layer multiplies are the file's bytes
        q_file = np.fromfile(os.path.join(td, f"L{L}.e3.up.bin"), dtype=np.int8, offset=F * 4).reshape(F, d)
        np.testing.assert_array_equal(layer._keep[2][3].cpu().numpy(), q_file)


@pytest.mark.parametrize("name,family,key,conv,renorm", [
    ("mixtral_layer0", "mixtral", "atenia_ref", "Atenia", True),
    ("qwen15_moe_layer0", "qwen", "atenia_hf_ref", "HuggingFaceQwen", False),
    ("qwen2_moe_layer0", "qwen", "atenia_ref", "Atenia", True),
    ("qwen3_moe_layer0", "qwen3", "atenia_ref", "Atenia", True),
    ("deepseek_block", "deepseek", "mlp_output", "Atenia", False)])
@pytest.mark.parametrize("packed", [False, True])
def test_checkpoint_dict_to_device_layer(golden_dir, name, family, key, conv, renorm, packed):
    import ateniaengine_b200 as ae
    from ateniaengine_b200 import binding as b
    dev = _dev()
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    g = {kk: z[kk] for kk in z.files}
    E = g["gate"].shape[0]
    pre = "model.layers.0.block_sparse_moe" if family == "mixtral" else "model.layers.0.mlp"
    names = ("w1", "w3", "w2") if family == "mixtral" else ("gate_proj", "up_proj", "down_proj")
    router_name = f"{pre}.router.weight" if family == "qwen3" else f"{pre}.gate.weight"
    ckpt = {router_name: g["router"], "model.layers.0.self_attn.q_proj.weight": np.zeros((4, 4), np.float32)}
    if packed:
        ckpt[f"{pre}.experts.gate_up_proj"] = np.concatenate([g["gate"], g["up"]], axis=1)
        ckpt[f"{pre}.experts.down_proj"] = g["down"]
    else:
        for e in range(E):
            for role, n in zip(("gate", "up", "down"), names):
                ckpt[f"{pre}.experts.{e}.{n}.weight"] = g[role][e]
    if "shared_gate_proj" in g:
        sh = "shared_experts" if family == "deepseek" else "shared_expert"
        for role in ("gate_proj", "up_proj", "down_proj"):
            ckpt[f"{pre}.{sh}.{role}.weight"] = g["shared_" + role]
        if "shared_gate_vec" in g:
            ckpt[f"{pre}.shared_expert_gate.weight"] = g["shared_gate_vec"][None, :]
    bound = b.bind_layer(ckpt, 0)
    layer = b.to_device_layer(bound, int(g["top_k"]), dev, convention=ae.MoeExecutionConvention[conv],
                              renormalize=renorm, max_tokens=64)
    x = torch.from_numpy(g["input"].astype(np.float32)).to(dev)
    out = layer.forward(x, out_dtype=torch.float32, sync=True).cpu().numpy()
    assert rel_l2(out, g[key]) <= 1e-2
    # the same checkpoint held as INT8 (quantised per row on the GPU, bit-identical to the reference's tier
    # quantiser): against the oracle on the CPU-quantised arrays, W8A16 bar
    l8 = b.to_device_layer(bound, int(g["top_k"]), dev, convention=ae.MoeExecutionConvention[conv],
                           renormalize=renorm, max_tokens=64, int8=True)
    out8 = l8.forward(x, out_dtype=torch.float32, sync=True).cpu().numpy()
    qs = {r: [orc.quantize_per_row_i8(a) for a in bound[r]] for r in ("gate", "up", "down")}
    sh_q = None if bound["shared"] is None else [orc.quantize_per_row_i8(a) for a in bound["shared"]]
    gated = conv == "HuggingFaceQwen" and bound["shared_gate"] is not None
    ol8 = orc.OracleLayer(bound["router"], [q for q, _ in qs["gate"]], [q for q, _ in qs["up"]], [q for q, _ in qs["down"]],
                          int(g["top_k"]), renorm, shared=None if sh_q is None else [q for q, _ in sh_q],
                          shared_gate_vec=bound["shared_gate"] if gated else None, shared_gated=gated,
                          scales={r: [s_ for _, s_ in qs[r]] for r in qs},
                          shared_scales=None if sh_q is None else [s_ for _, s_ in sh_q])
    assert rel_l2(out8, ol8.forward(g["input"].astype(np.float32))) <= 2e-2
