"""Regenerate tests/golden/*.npz from the reference's committed MoE fixtures.

Run once on a machine that has the reference checkout:

    python tests/golden/make_golden.py /path/to/ateniaengine

The reference pins its MoE block with small golden vectors under
`fixtures/moe/` (a `.json` sidecar with the probe input and the expected block
outputs, and a `.safetensors` file with the layer-0 weights).  This script
re-packs each fixture into one `.npz` so the tests need neither the reference
checkout nor the safetensors package.  Nothing is computed here: tensors and
expected outputs are copied bit for bit; the only transformation is slicing the
packed `gate_up_proj [E, 2F, d]` into gate (first half of dim 1) and up (second
half), which is how the reference binds packed experts
(src/moe/binding.rs:381-410).

Fields of each .npz:
  router [E,d], gate [E,F,d], up [E,F,d], down [E,d,F]            f32
  shared_gate_proj [Fs,d], shared_up_proj [Fs,d], shared_down_proj [d,Fs]  (optional)
  shared_gate_vec [d]                                               (optional)
  input [T,d]  (T = 1 for the layer-0 fixtures)
  expected outputs, by the name the reference uses:
    atenia_ref     renormalised top-k, ungated shared   (f64 restatement)
    atenia_hf_ref  non-renormalised top-k, sigmoid-gated shared
    hf_ref         HuggingFace transformers f64 output
    mlp_output     (deepseek_block) non-renormalised top-k, ungated shared
  top_k, norm_topk_prob                                             int
v3_route_ref.npz: router [n,d], router_bias [n], gate/up/down per expert, shared_*, hidden [T,d],
  selected_experts [T,k], dense_combine_weights [T,n], block_out [T,d] and the routing parameters.
"""
import json
import os
import sys

import numpy as np
from safetensors import safe_open


def load_st(path):
    out = {}
    with safe_open(path, "np") as f:
        for k in f.keys():
            out[k] = f.get_tensor(k)
    return out


def pack_layer0(fix_dir, name, out_dir):
    meta = json.load(open(os.path.join(fix_dir, name + ".json")))
    st = load_st(os.path.join(fix_dir, name + ".safetensors"))
    pre = meta.get("tensor_prefix", "model.layers.0.mlp")
    router_key = pre + (".gate.weight" if pre + ".gate.weight" in st else ".router.weight")
    gu = st[pre + ".experts.gate_up_proj"]
    F = gu.shape[1] // 2
    rec = {
        "router": st[router_key].astype(np.float32),
        "gate": np.ascontiguousarray(gu[:, :F, :]).astype(np.float32),
        "up": np.ascontiguousarray(gu[:, F:, :]).astype(np.float32),
        "down": st[pre + ".experts.down_proj"].astype(np.float32),
    }
    for sh in ("shared_expert", "shared_experts"):
        if f"{pre}.{sh}.gate_proj.weight" in st:
            rec["shared_gate_proj"] = st[f"{pre}.{sh}.gate_proj.weight"].astype(np.float32)
            rec["shared_up_proj"] = st[f"{pre}.{sh}.up_proj.weight"].astype(np.float32)
            rec["shared_down_proj"] = st[f"{pre}.{sh}.down_proj.weight"].astype(np.float32)
    if pre + ".shared_expert_gate.weight" in st:
        rec["shared_gate_vec"] = st[pre + ".shared_expert_gate.weight"].reshape(-1).astype(np.float32)
    if "input" in meta:
        rec["input"] = np.asarray(meta["input"], dtype=np.float64)[None, :]
        rec["top_k"] = np.int32(meta["experts_per_token"])
        rec["norm_topk_prob"] = np.int32(bool(meta.get("norm_topk_prob", False)))
        for key in ("atenia_ref", "atenia_hf_ref", "hf_ref"):
            rec[key] = np.asarray(meta[key], dtype=np.float64)[None, :]
    else:  # deepseek_block
        rec["input"] = np.asarray(meta["probe"], dtype=np.float64)[None, :]
        rec["top_k"] = np.int32(meta["num_experts_per_tok"])
        rec["norm_topk_prob"] = np.int32(0)
        rec["mlp_output"] = np.asarray(meta["mlp_output"], dtype=np.float64)[None, :]
    np.savez_compressed(os.path.join(out_dir, name + ".npz"), **rec)
    print(name, {k: getattr(v, "shape", v) for k, v in rec.items()})


def pack_v3_route(fix_dir, out_dir):
    """fixtures/moe/v3_route_ref.*: DeepSeek-V3-like routing on a reduced block, HF transformers f64
    reference (asserted by tests/moe_v3_route_scale_cert_test.rs)."""
    meta = json.load(open(os.path.join(fix_dir, "v3_route_ref.json")))
    st = load_st(os.path.join(fix_dir, "v3_route_ref.safetensors"))
    n = meta["n_routed_experts"]
    rec = {
        "router": st["router.weight"].astype(np.float32), "router_bias": st["router.bias"].astype(np.float32),
        "gate": np.stack([st[f"expert.{e}.w_gate"] for e in range(n)]).astype(np.float32),
        "up": np.stack([st[f"expert.{e}.w_up"] for e in range(n)]).astype(np.float32),
        "down": np.stack([st[f"expert.{e}.w_down"] for e in range(n)]).astype(np.float32),
        "shared_gate_proj": st["shared.w_gate"].astype(np.float32),
        "shared_up_proj": st["shared.w_up"].astype(np.float32),
        "shared_down_proj": st["shared.w_down"].astype(np.float32),
        "hidden": st["hidden"].astype(np.float32),
        "selected_experts": np.asarray(meta["selected_experts"], dtype=np.int32),
        "dense_combine_weights": np.asarray(meta["dense_combine_weights"], dtype=np.float64).reshape(meta["tokens"], n),
        "block_out": np.asarray(meta["block_out"], dtype=np.float64).reshape(meta["tokens"], meta["hidden_size"]),
        "top_k": np.int32(meta["top_k"]), "n_group": np.int32(meta["n_group"]),
        "topk_group": np.int32(meta["topk_group"]),
        "routed_scaling_factor": np.float64(meta["routed_scaling_factor"]),
        "norm_topk_prob": np.int32(bool(meta["norm_topk_prob"])),
    }
    np.savez_compressed(os.path.join(out_dir, "v3_route_ref.npz"), **rec)
    print("v3_route_ref", {k: getattr(v, "shape", v) for k, v in rec.items()})


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/ateniaengine")
    ref = sys.argv[1]
    fix_dir = os.path.join(ref, "fixtures", "moe")
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for name in ("mixtral_layer0", "qwen15_moe_layer0", "qwen2_moe_layer0", "qwen3_moe_layer0",
                 "deepseek_block"):
        pack_layer0(fix_dir, name, out_dir)
    pack_v3_route(fix_dir, out_dir)


if __name__ == "__main__":
    main()
