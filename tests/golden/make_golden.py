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


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/ateniaengine")
    ref = sys.argv[1]
    fix_dir = os.path.join(ref, "fixtures", "moe")
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for name in ("mixtral_layer0", "qwen15_moe_layer0", "qwen2_moe_layer0", "qwen3_moe_layer0",
                 "deepseek_block"):
        pack_layer0(fix_dir, name, out_dir)


if __name__ == "__main__":
    main()
