"""Every struct that crosses the C ABI has the same size and field offsets in the public header (as
gcc lays it out) and in the ctypes mirror the tests and the bench call through."""
import ctypes as C
import os
import subprocess
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

STRUCTS = {
    "AteniaMoeConfig": ("MoeConfig", ["num_experts", "experts_per_token", "d_model", "d_ff", "shared_d_ff", "renormalize",
                                      "shared_gated", "weight_dtype", "max_tokens", "ep_rank", "ep_world", "router_mode",
                                      "n_group", "topk_group", "routed_scaling_factor"]),
    "AteniaMoeWeights": ("MoeWeights", ["w_router", "router_bias", "w_gate", "w_up", "w_down", "s_gate", "s_up", "s_down",
                                        "shared_w_gate", "shared_w_up", "shared_w_down", "shared_s_gate", "shared_s_up",
                                        "shared_s_down", "shared_gate_vec", "e_score_bias"]),
    "AteniaMoeAux": ("MoeAux", ["topk_idx", "topk_w", "logits", "perm", "expert_offsets"]),
    "AteniaHostMoeLayer": ("HostMoeLayer", ["config", "w_router", "w_gate", "w_up", "w_down", "shared_w_gate",
                                            "shared_w_up", "shared_w_down", "shared_gate_vec", "e_score_bias"]),
}


def test_ctypes_mirror_matches_the_header(tmp_path):
    from ateniaengine_b200 import _lib
    lines = []
    for cname, (_, fields) in STRUCTS.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for f in fields:
            lines.append(f'printf("{cname}.{f} %zu\\n", offsetof({cname}, {f}));')
    src = tmp_path / "layout.c"
    src.write_text("#include <stddef.h>\n#include <stdio.h>\n#include \"atenia_moe.h\"\nint main(void) {\n"
                   + "\n".join(lines) + "\nreturn 0;\n}\n")
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = dict(l.split() for l in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.splitlines())
    for cname, (pyname, fields) in STRUCTS.items():
        cls = getattr(_lib, pyname)
        assert int(got[cname]) == C.sizeof(cls), cname
        assert [n for n, _ in cls._fields_] == fields, f"{pyname} lists other fields than the header"
        for f in fields:
            assert int(got[f"{cname}.{f}"]) == getattr(cls, f).offset, f"{cname}.{f}"
