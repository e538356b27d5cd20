"""The reference's persistent expert tier (directory of `L{l}.*.bin` files + `tier_manifest.json`)
read into the arrays the GPU layer consumes.  File parsing is done by the C library
(`atenia_tier_*`, host code); this module walks the directory layout:

  L{l}.router.bin                      [E, d]      f32 or bf16      src/moe/residency.rs:638, :674
  L{l}.e{i}.{gate,up,down}.bin         [F,d],[F,d],[d,F]  f32 / bf16 / qint8   residency.rs:492-505
  L{l}.shared.{gate,up,down}.bin       shared expert (its own width)            residency.rs:630-634
  L{l}.shared_gate.bin                 [d]                                      residency.rs:639-641
  tier_manifest.json (version 5)       src/moe/runtime.rs:146-206
"""
import ctypes as C
import json
import os

import numpy as np

from . import _lib

F32, BF16, QINT8 = 0, 1, 2
MANIFEST_VERSION = 5


class TierError(RuntimeError):
    def __init__(self, status, path):
        super().__init__(f"tier: {path}: status {status}: "
                         f"{_lib.lib().atenia_moe_status_str(C.c_int(status)).decode()}")
        self.status = status


def _p(a):
    return C.c_void_p(a.ctypes.data)


def detect(path, rows, cols):
    rc = _lib.lib().atenia_tier_detect_dtype(path.encode(), rows, cols)
    if rc < 0:
        raise TierError(rc, path)
    return rc


def read_tensor(path, rows, cols):
    """Returns (kind, array, scales): f32 -> float32 [rows, cols]; bf16 -> uint16 [rows, cols] (the
    stored words); qint8 -> int8 [rows, cols] plus float32 [rows] scales."""
    kind = detect(path, rows, cols)
    L = _lib.lib()
    if kind == QINT8:
        q = np.empty((rows, cols), dtype=np.int8)
        s = np.empty(rows, dtype=np.float32)
        rc = L.atenia_tier_read_qint8(path.encode(), rows, cols, _p(q), _p(s))
        if rc:
            raise TierError(rc, path)
        return kind, q, s
    if kind == BF16:
        w = np.empty((rows, cols), dtype=np.uint16)
        rc = L.atenia_tier_read_bf16(path.encode(), rows, cols, _p(w))
        if rc:
            raise TierError(rc, path)
        return kind, w, None
    out = np.empty((rows, cols), dtype=np.float32)
    rc = L.atenia_tier_read_f32(path.encode(), rows, cols, _p(out))
    if rc:
        raise TierError(rc, path)
    return kind, out, None


def read_f32(path, rows, cols):
    out = np.empty((rows, cols), dtype=np.float32)
    rc = _lib.lib().atenia_tier_read_f32(path.encode(), rows, cols, _p(out))
    if rc:
        raise TierError(rc, path)
    return out


def read_manifest(tier_dir):
    """tier_manifest.json, checked for the version this reader understands."""
    m = json.load(open(os.path.join(tier_dir, "tier_manifest.json")))
    if m.get("version") != MANIFEST_VERSION:
        raise ValueError(f"tier manifest version {m.get('version')} != {MANIFEST_VERSION}")
    return m


def read_layer(tier_dir, layer_id, num_experts, d_model, d_ff, shared_d_ff=0, shared_gate=False):
    """One MoE layer of a tier as host arrays:
    {"router": f32 [E,d], "kind": F32|BF16|QINT8, "gate"/"up"/"down": lists of arrays,
     "scales": {"gate": [...], ...} (qint8), "shared": [g,u,d] or None, "shared_scales", "shared_gate"}.
    All expert files of a layer must share one encoding (the reference writes them that way)."""
    j = lambda name: os.path.join(tier_dir, name)
    out = {"router": read_f32(j(f"L{layer_id}.router.bin"), num_experts, d_model),
           "gate": [], "up": [], "down": [], "scales": {"gate": [], "up": [], "down": []}}
    kinds = set()
    for e in range(num_experts):
        for role, (r, c) in (("gate", (d_ff, d_model)), ("up", (d_ff, d_model)), ("down", (d_model, d_ff))):
            k, a, s = read_tensor(j(f"L{layer_id}.e{e}.{role}.bin"), r, c)
            kinds.add(k)
            out[role].append(a)
            out["scales"][role].append(s)
    out["shared"] = out["shared_scales"] = out["shared_gate"] = None
    if shared_d_ff:
        sh, ss = [], []
        for role, (r, c) in (("gate", (shared_d_ff, d_model)), ("up", (shared_d_ff, d_model)),
                             ("down", (d_model, shared_d_ff))):
            k, a, s = read_tensor(j(f"L{layer_id}.shared.{role}.bin"), r, c)
            kinds.add(k)
            sh.append(a)
            ss.append(s)
        out["shared"], out["shared_scales"] = sh, ss
        if shared_gate:
            out["shared_gate"] = read_f32(j(f"L{layer_id}.shared_gate.bin"), 1, d_model).reshape(-1)
    if len(kinds) != 1:
        raise ValueError(f"layer {layer_id}: mixed tier encodings {sorted(kinds)}")
    out["kind"] = kinds.pop()
    if out["kind"] != QINT8:
        out["scales"] = None
        out["shared_scales"] = None
    return out


def to_device_layer(host, config, device, convention=None, renormalize=None, max_tokens=4096):
    """Upload a layer read by `read_layer` and bind it: int8 codes and scales, or bf16 words, go to
    the GPU as they are; an f32 tier is rounded to bf16."""
    import torch

    from .moe import RealMoeLayer

    def up(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
        if a.dtype == np.uint16:
            return t.view(torch.bfloat16)
        if a.dtype == np.float32:
            return t.to(torch.bfloat16)
        return t

    f32 = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device)
    q = host["kind"] == QINT8
    scales = {k: [f32(s) for s in host["scales"][k]] for k in ("gate", "up", "down")} if q else None
    return RealMoeLayer(config, f32(host["router"]), [up(a) for a in host["gate"]], [up(a) for a in host["up"]],
                        [up(a) for a in host["down"]],
                        shared=None if host["shared"] is None else [up(a) for a in host["shared"]],
                        shared_gate=f32(host["shared_gate"]), scales=scales,
                        shared_scales=[f32(s) for s in host["shared_scales"]] if q and host["shared"] else None,
                        convention=convention, renormalize=renormalize, max_tokens=max_tokens)
