"""Seeded synthetic MoE layers with the shapes and value distributions of the benchmark configs.

No public dataset is involved: weights ~ N(0, 0.02^2), router ~ N(0, 0.02^2), activations ~ N(0, 1),
shared gate vector ~ N(0, 0.02^2); values are drawn in f32 and rounded once to bf16 so that every
consumer sees identical numbers.  Router load skew is an input-side construct (the reference router
has no bias): an additive per-expert logit term, N(0, 0.5^2) ("normal") or the log of a Zipf(1.1)
popularity over a seeded random permutation of the experts ("zipf").
"""
from dataclasses import dataclass, replace

import torch


@dataclass(frozen=True)
class MoeShape:
    name: str
    d_model: int
    d_ff: int
    num_experts: int
    top_k: int
    renormalize: bool
    shared_d_ff: int = 0
    shared_gated: bool = False
    bias: str = "none"  # none | normal | zipf
    int8: bool = False
    tokens: int = 64


SHAPES = {
    # tiny Mixtral-style layer, the reference's own CPU-runnable case
    "tiny": MoeShape("tiny", 512, 1408, 8, 2, True, tokens=64),
    # Mixtral-8x7B: top-2 renormalised, skewed routing
    "mixtral": MoeShape("mixtral", 4096, 14336, 8, 2, True, bias="normal", tokens=4096),
    # Qwen1.5-MoE-A2.7B: 60 experts top-4 raw weights + sigmoid-gated shared expert
    "qwen_moe": MoeShape("qwen_moe", 2048, 1408, 60, 4, False, 5632, True, tokens=2048),
    # DeepSeek-V2-Lite: 64 experts top-6 raw weights + two ungated shared experts fused to 2816
    "deepseek_v2_lite": MoeShape("deepseek_v2_lite", 2048, 1408, 64, 6, False, 2816, False, tokens=8192),
    # Mixtral-8x7B W8A16, Zipf routing, decode batches
    "mixtral_int8": MoeShape("mixtral_int8", 4096, 14336, 8, 2, True, bias="zipf", int8=True, tokens=64),
}


def small(shape, d_model=None, d_ff=None, shared_d_ff=None, tokens=None):
    """Same routing structure at reduced widths (parity cases the CPU oracle finishes quickly)."""
    return replace(shape, d_model=d_model or shape.d_model, d_ff=d_ff or shape.d_ff,
                   shared_d_ff=shape.shared_d_ff if shared_d_ff is None else shared_d_ff,
                   tokens=tokens or shape.tokens)


def _randn(gen, shape, std, device):
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std


def make_weights(shape, seed, device, experts=None):
    """Returns a dict of device tensors.  `experts` = (first, count) restricts the expert matrices to a
    contiguous slice (expert parallelism); the random stream is still consumed for all experts so
    that every rank sees the same layer."""
    from . import moe  # deferred: needs the CUDA library only for int8

    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    E, d, F, Fs = shape.num_experts, shape.d_model, shape.d_ff, shape.shared_d_ff
    first, count = experts if experts is not None else (0, E)
    w = {}
    w["router"] = _randn(gen, (E, d), 0.02, dev).to(torch.bfloat16).float()
    if shape.bias == "normal":
        w["router_bias"] = _randn(gen, (E,), 0.5, dev)
    elif shape.bias == "zipf":
        order = torch.randperm(E, generator=gen, device=dev)
        rank = torch.empty(E, device=dev)
        rank[order] = torch.arange(1, E + 1, device=dev, dtype=torch.float32)
        w["router_bias"] = -1.1 * torch.log(rank)
    else:
        w["router_bias"] = None

    def matrix(rows, cols, keep):
        m = _randn(gen, (rows, cols), 0.02, dev)
        if not keep:
            return None, None
        if shape.int8:
            q, s = moe.quantize_per_row_i8(m)
            return q, s
        return m.to(torch.bfloat16), None

    w["gate"], w["up"], w["down"] = [], [], []
    w["scales"] = {"gate": [], "up": [], "down": []} if shape.int8 else None
    for e in range(E):
        keep = first <= e < first + count
        for name, (r, c) in (("gate", (F, d)), ("up", (F, d)), ("down", (d, F))):
            m, s = matrix(r, c, keep)
            if keep:
                w[name].append(m)
                if shape.int8:
                    w["scales"][name].append(s)
    if Fs > 0:
        sh = [matrix(Fs, d, True), matrix(Fs, d, True), matrix(d, Fs, True)]
        w["shared"] = [m for m, _ in sh]
        w["shared_scales"] = [s for _, s in sh] if shape.int8 else None
        w["shared_gate"] = _randn(gen, (d,), 0.02, dev).to(torch.bfloat16).float() if shape.shared_gated else None
    else:
        w["shared"] = w["shared_scales"] = w["shared_gate"] = None
    return w


def make_activations(shape, seed, device, tokens=None, dtype=torch.bfloat16):
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed) + 7919)
    T = tokens if tokens is not None else shape.tokens
    return torch.randn((T, shape.d_model), generator=gen, device=dev, dtype=torch.float32).to(dtype)


def build_layer(shape, w, max_tokens, ep_rank=0, ep_world=1):
    from .moe import MoeExecutionConvention, MoeLayerConfig, RealMoeLayer

    cfg = MoeLayerConfig(shape.num_experts, shape.top_k, shape.shared_d_ff > 0, shape.d_model, shape.d_ff)
    conv = MoeExecutionConvention.HuggingFaceQwen if shape.shared_gated else MoeExecutionConvention.Atenia
    return RealMoeLayer(cfg, w["router"], w["gate"], w["up"], w["down"], shared=w["shared"],
                        shared_gate=w["shared_gate"], scales=w["scales"], shared_scales=w["shared_scales"],
                        convention=conv, renormalize=shape.renormalize, router_bias=w["router_bias"],
                        max_tokens=max_tokens, ep_rank=ep_rank, ep_world=ep_world)
