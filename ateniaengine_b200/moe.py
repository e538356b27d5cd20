"""Host-side mirror of the reference's MoE block operator, on top of the C ABI.

Names and argument meaning follow the reference (paths relative to its project root):
  MoeLayerConfig, MoeExecutionConvention, RealMoeLayer        src/moe/layer.rs:37-43, :185-212
  RealMoeLayer.forward / forward_with / forward_auto          src/moe/layer.rs:374-431
  register_real_moe_layer / execute_real_moe_layer            src/moe/graph_op.rs:228, :327
  quantize_per_row_i8                                         src/tensor/disk_tier.rs:231-245
  quantize_per_group_i8 (absmax_per_{channel,group}_symmetric) src/tensor/quantizer.rs:67-118, 176-246
  int8_to_bf16_per_group                                      src/cuda/int8_to_bf16.cu:24-40, 99-117
Every computation runs in the CUDA library; torch only owns device memory and streams.
"""
import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import IO_BF16, IO_F32, W_BF16, W_INT8_ROW


class MoeLayerError(RuntimeError):
    """Mirrors MoeLayerError: `kind` is 'LayerNotFound', 'DimMismatch' or 'Status'."""

    def __init__(self, kind, status, msg):
        super().__init__(f"moe-layer: {kind}: {msg}")
        self.kind = kind
        self.status = status


class MoeExecutionConvention(enum.Enum):
    Atenia = 0           # renormalised top-k, ungated shared expert
    HuggingFaceQwen = 1  # raw top-k weights, shared expert scaled by sigmoid(gate . x)


@dataclass
class MoeLayerConfig:
    num_experts: int
    experts_per_token: int
    has_shared_expert: bool
    d_model: int
    d_ff: int

    def validate(self):
        if self.num_experts < 1 or self.experts_per_token < 1 or self.experts_per_token > self.num_experts:
            raise ValueError("moe-layer: invalid expert counts")
        if self.d_model < 1 or self.d_ff < 1:
            raise ValueError("moe-layer: invalid dims")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _io_dtype(t):
    if t.dtype == torch.bfloat16:
        return IO_BF16
    if t.dtype == torch.float32:
        return IO_F32
    raise TypeError(f"activations must be bf16 or f32, got {t.dtype}")


def quantize_per_row_i8(w):
    """Per-row symmetric int8 of a CUDA f32 [rows, cols] tensor -> (q int8, scales f32)."""
    assert w.is_cuda and w.dtype == torch.float32 and w.dim() == 2
    w = w.contiguous()
    q = torch.empty(w.shape, dtype=torch.int8, device=w.device)
    s = torch.empty(w.shape[0], dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib().atenia_quantize_per_row_i8(_ptr(w), w.shape[0], w.shape[1], _ptr(q), _ptr(s),
                                                         C.c_void_p(st)), "quantize_per_row_i8")
    return q, s


def quantize_per_group_i8(w, group_size=0):
    """Dense W8A16 quantiser of a CUDA f32 [K, N] weight: one scale per (group of `group_size` rows,
    column); group_size 0 = per output channel.  Mirrors absmax_per_channel_symmetric /
    absmax_per_group_symmetric (src/tensor/quantizer.rs:67-118, :176-246) -> (q int8 [K, N],
    scales f32 [groups, N])."""
    assert w.is_cuda and w.dtype == torch.float32 and w.dim() == 2 and group_size >= 0
    w = w.contiguous()
    K, N = w.shape
    g = K if group_size == 0 or group_size > K else group_size
    groups = (K + g - 1) // g if K else 0
    q = torch.empty((K, N), dtype=torch.int8, device=w.device)
    s = torch.empty((groups, N), dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib().atenia_quantize_per_group_i8(_ptr(w), K, N, group_size, _ptr(q), _ptr(s), C.c_void_p(st)),
                   "quantize_per_group_i8")
    return q, s


def int8_to_bf16_per_group(q, scales, group_size=0):
    """The reference's truncating dequant of the dense W8A16 layout (src/cuda/int8_to_bf16.cu:24-40,
    :99-117) -> bf16 [K, N]."""
    assert q.is_cuda and q.dtype == torch.int8 and q.dim() == 2 and scales.dtype == torch.float32
    q, scales = q.contiguous(), scales.contiguous()
    K, N = q.shape
    out = torch.empty((K, N), dtype=torch.bfloat16, device=q.device)
    with torch.cuda.device(q.device):
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib().atenia_int8_to_bf16_per_group(_ptr(q), _ptr(scales), K, N, group_size, _ptr(out),
                                                            C.c_void_p(st)), "int8_to_bf16_per_group")
    return out


class RealMoeLayer:
    """A runnable MoE layer whose weights live in device memory.

    `gate`, `up` are lists of [F, d] tensors, `down` a list of [d, F] tensors (bf16, or int8 with
    `scales = {"gate": [...], "up": [...], "down": [...]}` of f32 [rows] tensors).  `router` is
    f32 [E, d].  `shared` is an optional (gate [Fs, d], up [Fs, d], down [d, Fs]) triple with
    `shared_scales` for int8; `shared_gate` the optional f32 [d] sigmoid-gate vector.
    `convention` None means "auto": HuggingFaceQwen when a shared gate is present, else Atenia
    (RealMoeLayer::resolve_convention); pass `renormalize` to override only the top-k rule (the
    DeepSeek runtime does this from norm_topk_prob).
    Under expert parallelism (`ep_world > 1`) the lists hold this rank's experts only.
    `v3 = {"n_group", "topk_group", "scaling", "e_score_bias" (f32 [E] tensor or None)}` selects
    DeepSeek-V3 routing (src/moe/v3_router.rs); `renormalize` then means norm_topk_prob.
    """

    def __init__(self, config, router, gate, up, down, shared=None, shared_gate=None, scales=None,
                 shared_scales=None, convention=None, renormalize=None, router_bias=None, max_tokens=4096,
                 ep_rank=0, ep_world=1, v3=None):
        config.validate()
        self.config = config
        dev = router.device
        assert dev.type == "cuda", "weights must be CUDA tensors"
        self.device = dev
        if convention is None:
            convention = (MoeExecutionConvention.HuggingFaceQwen if shared_gate is not None
                          else MoeExecutionConvention.Atenia)
        self.convention = convention
        if renormalize is None:
            renormalize = convention == MoeExecutionConvention.Atenia
        gated = convention == MoeExecutionConvention.HuggingFaceQwen and shared_gate is not None
        int8 = gate[0].dtype == torch.int8
        self._keep = [router, gate, up, down, shared, shared_gate, scales, shared_scales, router_bias, v3]
        Fs = shared[0].shape[0] if shared is not None else 0
        cfg = _lib.MoeConfig(config.num_experts, config.experts_per_token, config.d_model, config.d_ff, Fs,
                             int(renormalize), int(gated), W_INT8_ROW if int8 else W_BF16, int(max_tokens),
                             ep_rank, ep_world)
        if v3 is not None:
            cfg.router_mode = 1
            cfg.n_group = int(v3["n_group"])
            cfg.topk_group = int(v3["topk_group"])
            cfg.routed_scaling_factor = float(v3["scaling"])
        self.max_tokens = int(max_tokens)
        self.ep_world = ep_world
        self._h = C.c_void_p()
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().atenia_moe_create(C.byref(cfg), C.byref(self._h)), "atenia_moe_create")
            n = len(gate)
            assert n == config.num_experts // ep_world
            arr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() for t in ts])
            w = _lib.MoeWeights()
            router = router.contiguous()
            assert router.dtype == torch.float32
            w.w_router = router.data_ptr()
            w.router_bias = None if router_bias is None else router_bias.data_ptr()
            self._arrs = [arr(gate), arr(up), arr(down)]
            w.w_gate, w.w_up, w.w_down = self._arrs
            if int8:
                self._sarrs = [arr(scales["gate"]), arr(scales["up"]), arr(scales["down"])]
                w.s_gate, w.s_up, w.s_down = self._sarrs
            if shared is not None:
                w.shared_w_gate, w.shared_w_up, w.shared_w_down = [t.data_ptr() for t in shared]
                if int8:
                    w.shared_s_gate, w.shared_s_up, w.shared_s_down = [t.data_ptr() for t in shared_scales]
                if shared_gate is not None:
                    w.shared_gate_vec = shared_gate.data_ptr()
            if v3 is not None and v3.get("e_score_bias") is not None:
                w.e_score_bias = v3["e_score_bias"].data_ptr()
            _lib.check(_lib.lib().atenia_moe_set_weights(self._h, C.byref(w)), "atenia_moe_set_weights")

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().atenia_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def ep_init(self, unique_id: bytes):
        buf = C.create_string_buffer(unique_id, len(unique_id))
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().atenia_moe_ep_init(self._h, buf), "atenia_moe_ep_init")

    def ep_attach(self, owner):
        """Share the NCCL communicator `owner` joined with ep_init (one communicator per model, not per layer)."""
        _lib.check(_lib.lib().atenia_moe_ep_attach(self._h, owner._h), "atenia_moe_ep_attach")

    def ep_ipc_export(self) -> bytes:
        """Handles to this rank's receive and result buffers, for the direct (peer-store) exchange."""
        nb = _lib.lib().atenia_moe_ep_ipc_bytes()
        buf = C.create_string_buffer(nb)
        _lib.check(_lib.lib().atenia_moe_ep_ipc_export(self._h, buf), "atenia_moe_ep_ipc_export")
        return bytes(buf.raw)

    def ep_ipc_import(self, blobs_of_all_ranks: bytes):
        """Map the buffers of all ranks (blobs concatenated in rank order) and switch the layer's
        forward to the direct exchange."""
        buf = C.create_string_buffer(blobs_of_all_ranks, len(blobs_of_all_ranks))
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().atenia_moe_ep_ipc_import(self._h, buf), "atenia_moe_ep_ipc_import")

    def ep_replicated_tokens(self, enable=True):
        """Expert parallelism over a batch that every rank holds (decode): no token exchange, one
        all-reduce of the expert outputs, capturable in a CUDA graph."""
        _lib.check(_lib.lib().atenia_moe_ep_set_token_layout(self._h, 1 if enable else 0), "atenia_moe_ep_set_token_layout")

    def forward(self, x, out=None, out_dtype=None, aux=False, sync=False):
        """x: [T, d] CUDA bf16 or f32.  Returns out (and a dict of routing tensors when aux)."""
        assert x.is_cuda and x.dim() == 2 and x.shape[1] == self.config.d_model
        x = x.contiguous()
        T = x.shape[0]
        if out is None:
            out = torch.empty((T, self.config.d_model), dtype=out_dtype or x.dtype, device=x.device)
        auxs = None
        aux_t = None
        if aux:
            k, E = self.config.experts_per_token, self.config.num_experts
            aux_t = {
                "topk_idx": torch.empty((T, k), dtype=torch.int32, device=x.device),
                "topk_w": torch.empty((T, k), dtype=torch.float32, device=x.device),
                "logits": torch.empty((T, E), dtype=torch.float32, device=x.device),
                "perm": torch.empty((T * k,), dtype=torch.int32, device=x.device),
                "expert_offsets": torch.empty((E + 1,), dtype=torch.int32, device=x.device),
            }
            auxs = _lib.MoeAux(*[aux_t[n].data_ptr() for n in ("topk_idx", "topk_w", "logits", "perm",
                                                               "expert_offsets")])
        with torch.cuda.device(x.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            fn = _lib.lib().atenia_moe_forward_sync if sync else _lib.lib().atenia_moe_forward
            _lib.check(fn(self._h, _ptr(x), _io_dtype(x), T, _ptr(out), _io_dtype(out),
                          C.byref(auxs) if auxs is not None else None, st), "atenia_moe_forward")
        return (out, aux_t) if aux else out

    def forward_with(self, x, convention, out=None, out_dtype=None, sync=False):
        """RealMoeLayer::forward_with: the block under an explicit MoeExecutionConvention for this call
        (Atenia: renormalised weights, ungated shared expert; HuggingFaceQwen: raw weights, shared
        expert scaled by sigmoid(gate . x) when the layer was given a gate vector)."""
        assert x.is_cuda and x.dim() == 2 and x.shape[1] == self.config.d_model
        x = x.contiguous()
        T = x.shape[0]
        if out is None:
            out = torch.empty((T, self.config.d_model), dtype=out_dtype or x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().atenia_moe_forward_with(self._h, _ptr(x), _io_dtype(x), T, _ptr(out), _io_dtype(out),
                                                          None, st, int(convention.value)), "atenia_moe_forward_with")
            if sync:
                _lib.check(_lib.lib().atenia_moe_check(self._h, st), "atenia_moe_forward_with")
        return out

    def block_forward(self, x, gamma=None, eps=1e-5, out=None, sync=False):
        """The decoder-layer step around the block: x + MoE(rms_norm(x, eps) * gamma)
        (src/moe/full_forward.rs:239-252).  x: CUDA f32 [T, d]; gamma: CUDA f32 [d] or None."""
        assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[1] == self.config.d_model
        x = x.contiguous()
        if gamma is not None:
            assert gamma.is_cuda and gamma.dtype == torch.float32 and gamma.numel() == self.config.d_model
            gamma = gamma.contiguous()
        if out is None:
            out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().atenia_moe_block_forward(self._h, _ptr(x), _ptr(gamma), float(eps), x.shape[0],
                                                           _ptr(out), st), "atenia_moe_block_forward")
            if sync:
                _lib.check(_lib.lib().atenia_moe_check(self._h, st), "atenia_moe_block_forward")
        return out

    def forward_auto(self, x, **kw):
        """RealMoeLayer::forward_auto: HuggingFaceQwen when a shared gate vector is present, else Atenia
        (resolve_convention); the convention the constructor resolved when none was given."""
        return self.forward(x, **kw)

    def forward_selected(self, x, topk_idx, topk_w, out_dtype=None, sync=True):
        """The block with a caller-supplied selection (the graph primitives MoeDynamicDispatch /
        MoeSparseCombine in batched form): topk_idx [T, k] int32, topk_w [T, k] f32."""
        x = x.contiguous()
        T = x.shape[0]
        out = torch.empty((T, self.config.d_model), dtype=out_dtype or x.dtype, device=x.device)
        topk_idx = topk_idx.contiguous()
        topk_w = topk_w.contiguous()
        assert topk_idx.dtype == torch.int32 and topk_w.dtype == torch.float32
        with torch.cuda.device(x.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().atenia_moe_forward_selected(self._h, _ptr(x), _io_dtype(x), T, _ptr(topk_idx),
                                                              _ptr(topk_w), _ptr(out), _io_dtype(out), st),
                       "atenia_moe_forward_selected")
            if sync:
                _lib.check(_lib.lib().atenia_moe_check(self._h, st), "atenia_moe_forward_selected")
        return out

    def check(self):
        with torch.cuda.device(self.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().atenia_moe_check(self._h, st), "atenia_moe_check")

    def route_from_logits(self, logits, want_perm=True):
        assert logits.is_cuda and logits.dtype == torch.float32
        logits = logits.contiguous()
        T, E = logits.shape
        k = self.config.experts_per_token
        idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        perm = torch.empty((T * k,), dtype=torch.int32, device=logits.device) if want_perm else None
        inv = torch.empty((T * k,), dtype=torch.int32, device=logits.device) if want_perm else None
        off = torch.empty((E + 1,), dtype=torch.int32, device=logits.device) if want_perm else None
        with torch.cuda.device(logits.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().atenia_moe_route_from_logits(self._h, _ptr(logits), T, _ptr(idx), _ptr(w),
                                                               _ptr(perm), _ptr(inv), _ptr(off), st),
                       "atenia_moe_route_from_logits")
            _lib.check(_lib.lib().atenia_moe_check(self._h, st), "atenia_moe_route_from_logits")
        return idx, w, perm, inv, off

    def enable_timing(self, on=True):
        _lib.lib().atenia_moe_enable_timing(self._h, int(on))

    def last_gemm_ms(self, which):
        return float(_lib.lib().atenia_moe_last_gemm_ms(self._h, which))

    def last_phase_ms(self, which):
        """0 route+permute+gather, 1 rows out (EP), 2 routed GEMMs, 3 rows back (EP), 4 shared+combine, 5 all."""
        return float(_lib.lib().atenia_moe_last_phase_ms(self._h, which))

    def last_recv_rows(self):
        return int(_lib.lib().atenia_moe_last_recv_rows(self._h))


# ---- operator registry (host buffers) ---------------------------------------------------------

def register_real_moe_layer(config, router, gate, up, down, shared=None, shared_gate=None,
                            convention=None, renormalize=None, int8=False, max_tokens=4096):
    """Host numpy f32 weights -> layer id.  Mirrors register_real_moe_layer(RealMoeLayer)."""
    config.validate()
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
    router = f32(router)
    gate, up, down = [f32(a) for a in gate], [f32(a) for a in up], [f32(a) for a in down]
    if convention is None:
        convention = (MoeExecutionConvention.HuggingFaceQwen if shared_gate is not None
                      else MoeExecutionConvention.Atenia)
    if renormalize is None:
        renormalize = convention == MoeExecutionConvention.Atenia
    gated = convention == MoeExecutionConvention.HuggingFaceQwen and shared_gate is not None
    n = config.num_experts
    arr = lambda ts: (C.c_void_p * n)(*[t.ctypes.data for t in ts])
    h = _lib.HostMoeLayer()
    Fs = 0
    keep = [router, gate, up, down]
    if shared is not None:
        shared = [f32(a) for a in shared]
        Fs = shared[0].shape[0]
        h.shared_w_gate, h.shared_w_up, h.shared_w_down = [a.ctypes.data for a in shared]
        keep.append(shared)
        if shared_gate is not None:
            shared_gate = f32(shared_gate).reshape(-1)
            h.shared_gate_vec = shared_gate.ctypes.data
            keep.append(shared_gate)
    h.config = _lib.MoeConfig(config.num_experts, config.experts_per_token, config.d_model, config.d_ff, Fs,
                              int(renormalize), int(gated), W_INT8_ROW if int8 else W_BF16, int(max_tokens), 0, 1)
    h.w_router = router.ctypes.data
    a1, a2, a3 = arr(gate), arr(up), arr(down)
    h.w_gate, h.w_up, h.w_down = a1, a2, a3
    lid = _lib.lib().atenia_register_real_moe_layer(C.byref(h))
    if lid < 0:
        raise MoeLayerError("Status", int(lid), _lib.lib().atenia_moe_status_str(C.c_int(int(lid))).decode())
    return int(lid)


def register_resident_moe_layer(layer):
    """Enter a device-resident RealMoeLayer into the registry (register_resident_moe_layer).  The
    registry borrows the layer; keep the Python object alive while the id is used."""
    lid = _lib.lib().atenia_register_resident_moe_layer(layer.handle)
    if lid < 0:
        raise MoeLayerError("Status", int(lid), _lib.lib().atenia_moe_status_str(C.c_int(int(lid))).decode())
    return int(lid)


def execute_real_moe_layer(layer_id, input, out=None, convention=None):
    """Flat host f32 [n * d_model] -> [n * d_model], the graph op's contract.  `convention` (a
    MoeExecutionConvention) makes it execute_real_moe_layer_with."""
    inp = np.ascontiguousarray(input, dtype=np.float32).reshape(-1)
    if out is None:
        out = np.empty_like(inp)
    if convention is None:
        rc = _lib.lib().atenia_execute_real_moe_layer(int(layer_id), C.c_void_p(inp.ctypes.data), inp.size,
                                                      C.c_void_p(out.ctypes.data))
    else:
        rc = _lib.lib().atenia_execute_real_moe_layer_with(int(layer_id), C.c_void_p(inp.ctypes.data), inp.size,
                                                           C.c_void_p(out.ctypes.data), int(convention.value))
    if rc == _lib.ERR_POLICY:
        raise MoeLayerError("NumericPolicy", rc, "the selected numeric policy keeps the block on the CPU arms")
    if rc == _lib.ERR_LAYER_NOT_FOUND:
        raise MoeLayerError("LayerNotFound", rc, f"layer_id {layer_id}")
    if rc == _lib.ERR_DIM_MISMATCH:
        raise MoeLayerError("DimMismatch", rc, f"input length {inp.size}")
    if rc != 0:
        raise MoeLayerError("Status", rc, _lib.lib().atenia_moe_status_str(C.c_int(rc)).decode())
    return out


def execute_real_moe_layer_with(layer_id, input, convention, out=None):
    """execute_real_moe_layer_with (src/moe/graph_op.rs:352-364)."""
    return execute_real_moe_layer(layer_id, input, out=out, convention=convention)


class NumericPolicy(enum.Enum):
    """NumericPolicy (src/moe/numeric_policy.rs:37-47).  The library is the Fast arm."""
    Certified = 0
    Strict = 1
    Fast = 2

    def as_str(self):
        return _lib.lib().atenia_numeric_policy_str(self.value).decode()

    @staticmethod
    def from_str(name):
        v = _lib.lib().atenia_numeric_policy_from_str(name.encode())
        return None if v < 0 else NumericPolicy(v)

    def ffn_uses_f32(self):
        return bool(_lib.lib().atenia_numeric_policy_ffn_uses_f32(self.value))

    def ffn_uses_cuda(self):
        return bool(_lib.lib().atenia_numeric_policy_ffn_uses_cuda(self.value))


def numeric_policy():
    return NumericPolicy(_lib.lib().atenia_numeric_policy())


def set_numeric_policy(p):
    _lib.check(_lib.lib().atenia_set_numeric_policy(p.value), "set_numeric_policy")


def clear_numeric_policy_override():
    _lib.lib().atenia_clear_numeric_policy_override()


def auto_expert_cache_capacity(ram_budget_bytes, n_layers, per_expert_bytes, num_experts):
    """auto_expert_cache_capacity (src/moe/residency.rs:201-211)."""
    return int(_lib.lib().atenia_auto_expert_cache_capacity(int(ram_budget_bytes), int(n_layers),
                                                            int(per_expert_bytes), int(num_experts)))


def _plan_config(config, shared_d_ff, int8, max_tokens, ep_world=1):
    return _lib.MoeConfig(config.num_experts, config.experts_per_token, config.d_model, config.d_ff, int(shared_d_ff),
                          1, 0, W_INT8_ROW if int8 else W_BF16, int(max_tokens), 0, int(ep_world))


def plan_residency(config, n_layers, hbm_budget_bytes, shared_d_ff=0, int8=False, max_tokens=4096):
    """Smallest expert-parallel world (1, 2, 4, 8) in which `n_layers` layers of `config` are resident
    within `hbm_budget_bytes` per GPU.  Returns (status, plan dict); status -3 (capacity) when even
    8 ranks do not hold the model."""
    cfg = _plan_config(config, shared_d_ff, int8, max_tokens)
    plan = _lib.ResidencyPlan()
    rc = _lib.lib().atenia_moe_plan_residency(C.byref(cfg), int(n_layers), int(hbm_budget_bytes), C.byref(plan))
    return rc, {n: getattr(plan, n) for n, _ in _lib.ResidencyPlan._fields_ if n != "reserved"}


def workspace_bytes(config, shared_d_ff=0, int8=False, max_tokens=4096, ep_world=1):
    """Device bytes a RealMoeLayer of this configuration allocates besides its weights."""
    cfg = _plan_config(config, shared_d_ff, int8, max_tokens, ep_world)
    return int(_lib.lib().atenia_moe_workspace_bytes(C.byref(cfg)))


def plan_exec_pieces(config, n_tokens, shared_d_ff=0, int8=False, max_tokens=4096, measured=None):
    """Sub-batch sizes execute_real_moe_layer uses for a batch of `n_tokens` (their sum is n_tokens;
    one piece: the batch runs whole, without copy / compute overlap).  `measured` =
    (forward_base_ms, forward_token_ms, copy_token_ms) plans from timings instead of the model."""
    cfg = _plan_config(config, shared_d_ff, int8, max_tokens)
    buf = (C.c_uint64 * 64)()
    a, b, c = measured if measured is not None else (0.0, 0.0, 0.0)
    n = _lib.lib().atenia_moe_plan_exec_pieces_measured(C.byref(cfg), int(n_tokens), float(a), float(b), float(c),
                                                        buf, 64)
    if n < 0:
        raise _lib.AteniaError(n, "atenia_moe_plan_exec_pieces_measured")
    return [int(buf[i]) for i in range(n)]


def execute_real_moe_layer_ptr(layer_id, in_ptr, n_floats, out_ptr):
    """Same call on raw host pointers (e.g. pinned buffers); returns the status."""
    return _lib.lib().atenia_execute_real_moe_layer(int(layer_id), C.c_void_p(in_ptr), n_floats,
                                                    C.c_void_p(out_ptr))


def dispatch_noalloc(topk_idx, num_experts, perm, inv_perm, expert_offsets):
    """Dispatch order of a routed batch through the entry point that allocates nothing.

    For hosts that cannot allocate device memory (everything already sits in the host runtime's
    pool, or an allocation's synchronisation is not acceptable) and so cannot hold a RealMoeLayer.
    All five tensors are the caller's: topk_idx [T, k] int32 in, perm / inv_perm [T*k] and
    expert_offsets [E+1] int32 out.  Limits: T*k <= 65536 and E <= 128.  Returns the status code.
    """
    T, k = topk_idx.shape
    with torch.cuda.device(topk_idx.device):
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        return _lib.lib().atenia_moe_dispatch_noalloc(_ptr(topk_idx), T, k, int(num_experts), _ptr(perm),
                                                      _ptr(inv_perm), _ptr(expert_offsets), st)


class RealMoeStack:
    """A sequence of RealMoeLayer applied one after the other (RealMoeStack, src/moe/stack.rs).

    `residual=True` (or 1) computes x <- x + layer(x) per layer; `residual=2` computes the pre-norm
    block x <- x + layer(rmsnorm(x)) (unit gain, eps 1e-5); both need f32 input.  The layers are
    borrowed: keep them alive.  Call on a non-default CUDA stream to get CUDA-graph replay.
    """

    def __init__(self, layers, residual=False):
        assert len(layers) >= 1
        self.layers = list(layers)
        self.device = layers[0].device
        self.d_model = layers[0].config.d_model
        arr = (C.c_void_p * len(layers))(*[l.handle.value for l in layers])
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().atenia_moe_stack_create(arr, len(layers), int(residual), C.byref(self._h)),
                       "atenia_moe_stack_create")

    def forward(self, x, out=None, out_dtype=None, sync=False):
        assert x.is_cuda and x.dim() == 2 and x.shape[1] == self.d_model
        x = x.contiguous()
        if out is None:
            out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().atenia_moe_stack_forward(self._h, _ptr(x), _io_dtype(x), x.shape[0], _ptr(out),
                                                           _io_dtype(out), st), "atenia_moe_stack_forward")
            if sync:
                _lib.check(_lib.lib().atenia_moe_stack_check(self._h, st), "atenia_moe_stack_check")
        return out

    def set_norm(self, gammas=None, eps=1e-5):
        """Gains (one CUDA f32 [d] tensor per layer, or None for unit gain) and epsilon of the pre-norm of
        a residual=2 stack."""
        arr = None
        if gammas is not None:
            assert len(gammas) == len(self.layers)
            self._gammas = [None if g is None else g.contiguous() for g in gammas]
            arr = (C.c_void_p * len(gammas))(*[None if g is None else g.data_ptr() for g in self._gammas])
        _lib.check(_lib.lib().atenia_moe_stack_set_norm(self._h, arr, float(eps)), "atenia_moe_stack_set_norm")

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().atenia_moe_stack_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
