"""ctypes binding of the CPU oracle (oracle/moe_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the product package never does.  The oracle restates the reference's CPU
MoE block; this wrapper passes numpy arrays to it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmoe_oracle.so")

W_F32, W_BF16, W_INT8_ROW = 0, 1, 2
ACC_F64, ACC_F32 = 0, 1


class _Mat(C.Structure):
    _fields_ = [("data", C.c_void_p), ("scales", C.c_void_p)]


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "num_experts", "top_k", "d_model", "d_ff", "shared_d_ff", "renormalize", "shared_gated",
        "weight_kind", "accum", "router_mode", "n_group", "topk_group")] + [("scaling", C.c_double)]


class _Weights(C.Structure):
    _fields_ = [
        ("w_router", C.c_void_p), ("router_bias", C.c_void_p),
        ("gate", C.POINTER(_Mat)), ("up", C.POINTER(_Mat)), ("down", C.POINTER(_Mat)),
        ("shared_gate_proj", _Mat), ("shared_up_proj", _Mat), ("shared_down_proj", _Mat),
        ("shared_gate", C.c_void_p), ("e_score_bias", C.c_void_p),
    ]


def build(force=False):
    """Compile the oracle with the Makefile next to it (gcc only)."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "moe_oracle.c"))):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libmoe_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_moe_forward.restype = C.c_int
        _lib.oracle_top_k.restype = C.c_int
        _lib.oracle_route_from_logits.restype = C.c_int
        _lib.oracle_combine_selected.restype = C.c_int
        _lib.oracle_max_threads.restype = C.c_int
    return _lib


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _kind_of(arr):
    if arr.dtype == np.float32:
        return W_F32
    if arr.dtype == np.uint16:
        return W_BF16
    if arr.dtype == np.int8:
        return W_INT8_ROW
    raise TypeError(f"unsupported weight dtype {arr.dtype}")


class OracleLayer:
    """Weights of one MoE block held as numpy arrays.

    Expert matrices may be f32, bf16 stored as uint16 (decoded as bits << 16), or int8 with one f32
    scale per row; all experts of a layer share one kind.  gate/up are [E, F, d], down is [E, d, F]
    (or lists of per-expert 2-D arrays).  The router is always f32 [E, d].
    """

    def __init__(self, router, gate, up, down, top_k, renormalize, shared=None, shared_gate_vec=None,
                 shared_gated=None, router_bias=None, scales=None, shared_scales=None, v3=None):
        self.router = np.ascontiguousarray(router, dtype=np.float32)
        self.E, self.d = self.router.shape
        self.gate = [np.ascontiguousarray(g) for g in gate]
        self.up = [np.ascontiguousarray(g) for g in up]
        self.down = [np.ascontiguousarray(g) for g in down]
        self.F = self.gate[0].shape[0]
        self.kind = _kind_of(self.gate[0])
        self.top_k = int(top_k)
        self.renormalize = bool(renormalize)
        self.shared = None if shared is None else [np.ascontiguousarray(s) for s in shared]
        self.Fs = 0 if self.shared is None else self.shared[0].shape[0]
        self.shared_gate_vec = None if shared_gate_vec is None else np.ascontiguousarray(
            shared_gate_vec, dtype=np.float32).reshape(-1)
        self.shared_gated = (self.shared_gate_vec is not None) if shared_gated is None else bool(shared_gated)
        self.router_bias = None if router_bias is None else np.ascontiguousarray(router_bias, dtype=np.float32)
        # v3: {"n_group", "topk_group", "scaling", "e_score_bias"} selects DeepSeek-V3 routing
        self.v3 = v3
        self.e_score_bias = None
        if v3 is not None and v3.get("e_score_bias") is not None:
            self.e_score_bias = np.ascontiguousarray(v3["e_score_bias"], dtype=np.float32)
        # scales: dict with "gate","up","down" lists of per-expert f32 [rows]
        self.scales = scales
        self.shared_scales = shared_scales
        if self.kind == W_INT8_ROW:
            assert scales is not None
            for key in ("gate", "up", "down"):
                self.scales[key] = [np.ascontiguousarray(s, dtype=np.float32) for s in self.scales[key]]
            if self.shared is not None:
                self.shared_scales = [np.ascontiguousarray(s, dtype=np.float32) for s in shared_scales]

    def _mats(self, arrs, scl):
        m = (_Mat * len(arrs))()
        for i, a in enumerate(arrs):
            m[i].data = a.ctypes.data
            m[i].scales = scl[i].ctypes.data if scl is not None else None
        return m

    def forward(self, x, accum=ACC_F64, nthreads=0, want_aux=False):
        """x: [T, d] f32.  Returns out [T, d] f32 (and aux dict when want_aux)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        T = x.shape[0]
        assert x.shape[1] == self.d
        cfg = _Config(self.E, self.top_k, self.d, self.F, self.Fs, int(self.renormalize),
                      int(self.shared_gated), self.kind, accum)
        if self.v3 is not None:
            cfg.router_mode = 1
            cfg.n_group = int(self.v3["n_group"])
            cfg.topk_group = int(self.v3["topk_group"])
            cfg.scaling = float(self.v3["scaling"])
        sc = self.scales if self.kind == W_INT8_ROW else None
        g = self._mats(self.gate, sc["gate"] if sc else None)
        u = self._mats(self.up, sc["up"] if sc else None)
        dn = self._mats(self.down, sc["down"] if sc else None)
        w = _Weights()
        w.w_router = self.router.ctypes.data
        w.router_bias = None if self.router_bias is None else self.router_bias.ctypes.data
        w.gate, w.up, w.down = g, u, dn
        if self.shared is not None:
            ss = self.shared_scales if self.kind == W_INT8_ROW else [None] * 3
            for name, a, s in zip(("shared_gate_proj", "shared_up_proj", "shared_down_proj"),
                                  self.shared, ss):
                mm = _Mat(a.ctypes.data, None if s is None else s.ctypes.data)
                setattr(w, name, mm)
        w.shared_gate = None if self.shared_gate_vec is None else self.shared_gate_vec.ctypes.data
        w.e_score_bias = None if self.e_score_bias is None else self.e_score_bias.ctypes.data
        out = np.empty((T, self.d), dtype=np.float32)
        idx = np.empty((T, self.top_k), dtype=np.int32)
        tw = np.empty((T, self.top_k), dtype=np.float32)
        lg = np.empty((T, self.E), dtype=np.float32)
        rc = lib().oracle_moe_forward(C.byref(cfg), C.byref(w), _ptr(x), C.c_int(T), _ptr(out),
                                      _ptr(idx), _ptr(tw), _ptr(lg), C.c_int(nthreads))
        if rc != 0:
            raise RuntimeError(f"oracle_moe_forward failed with {rc}")
        if want_aux:
            return out, {"topk_idx": idx, "topk_w": tw, "logits": lg}
        return out


def softmax(logits):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    out = np.empty_like(logits)
    lib().oracle_softmax(_ptr(logits), C.c_int(logits.size), _ptr(out))
    return out


def top_k(weights, k, renormalize=True):
    """Returns (rc, indices, weights)."""
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    kk = max(int(k), 0)
    idx = np.zeros(max(kk, 1), dtype=np.int32)
    w = np.zeros(max(kk, 1), dtype=np.float32)
    if kk > weights.size:
        return lib().oracle_top_k(_ptr(weights), C.c_int(weights.size), C.c_int(kk), C.c_int(int(renormalize)),
                                  _ptr(idx), _ptr(w)), None, None
    rc = lib().oracle_top_k(_ptr(weights), C.c_int(weights.size), C.c_int(kk),
                            C.c_int(int(renormalize)), _ptr(idx), _ptr(w))
    return rc, idx[:kk], w[:kk]


def route_from_logits(logits, k, renormalize):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = logits.shape
    idx = np.empty((T, k), dtype=np.int32)
    w = np.empty((T, k), dtype=np.float32)
    rc = lib().oracle_route_from_logits(_ptr(logits), C.c_int(T), C.c_int(E), C.c_int(k),
                                        C.c_int(int(renormalize)), _ptr(idx), _ptr(w))
    if rc:
        raise RuntimeError(f"oracle_route_from_logits failed with {rc}")
    return idx, w


def dispatch_permutation(topk_idx, E):
    topk_idx = np.ascontiguousarray(topk_idx, dtype=np.int32)
    T, k = topk_idx.shape
    off = np.empty(E + 1, dtype=np.int32)
    perm = np.empty(T * k, dtype=np.int32)
    inv = np.empty(T * k, dtype=np.int32)
    lib().oracle_dispatch_permutation(_ptr(topk_idx), C.c_int(T), C.c_int(k), C.c_int(E), _ptr(off),
                                      _ptr(perm), _ptr(inv))
    return off, perm, inv


def quantize_per_row_i8(w):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    q = np.empty((rows, cols), dtype=np.int8)
    s = np.empty(rows, dtype=np.float32)
    lib().oracle_quantize_per_row_i8(_ptr(w), C.c_size_t(rows), C.c_size_t(cols), _ptr(q), _ptr(s))
    return q, s


def dequantize_per_row_i8(q, s):
    q = np.ascontiguousarray(q, dtype=np.int8)
    s = np.ascontiguousarray(s, dtype=np.float32)
    rows, cols = q.shape
    out = np.empty((rows, cols), dtype=np.float32)
    lib().oracle_dequantize_per_row_i8(_ptr(q), _ptr(s), C.c_size_t(rows), C.c_size_t(cols), _ptr(out))
    return out


def absmax_per_group_symmetric(w, group_size=0):
    """Dense W8A16 quantiser over a [K, N] weight; group_size 0 = one group of K rows (per channel)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    K, N = w.shape
    g = group_size if group_size > 0 else max(K, 1)
    groups = (K + g - 1) // g
    q = np.zeros((K, N), dtype=np.int8)
    s = np.zeros((groups, N), dtype=np.float32)
    lib().oracle_absmax_per_group_symmetric(_ptr(w), C.c_size_t(K), C.c_size_t(N), C.c_size_t(g), _ptr(q), _ptr(s))
    return q, s


def int8_to_bf16_per_group(q, s, group_size=0):
    """bf16 bit patterns (uint16) of the reference's truncating dequant."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    s = np.ascontiguousarray(s, dtype=np.float32)
    K, N = q.shape
    g = group_size if group_size > 0 else max(K, 1)
    out = np.zeros((K, N), dtype=np.uint16)
    lib().oracle_int8_to_bf16_per_group(_ptr(q), _ptr(s), C.c_size_t(K), C.c_size_t(N), C.c_size_t(g), _ptr(out))
    return out


def combine_selected(indices, weights, expert_outputs, d):
    indices = np.ascontiguousarray(indices, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    eo = np.ascontiguousarray(expert_outputs, dtype=np.float32).reshape(-1)
    out = np.empty(d, dtype=np.float32)
    rc = lib().oracle_combine_selected(_ptr(indices), _ptr(weights), C.c_int(indices.size), _ptr(eo),
                                       C.c_size_t(eo.size), C.c_int(d), _ptr(out))
    return rc, out


def max_threads():
    return lib().oracle_max_threads()


def v3_route(logits, bias, top_k, n_group, topk_group, scaling, norm_topk_prob):
    """DeepSeek-V3 routing of one token.  Returns (rc, indices, weights, dense_weights)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    n = logits.size
    idx = np.zeros(max(top_k, 1), dtype=np.int32)
    w = np.zeros(max(top_k, 1), dtype=np.float32)
    dense = np.zeros(n, dtype=np.float32)
    rc = lib().oracle_v3_route(_ptr(logits), _ptr(bias), C.c_int(n), C.c_int(top_k), C.c_int(n_group),
                               C.c_int(topk_group), C.c_double(scaling), C.c_int(int(norm_topk_prob)),
                               _ptr(idx), _ptr(w), _ptr(dense))
    return rc, idx[:top_k], w[:top_k], dense


def router_logits(w_router, x, bias=None):
    w_router = np.ascontiguousarray(w_router, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    E, d = w_router.shape
    out = np.empty(E, dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    lib().oracle_router_logits(_ptr(w_router), _ptr(b), C.c_int(E), C.c_int(d), _ptr(x), _ptr(out))
    return out


def expert_forward(w_gate, w_up, w_down, x, accum=ACC_F64):
    w_gate = np.ascontiguousarray(w_gate, dtype=np.float32)
    w_up = np.ascontiguousarray(w_up, dtype=np.float32)
    w_down = np.ascontiguousarray(w_down, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    F, d = w_gate.shape
    y = np.empty(d, dtype=np.float32)
    lib().oracle_expert_forward_f32(_ptr(w_gate), _ptr(w_up), _ptr(w_down), C.c_int(d), C.c_int(F),
                                    C.c_int(accum), _ptr(x), _ptr(y))
    return y


def rms_norm_gamma(x, gamma=None, eps=1e-5):
    """rms_norm(x, eps) * gamma over the last dimension of a [T, d] f32 array."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, d = x.shape
    g = None if gamma is None else np.ascontiguousarray(gamma, dtype=np.float32).reshape(-1)
    out = np.empty_like(x)
    lib().oracle_rms_norm_gamma(_ptr(x), C.c_int(T), C.c_int(d), _ptr(g), C.c_float(eps), _ptr(out))
    return out

