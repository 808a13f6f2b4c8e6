"""ctypes binding of the CPU oracle (oracle/sanic_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's cpu_baseline / reference arm. The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsanic_oracle.so")

DT_F64, DT_F32, DT_F16, DT_BF16 = 0, 1, 2, 3


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "sanic_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libsanic_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_llama_create.restype = C.c_void_p
        _lib.orc_llama_kcache.restype = C.POINTER(C.c_double)
        _lib.orc_llama_vcache.restype = C.POINTER(C.c_double)
        _lib.orc_llama_logits.restype = C.POINTER(C.c_double)
    return _lib


def _d(a):
    a = np.ascontiguousarray(a, dtype=np.float64)
    return a, a.ctypes.data_as(C.POINTER(C.c_double))


def _sz(x):
    return C.c_size_t(int(x))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


class Xorshift:
    """The reference tests' generator (tests/oracle.rs:49-59)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed)

    def uniform(self, *shape) -> np.ndarray:
        out = np.empty(int(np.prod(shape)) if shape else 1, dtype=np.float64)
        lib().orc_xorshift_uniform(C.byref(self.state), out.ctypes.data_as(C.POINTER(C.c_double)), _sz(out.size))
        return out.reshape(shape)

    def normal(self, *shape) -> np.ndarray:
        out = np.empty(int(np.prod(shape)) if shape else 1, dtype=np.float64)
        lib().orc_xorshift_normal(C.byref(self.state), out.ctypes.data_as(C.POINTER(C.c_double)), _sz(out.size))
        return out.reshape(shape)


def round_to(dtype: int, x) -> np.ndarray:
    a, p = _d(x)
    out = np.empty_like(a)
    lib().orc_round_to(C.c_int(dtype), p, out.ctypes.data_as(C.POINTER(C.c_double)), _sz(a.size))
    return out


def to_bf16_bits(x) -> np.ndarray:
    a, p = _d(x)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_to_bf16_bits(p, out.ctypes.data_as(C.POINTER(C.c_uint16)), _sz(a.size))
    return out


def from_bf16_bits(bits) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(b.shape, dtype=np.float64)
    lib().orc_from_bf16_bits(b.ctypes.data_as(C.POINTER(C.c_uint16)), out.ctypes.data_as(C.POINTER(C.c_double)), _sz(b.size))
    return out


def w4_pack(q) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.int8)
    out = np.zeros((q.size + 1) // 2, dtype=np.uint8)
    lib().orc_w4_pack(q.ctypes.data_as(C.POINTER(C.c_int8)), _sz(q.size), out.ctypes.data_as(C.POINTER(C.c_uint8)))
    return out


def w4_unpack(packed, n: int) -> np.ndarray:
    p = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(n, dtype=np.float64)
    lib().orc_w4_unpack(p.ctypes.data_as(C.POINTER(C.c_uint8)), _sz(n), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def _mask_args(mask):
    if mask is None:
        return None, None, None
    m = np.ascontiguousarray(mask, dtype=np.float64)
    shape4 = (1,) * (4 - m.ndim) + tuple(m.shape)
    arr = (C.c_size_t * 4)(*shape4)
    return m, m.ctypes.data_as(C.POINTER(C.c_double)), arr


def _qkv4(q, k, v):
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    lead = q.shape[:-2]
    q4 = q.reshape((1,) * (4 - q.ndim) + q.shape) if q.ndim <= 4 else q
    k4 = k.reshape((1,) * (4 - k.ndim) + k.shape)
    v4 = v.reshape((1,) * (4 - v.ndim) + v.shape)
    return q4, k4, v4, lead


def sdpa(q, k, v, mask=None, is_causal=False, scale=None, enable_gqa=False) -> np.ndarray:
    """eval(scaled_dot_product_attention(...)), torch layout [N, H, L, E] (src/nn.rs:27-105)."""
    q4, k4, v4, lead = _qkv4(q, k, v)
    N, Hq, L, E = q4.shape
    _, H, S, _ = k4.shape
    Ev = v4.shape[-1]
    if scale is None:
        scale = 1.0 / np.sqrt(E)
    (qa, qp), (ka, kp), (va, vp) = _d(q4), _d(k4), _d(v4)
    m, mp, ms = _mask_args(mask)
    out = np.empty((N, Hq, L, Ev), dtype=np.float64)
    rc = lib().orc_sdpa(qp, kp, vp, mp, ms, _sz(N), _sz(Hq), _sz(H), _sz(L), _sz(S), _sz(E), _sz(Ev),
                        C.c_int(int(is_causal)), C.c_double(scale), C.c_int(int(enable_gqa)),
                        out.ctypes.data_as(C.POINTER(C.c_double)))
    assert rc == 0
    return out.reshape(lead + (L, Ev))


def sdpa_window(q, k, v, window: int, scale=None) -> np.ndarray:
    """Sliding-window attention as the reference formulates it (tests/movement.rs:294-345)."""
    q4, k4, v4, lead = _qkv4(q, k, v)
    N, Hq, L, E = q4.shape
    H = k4.shape[1]
    Ev = v4.shape[-1]
    if scale is None:
        scale = 1.0 / np.sqrt(E)
    (qa, qp), (ka, kp), (va, vp) = _d(q4), _d(k4), _d(v4)
    out = np.empty((N, Hq, L, Ev), dtype=np.float64)
    lib().orc_sdpa_window(qp, kp, vp, _sz(N), _sz(Hq), _sz(H), _sz(L), _sz(E), _sz(Ev), _sz(window),
                          C.c_double(scale), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out.reshape(lead + (L, Ev))


def sdpa_carrier_split(q, k, v, blocks: int, mask=None, is_causal=False, scale=None, enable_gqa=False,
                       return_carriers=False):
    """run_carrier_split of the derived (m, l, o) carrier (src/interp.rs:555-643)."""
    q4, k4, v4, lead = _qkv4(q, k, v)
    N, Hq, L, E = q4.shape
    _, H, S, _ = k4.shape
    Ev = v4.shape[-1]
    if scale is None:
        scale = 1.0 / np.sqrt(E)
    (qa, qp), (ka, kp), (va, vp) = _d(q4), _d(k4), _d(v4)
    m, mp, ms = _mask_args(mask)
    out = np.empty((N, Hq, L, Ev), dtype=np.float64)
    car = np.empty((N, Hq, L, 2 + Ev), dtype=np.float64) if return_carriers else None
    rc = lib().orc_sdpa_carrier_split(qp, kp, vp, mp, ms, _sz(N), _sz(Hq), _sz(H), _sz(L), _sz(S), _sz(E), _sz(Ev),
                                      C.c_int(int(is_causal)), C.c_double(scale), C.c_int(int(enable_gqa)),
                                      _sz(blocks), out.ctypes.data_as(C.POINTER(C.c_double)),
                                      car.ctypes.data_as(C.POINTER(C.c_double)) if return_carriers else None)
    if rc != 0:
        raise ValueError("blocks must be in [1, extent]")
    out = out.reshape(lead + (L, Ev))
    return (out, car) if return_carriers else out


def carrier_merge_mlo(parts) -> np.ndarray:
    """Merge [n_parts, rows, 2+Ev] raw (m, l, o) accumulators left to right and project."""
    a, p = _d(parts)
    n_parts, rows, w = a.shape
    out = np.empty((rows, w - 2), dtype=np.float64)
    lib().orc_carrier_merge_mlo(p, _sz(n_parts), _sz(rows), _sz(w - 2), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def rms_norm(x, w, eps=1e-5) -> np.ndarray:
    a, p = _d(x)
    wa, wp = _d(w)
    n = a.shape[-1]
    out = np.empty_like(a)
    lib().orc_rms_norm(p, wp, _sz(a.size // n), _sz(n), C.c_double(eps), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def rmsnorm_gemm(x, gamma, w, eps=1e-5, w_is_nk=False, blocks=None) -> np.ndarray:
    a, p = _d(x)
    g, gp = _d(gamma)
    ww, wp = _d(w)
    M, K = a.shape
    N = ww.shape[0] if w_is_nk else ww.shape[1]
    out = np.empty((M, N), dtype=np.float64)
    op = out.ctypes.data_as(C.POINTER(C.c_double))
    if blocks is None:
        lib().orc_rmsnorm_gemm(p, gp, wp, _sz(M), _sz(K), _sz(N), C.c_int(int(w_is_nk)), C.c_double(eps), op)
    else:
        rc = lib().orc_rmsnorm_gemm_carrier_split(p, gp, wp, _sz(M), _sz(K), _sz(N), C.c_int(int(w_is_nk)),
                                                  C.c_double(eps), _sz(blocks), op)
        if rc != 0:
            raise ValueError("blocks must be in [1, extent]")
    return out


def w4_gemv(packed, scales, x, n_out: int, group: int = 64, blocks=None) -> np.ndarray:
    pk = np.ascontiguousarray(packed, dtype=np.uint8)
    s, sp = _d(scales)
    a, p = _d(x)
    a2 = a.reshape(-1, a.shape[-1])
    batch, K = a2.shape
    out = np.empty((batch, n_out), dtype=np.float64)
    op = out.ctypes.data_as(C.POINTER(C.c_double))
    pp = pk.ctypes.data_as(C.POINTER(C.c_uint8))
    if blocks is None:
        lib().orc_w4_gemv(pp, sp, p, _sz(batch), _sz(n_out), _sz(K), _sz(group), op)
    else:
        rc = lib().orc_w4_gemv_carrier_split(pp, sp, p, _sz(batch), _sz(n_out), _sz(K), _sz(group), _sz(blocks), op)
        if rc != 0:
            raise ValueError("blocks must be in [1, extent]")
    return out.reshape(a.shape[:-1] + (n_out,))


def gemv_bf16w(w_bits, x) -> np.ndarray:
    w = np.ascontiguousarray(w_bits, dtype=np.uint16)
    a, p = _d(x)
    a2 = a.reshape(-1, a.shape[-1])
    batch, K = a2.shape
    n_out = w.shape[0]
    out = np.empty((batch, n_out), dtype=np.float64)
    lib().orc_gemv_bf16w(w.ctypes.data_as(C.POINTER(C.c_uint16)), p, _sz(batch), _sz(n_out), _sz(K),
                         out.ctypes.data_as(C.POINTER(C.c_double)))
    return out.reshape(a.shape[:-1] + (n_out,))


def argmax(x, blocks=None) -> np.ndarray:
    a, p = _d(x)
    n = a.shape[-1]
    rows = a.size // n
    out = np.empty(rows, dtype=np.float64)
    op = out.ctypes.data_as(C.POINTER(C.c_double))
    if blocks is None:
        lib().orc_argmax(p, _sz(rows), _sz(n), op)
    else:
        rc = lib().orc_argmax_carrier_split(p, _sz(rows), _sz(n), _sz(blocks), op)
        if rc != 0:
            raise ValueError("blocks must be in [1, extent]")
    return out.reshape(a.shape[:-1])


def rope_inv_freq(theta: float, n_freq: int) -> np.ndarray:
    out = np.empty(n_freq, dtype=np.float64)
    lib().orc_rope_inv_freq(C.c_double(theta), _sz(n_freq), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def llama3_inv_freq(n_freq: int) -> np.ndarray:
    out = np.empty(n_freq, dtype=np.float64)
    lib().orc_llama3_inv_freq(_sz(n_freq), out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


def rope(x, positions, inv_freq) -> np.ndarray:
    """Rotate-half RoPE (src/nn.rs:176-194). x [..., D]; positions broadcast to x.shape[:-1]."""
    a, p = _d(x)
    D = a.shape[-1]
    pos = np.ascontiguousarray(np.broadcast_to(np.asarray(positions, dtype=np.float64), a.shape[:-1]))
    f, fp = _d(inv_freq)
    out = np.empty_like(a)
    lib().orc_rope(p, pos.ctypes.data_as(C.POINTER(C.c_double)), fp, _sz(a.size // D), _sz(D),
                   out.ctypes.data_as(C.POINTER(C.c_double)))
    return out


class _LlamaCfg(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("vocab", "layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn",
                                          "ctx", "batch")] + \
               [("w4", C.c_int32), ("group", C.c_int32), ("round_acts", C.c_int32), ("llama3_rope", C.c_int32),
                ("w4_head", C.c_int32), ("norm_store", C.c_int32), ("eps", C.c_double), ("theta", C.c_double)]


_PP = C.POINTER(C.c_void_p)


class _LlamaWeights(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("final_norm", C.c_void_p), ("attn_norm", _PP), ("mlp_norm", _PP)] + \
               [(n, _PP) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown",
                                   "sq", "sk", "sv", "so", "sgate", "sup", "sdown")] + [("sembed", C.c_void_p)]


class Llama:
    """Stateful oracle of the decode-step graph (examples/llama3_2.rs:112-253) with a batch axis.

    `weights` maps names to numpy arrays: 'embed' [vocab, hidden] uint16 (bf16 bits), 'final_norm',
    and per layer lists 'attn_norm', 'mlp_norm', 'wq', 'wk', 'wv', 'wo', 'wgate', 'wup', 'wdown'
    (uint16 bf16 bits [out, in], or uint8 packed int4 when w4) and 'sq' ... 'sdown' (bf16 bits scales).
    cfg['w4_head'] = 1: 'embed' is packed int4 [vocab, hidden/2] with 'sembed' [vocab, hidden/group] scales.
    cfg['norm_store'] = 1: stored(bf16) sits on x*g and the RMSNorm division is deferred past each contraction.
    cfg['norm_store'] = 2: the same at every norm a residual-add feeds; layer 0's attention norm (fed by the gather) keeps
    stored(rms_norm(x)).
    """

    def __init__(self, cfg: dict, weights: dict):
        self._keep = []
        c = _LlamaCfg()
        for k in ("vocab", "layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn", "ctx", "batch"):
            setattr(c, k, int(cfg[k]))
        c.w4 = int(cfg.get("w4", 0))
        c.group = int(cfg.get("group", 64))
        c.round_acts = int(cfg.get("round_acts", 1))
        c.llama3_rope = int(cfg.get("llama3_rope", 1))
        c.w4_head = int(cfg.get("w4_head", 0))
        c.norm_store = int(cfg.get("norm_store", 0))
        c.eps = float(cfg.get("eps", 1e-5))
        c.theta = float(cfg.get("theta", 500000.0))
        self.cfg = cfg
        w = _LlamaWeights()

        def ptr(a):
            a = np.ascontiguousarray(a)
            self._keep.append(a)
            return a.ctypes.data

        def ptrs(lst):
            arr = (C.c_void_p * len(lst))(*[ptr(a) for a in lst])
            self._keep.append(arr)
            return C.cast(arr, _PP)

        w.embed = ptr(weights["embed"])
        w.final_norm = ptr(weights["final_norm"])
        if c.w4_head:
            w.sembed = ptr(weights["sembed"])
        for name in ("attn_norm", "mlp_norm", "wq", "wk", "wv", "wo", "wgate", "wup", "wdown"):
            setattr(w, name, ptrs(weights[name]))
        if c.w4:
            for name in ("sq", "sk", "sv", "so", "sgate", "sup", "sdown"):
                setattr(w, name, ptrs(weights[name]))
        self._h = C.c_void_p(lib().orc_llama_create(C.byref(c), C.byref(w)))
        L, B, Hk, T, D = (int(cfg[k]) for k in ("layers", "batch", "kv_heads", "ctx", "head_dim"))
        self.kcache = np.ctypeslib.as_array(lib().orc_llama_kcache(self._h), shape=(L, B, Hk, T, D))
        self.vcache = np.ctypeslib.as_array(lib().orc_llama_vcache(self._h), shape=(L, B, Hk, D, T))

    def step(self, tokens, position: int) -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty_like(t)
        rc = lib().orc_llama_step(self._h, t.ctypes.data_as(C.POINTER(C.c_int32)), C.c_int64(position),
                                  out.ctypes.data_as(C.POINTER(C.c_int32)))
        if rc != 0:
            raise ValueError(f"orc_llama_step failed with {rc}")
        return out

    def logits(self) -> np.ndarray:
        B, V = int(self.cfg["batch"]), int(self.cfg["vocab"])
        return np.ctypeslib.as_array(lib().orc_llama_logits(self._h), shape=(B, V)).copy()

    def __del__(self):
        try:
            lib().orc_llama_destroy(self._h)
        except Exception:
            pass
