"""Host-side mirror of the reference's backend boundary over the C ABI.

`CudaDevice` plays the role `MetalDevice` plays behind `trait Backend` in the reference
(src/compile.rs:87-108 of the reference project): hardware facts, buffers, and one method per
kernel family the emitter can select. torch is used only for device memory and streams; every
computation goes through libsanic_b200.so.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _abi as abi


class CompileError(Exception):
    """Mirror of CompileError (reference src/compile.rs:18-40)."""


class RunError(Exception):
    """Mirror of RunError (reference src/compile.rs:42-76)."""


_TORCH_DTYPE = {abi.F32: torch.float32, abi.BF16: torch.bfloat16, abi.F16: torch.float16}


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class CudaDevice:
    def __init__(self, ordinal: int = 0):
        if not torch.cuda.is_available():
            raise RunError("sanic_b200 needs a CUDA device; there is no CPU fallback")
        self.lib = abi.load()
        self.ordinal = ordinal
        self.torch_device = torch.device("cuda", ordinal)
        h = C.c_void_p()
        rc = self.lib.sanic_cuda_open(ordinal, C.byref(h))
        if rc != abi.OK:
            raise RunError(f"sanic_cuda_open({ordinal}) failed with status {rc} (an sm_100 device is required)")
        self.h = h
        self._scratch = {}

    # ── plumbing ──
    def close(self):
        if getattr(self, "h", None):
            self.lib.sanic_cuda_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc == abi.OK:
            return
        msg = self.lib.sanic_last_error(self.h).decode()
        if rc in (abi.ERR_UNSUPPORTED,):
            raise CompileError(f"{what}: {msg}")
        raise RunError(f"{what}: status {rc}: {msg}")

    def stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.torch_device).cuda_stream)

    def sync(self):
        """Wait for the current stream and surface any device-side status (bounded waits that ran out)."""
        self._check(self.lib.sanic_sync(self.h, self.stream()), "sync")

    def specs(self) -> dict:
        s = abi.DeviceSpecs()
        self._check(self.lib.sanic_specs(self.h, C.byref(s)), "specs")
        return {f: getattr(s, f) for f, _ in s._fields_}

    def empty(self, shape, dtype):
        return torch.empty(shape, dtype=dtype, device=self.torch_device)

    def _on_device(self, name, t, dtype=None, strided=False):
        if not isinstance(t, torch.Tensor) or t.device != self.torch_device:
            raise RunError(f"input `{name}` is not a tensor on {self.torch_device}")
        if dtype is not None and t.dtype != dtype:
            raise RunError(f"input `{name}` has dtype {t.dtype}; expected {dtype}")
        if strided:      # the entry point takes element strides; only the innermost axis must be dense
            if t.stride(-1) != 1:
                raise RunError(f"input `{name}` must be contiguous along its last axis")
        elif not t.is_contiguous():
            raise RunError(f"input `{name}` must be contiguous")
        return t

    def emit_select(self, kinds, refs=None, leaf_dtype=abi.F32, in_body_contraction=False, deferred_div=False) -> int:
        c = make_carrier(kinds, refs, leaf_dtype, in_body_contraction, deferred_div)
        fam = C.c_int32(0)
        rc = self.lib.sanic_emit_select(C.byref(c), C.byref(fam))
        if rc != abi.OK:
            raise CompileError("no kernel for this carrier structure")
        return fam.value

    # ── K2a: online-softmax fold ──
    def _attn_params(self, q, k, v, out, causal, window, scale, mask, out_dtype):
        B, Hq, L, E = q.shape
        _, Hkv, S, _ = k.shape
        Ev = v.shape[-1]
        if k.shape[0] != B or v.shape[:3] != k.shape[:3] or k.shape[3] != E:
            raise RunError(f"attention shapes disagree: q {tuple(q.shape)} k {tuple(k.shape)} v {tuple(v.shape)}")
        p = abi.AttnParams()
        p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
        p.batch, p.q_heads, p.kv_heads = B, Hq, Hkv
        p.q_len, p.kv_len, p.head_dim, p.v_dim = L, S, E, Ev
        p.causal, p.window = int(causal), int(window)
        p.scale = float(scale if scale is not None else 1.0 / math.sqrt(E))
        p.mask = mask.data_ptr() if mask is not None else None
        p.out_dtype = out_dtype
        return p

    def attn_fwd_f32(self, q, k, v, causal=False, window=0, scale=None, mask=None, f64_accumulate=False):
        """q [B,Hq,L,E], k [B,Hkv,S,E], v [B,Hkv,S,Ev] f32 -> [B,Hq,L,Ev] f32. `f64_accumulate` keeps scores,
        exponentials and the carrier in f64 (one rounding, at the store)."""
        for n, t in (("q", q), ("k", k), ("v", v)):
            self._on_device(n, t, torch.float32)
        if mask is not None:
            self._on_device("mask", mask, torch.float32)
        out = self.empty((q.shape[0], q.shape[1], q.shape[2], v.shape[-1]), torch.float32)
        p = self._attn_params(q, k, v, out, causal, window, scale, mask, abi.F32)
        p.accum_dtype = abi.F64 if f64_accumulate else abi.F32
        self._check(self.lib.sanic_attn_fwd_f32(self.h, C.byref(p), self.stream()), "attn_fwd_f32")
        return out

    def attn_fwd_bf16(self, q, k, v, causal=False, window=0, scale=None):
        for n, t in (("q", q), ("k", k), ("v", v)):
            self._on_device(n, t, torch.bfloat16)
        out = self.empty((q.shape[0], q.shape[1], q.shape[2], v.shape[-1]), torch.bfloat16)
        p = self._attn_params(q, k, v, out, causal, window, scale, None, abi.BF16)
        self._check(self.lib.sanic_attn_fwd_bf16(self.h, C.byref(p), self.stream()), "attn_fwd_bf16")
        return out

    def attn_fwd_bf16_profile(self, q, k, v, causal=False, window=0, scale=None):
        """One launch of the flash forward with its clock counters on (CTA 0): returns (counters, out). Per query tile
        the clocks its first softmax warp spent in each part of its loop, and its MMA thread's polls and clocks
        (see sanic_attn_fwd_bf16_profile)."""
        for n, t in (("q", q), ("k", k), ("v", v)):
            self._on_device(n, t, torch.bfloat16)
        out = self.empty((q.shape[0], q.shape[1], q.shape[2], v.shape[-1]), torch.bfloat16)
        p = self._attn_params(q, k, v, out, causal, window, scale, None, abi.BF16)
        raw = (C.c_uint64 * 40)()
        self._check(self.lib.sanic_attn_fwd_bf16_profile(self.h, C.byref(p), self.stream(), raw), "attn_fwd_bf16_profile")
        names = ("wait_scores", "load_scores", "row_max", "first_half_exponentials", "wait_previous_pv", "rescale",
                 "stores_and_second_half", "store_wait_and_arrive", "epilogue_and_item_switch", "fence_after_scores_wait")
        prof = {}
        for t in range(2):
            tiles = max(1, raw[t * 12 + 10])
            prof[f"tile{t}"] = dict(key_tiles=int(raw[t * 12 + 10]), clocks=int(raw[t * 12 + 11]),
                                    clocks_per_key_tile={nm: raw[t * 12 + i] / tiles for i, nm in enumerate(names)})
        for t in range(2):
            m = raw[24 + 8 * t:32 + 8 * t]
            per = max(1, m[3])
            prof[f"mma_thread{t}"] = dict(polls=int(m[0]), idle_polls=int(m[1]), clocks=int(m[2]), qk_issued=int(m[3]),
                                          clocks_per_key_tile=dict(barrier_tests_and_sleep=m[4] / per, score_products=m[5] / per,
                                                                   value_products=m[6] / per, item_switch=m[7] / per))
        return prof, out

    def decode_scratch(self, batch, q_heads, head_dim, n_splits):
        nbytes = self.lib.sanic_attn_decode_scratch_bytes(batch, q_heads, head_dim, n_splits)
        key = ("decode", batch, q_heads, head_dim, n_splits)
        buf = self._scratch.get(key)
        if buf is None:
            buf = torch.zeros(nbytes // 4, dtype=torch.float32, device=self.torch_device)
            self._scratch[key] = buf
        return buf

    def suggest_splits(self, batch, kv_heads, head_dim, kv_len):
        return int(self.lib.sanic_attn_decode_suggest_splits(self.h, batch, kv_heads, head_dim, kv_len))

    def decode_params(self, q, k, v, kv_len, v_transposed=False, n_splits=None, window=0, scale=None,
                      kv_len_dev=None, out=None, carrier_out=None, partials=None, out_dtype=abi.BF16, kv_cap=None):
        """Fill a DecodeParams. q [B,Hq,D] bf16; k [B,Hkv,S,D]; v [B,Hkv,S,D] or [B,Hkv,D,S] when v_transposed.
        `kv_cap` (default: the key extent of k) bounds what a device-side length may make the kernel read."""
        B, Hq, D = q.shape
        Hkv = k.shape[1]
        if n_splits is None:
            n_splits = self.suggest_splits(B, Hkv, D, kv_len)
        p = abi.DecodeParams()
        p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        p.k_batch_stride, p.k_head_stride, p.k_seq_stride = k.stride(0), k.stride(1), k.stride(2)
        p.v_batch_stride, p.v_head_stride, p.v_row_stride = v.stride(0), v.stride(1), v.stride(2)
        p.v_transposed = int(v_transposed)
        p.batch, p.q_heads, p.kv_heads, p.head_dim = B, Hq, Hkv, D
        p.kv_len = int(kv_len)
        p.kv_len_dev = kv_len_dev.data_ptr() if kv_len_dev is not None else None
        p.window, p.n_splits = int(window), int(n_splits)
        p.scale = float(scale if scale is not None else 1.0 / math.sqrt(D))
        if partials is None:
            partials = self.decode_scratch(B, Hq, D, n_splits)
        p.partials = partials.data_ptr()
        p.carrier_out = carrier_out.data_ptr() if carrier_out is not None else None
        p.out = out.data_ptr() if out is not None else None
        p.out_dtype = out_dtype
        p.kv_cap = int(kv_cap if kv_cap is not None else k.shape[2])
        return p, partials

    def streamk_slots(self, batch, kv_heads, head_dim):
        return int(self.lib.sanic_attn_decode_streamk_slots(self.h, batch, kv_heads, head_dim))

    def attn_decode(self, q, k, v, kv_len, v_transposed=False, n_splits=None, window=0, scale=None,
                    return_carrier=False, out_dtype=torch.bfloat16, streamk=False, kv_len_dev=None):
        """Split-KV decode fold. `streamk`: one contiguous range of the (batch, kv head, key tile) space per resident CTA
        instead of n_splits fixed chunks per (batch, kv head)."""
        self._on_device("q", q, torch.bfloat16)
        self._on_device("k", k, torch.bfloat16, strided=True)      # slices of a longer cache are read in place
        self._on_device("v", v, torch.bfloat16, strided=True)
        B, Hq, D = q.shape
        out = self.empty((B, Hq, D), out_dtype)
        car = self.empty((B * Hq, D + 2), torch.float32) if return_carrier else None
        if streamk:
            n_splits = self.streamk_slots(B, k.shape[1], D)
        p, _keep = self.decode_params(q, k, v, kv_len, v_transposed, n_splits, window, scale, out=out, carrier_out=car,
                                      out_dtype=abi.BF16 if out_dtype == torch.bfloat16 else abi.F32, kv_len_dev=kv_len_dev)
        fn = self.lib.sanic_attn_decode_streamk if streamk else self.lib.sanic_attn_decode_splitkv
        self._check(fn(self.h, C.byref(p), self.stream()), "attn_decode")
        return (out, car) if return_carrier else out

    def carrier_merge(self, parts, out_dtype=torch.float32, return_carrier=False):
        """parts [n_parts, rows, 2+D] f32 -> projected [rows, D]."""
        self._on_device("parts", parts, torch.float32)
        n_parts, rows, W = parts.shape
        out = self.empty((rows, W - 2), out_dtype)
        car = self.empty((rows, W), torch.float32) if return_carrier else None
        rc = self.lib.sanic_carrier_merge(self.h, _ptr(parts), n_parts, rows, W - 2, _ptr(car), _ptr(out),
                                          abi.BF16 if out_dtype == torch.bfloat16 else abi.F32, self.stream())
        self._check(rc, "carrier_merge")
        return (out, car) if return_carrier else out

    # ── K2b: deferred-normaliser contraction ──
    def gemm_prescale_weights(self, gamma, w, w_is_nk=True):
        """bf16(W * g) along K, for weights that are bound once; pass the result to gemm_rmsnorm with gamma=None."""
        for n, t in (("gamma", gamma), ("w", w)):
            self._on_device(n, t, torch.bfloat16)
        N, K = (w.shape[0], w.shape[1]) if w_is_nk else (w.shape[1], w.shape[0])
        if gamma.shape[0] != K:
            raise RunError("gemm_prescale_weights: gamma must have one entry per contraction index")
        out = torch.empty_like(w)
        self._check(self.lib.sanic_gemm_prescale_weights(self.h, _ptr(gamma), _ptr(w), _ptr(out), N, K, int(w_is_nk), self.stream()),
                    "gemm_prescale_weights")
        return out

    def gemm_rmsnorm(self, x, gamma, w, eps=1e-5, w_is_nk=True, out_dtype=torch.bfloat16):
        for n, t in (("x", x), ("w", w)) + ((("gamma", gamma),) if gamma is not None else ()):
            self._on_device(n, t, torch.bfloat16)
        M, K = x.shape
        N = w.shape[0] if w_is_nk else w.shape[1]
        if (w.shape[1] if w_is_nk else w.shape[0]) != K or (gamma is not None and gamma.shape[0] != K):
            raise RunError("gemm_rmsnorm: contraction extents must match")
        y = self.empty((M, N), out_dtype)
        p = abi.GemmRmsnormParams()
        p.x, p.gamma, p.w, p.y = x.data_ptr(), (gamma.data_ptr() if gamma is not None else None), w.data_ptr(), y.data_ptr()
        p.M, p.N, p.K, p.w_is_nk, p.eps = M, N, K, int(w_is_nk), float(eps)
        p.out_dtype = abi.BF16 if out_dtype == torch.bfloat16 else abi.F32
        self._check(self.lib.sanic_gemm_rmsnorm(self.h, C.byref(p), self.stream()), "gemm_rmsnorm")
        return y

    def gemm_rmsnorm_pair_profile(self, x, gamma, w, eps=1e-5, w_is_nk=True):
        """One launch of the pair tile with A through registers with its clock counters on: a dict of clocks per k-block for
        the MMA thread, the B producer and transform warp 0 of each CTA of SM pair 0 (see sanic_gemm_rmsnorm_pair_profile)."""
        M, K = x.shape
        N = w.shape[0] if w_is_nk else w.shape[1]
        y = self.empty((M, N), torch.bfloat16)
        p = abi.GemmRmsnormParams()
        p.x, p.gamma, p.w, p.y = x.data_ptr(), (gamma.data_ptr() if gamma is not None else None), w.data_ptr(), y.data_ptr()
        p.M, p.N, p.K, p.w_is_nk, p.eps, p.out_dtype = M, N, K, int(w_is_nk), float(eps), abi.BF16
        out = (C.c_uint64 * 18)()
        self._check(self.lib.sanic_gemm_rmsnorm_pair_profile(self.h, C.byref(p), self.stream(), out), "gemm_rmsnorm_pair_profile")
        v = [int(t) for t in out]
        n = max(v[0], 1)
        res = {"k_blocks": v[0], "mma_thread_clocks_per_kb": v[1] / n, "of_which_reading_counters": v[2] / n,
               "counter_reads_per_kb": v[3] / n, "waiting_for_accumulator_total": v[4], "b_producer_wait_per_kb": v[5] / n}
        for name, o in (("leader", 6), ("peer", 12)):
            m = max(v[o], 1)
            res["transform_warp_" + name] = {"k_blocks": v[o], "arithmetic": v[o + 1] / m, "slot_wait": v[o + 2] / m,
                                             "stores": v[o + 3] / m, "proxy_fence": v[o + 4] / m, "arrival": v[o + 5] / m}
        return res, y

    # ── K2c: decode-batch contraction ──
    def gemv_params(self, x, weights, outs, scales=None, epilogue=abi.EPI_STORE, residual=None, out_dtype=abi.F32):
        batch, K = x.shape
        p = abi.GemvParams()
        p.x, p.batch, p.K = x.data_ptr(), batch, K
        w4 = weights[0].dtype == torch.uint8
        p.weight_dtype = abi.I4 if w4 else abi.BF16
        p.group = 64
        p.n_segments = len(weights)
        for i, w in enumerate(weights):
            p.w[i] = w.data_ptr()
            p.rows[i] = w.shape[0]
            if w4:
                p.scales[i] = scales[i].data_ptr()
            if i < len(outs) and outs[i] is not None:
                p.out[i] = outs[i].data_ptr()
        p.out_dtype, p.epilogue = out_dtype, epilogue
        p.residual = residual.data_ptr() if residual is not None else None
        return p

    def gemv(self, x, weights, scales=None, epilogue=abi.EPI_STORE, residual=None, out_dtype=torch.float32,
             norm_gamma=None, norm_eps=1e-5):
        """x [batch, K] bf16; weights: list of [rows, K] bf16 or [rows, K/2] uint8 (+ scales [rows, K/64] bf16).
        With norm_gamma, x is the f32 residual stream and its RMSNorm is inlined into the contraction."""
        self._on_device("x", x, torch.float32 if norm_gamma is not None else torch.bfloat16)
        weights = list(weights)
        for i, w in enumerate(weights):
            self._on_device(f"w[{i}]", w)
        batch = x.shape[0]
        n_out = 1 if epilogue == abi.EPI_SILU_MUL else len(weights)
        outs = [self.empty((batch, weights[i].shape[0]), out_dtype) for i in range(n_out)]
        p = self.gemv_params(x, weights, outs, scales, epilogue, residual,
                             abi.BF16 if out_dtype == torch.bfloat16 else abi.F32)
        if norm_gamma is not None:
            self._on_device("norm_gamma", norm_gamma, torch.bfloat16)
            p.norm_x, p.norm_gamma, p.norm_eps = x.data_ptr(), norm_gamma.data_ptr(), float(norm_eps)
        self._check(self.lib.sanic_gemv(self.h, C.byref(p), self.stream()), "gemv")
        return outs[0] if n_out == 1 else outs

    # ── K2d ──
    def argmax(self, x):
        self._on_device("x", x, torch.float32)
        rows, n = x.shape
        out = self.empty((rows,), torch.int32)
        scratch = self.empty((rows * 2 * 256,), torch.float32)
        self._check(self.lib.sanic_argmax(self.h, _ptr(x), rows, n, _ptr(out), _ptr(scratch), self.stream()), "argmax")
        return out

    # ── K3 ──
    def rmsnorm(self, x, gamma, eps=1e-5):
        self._on_device("x", x, torch.float32)
        self._on_device("gamma", gamma, torch.bfloat16)
        out = self.empty(x.shape, torch.bfloat16)
        rows = x.numel() // x.shape[-1]
        self._check(self.lib.sanic_rmsnorm(self.h, _ptr(x), _ptr(gamma), rows, x.shape[-1], eps, _ptr(out), self.stream()),
                    "rmsnorm")
        return out

    def embed_gather(self, table, tokens):
        self._on_device("table", table, torch.bfloat16)
        self._on_device("tokens", tokens, torch.int32)
        out = self.empty((tokens.shape[0], table.shape[1]), torch.float32)
        rc = self.lib.sanic_embed_gather(self.h, _ptr(table), _ptr(tokens), tokens.shape[0], table.shape[1],
                                         table.shape[0], _ptr(out), self.stream())
        self._check(rc, "embed_gather")
        return out

    def embed_gather_w4(self, table, scales, tokens, group=64):
        """table [vocab, hidden/2] uint8 nibbles, scales [vocab, hidden/group] bf16 -> widened rows [batch, hidden] f32."""
        self._on_device("table", table, torch.uint8)
        self._on_device("scales", scales, torch.bfloat16)
        self._on_device("tokens", tokens, torch.int32)
        hidden = table.shape[1] * 2
        out = self.empty((tokens.shape[0], hidden), torch.float32)
        rc = self.lib.sanic_embed_gather_w4(self.h, _ptr(table), _ptr(scales), _ptr(tokens), tokens.shape[0], hidden,
                                            table.shape[0], group, _ptr(out), self.stream())
        self._check(rc, "embed_gather_w4")
        return out

    def rope_table(self, inv_freq, n_pos):
        """inv_freq: host sequence of doubles -> table [n_pos, F, 2] f32 (cos, sin)."""
        F = len(inv_freq)
        arr = (C.c_double * F)(*[float(v) for v in inv_freq])
        table = self.empty((n_pos, F, 2), torch.float32)
        self._check(self.lib.sanic_rope_table(self.h, arr, F, n_pos, _ptr(table), self.stream()), "rope_table")
        return table

    def rope_bf16(self, x, table, pos0=0, out=None):
        """x [..., seq, D] bf16, rotate-half RoPE with position pos0 + s."""
        self._on_device("x", x, torch.bfloat16)
        seq, D = x.shape[-2], x.shape[-1]
        rows = x.numel() // (seq * D)
        if table.shape[0] < pos0 + seq or table.shape[1] != D // 2:
            raise RunError("rope_bf16: table does not cover the positions")
        if out is None:
            out = torch.empty_like(x)
        self._check(self.lib.sanic_rope_bf16(self.h, _ptr(x), _ptr(out), rows, seq, D, _ptr(table), pos0, self.stream()),
                    "rope_bf16")
        return out

    # ── K4 ──
    def round_to_bf16_bits(self, x):
        self._on_device("x", x, torch.float32)
        out = self.empty(x.shape, torch.int16)
        self._check(self.lib.sanic_round_to_bf16(self.h, _ptr(x), x.numel(), _ptr(out), self.stream()), "round_to_bf16")
        return out

    def store_u32_saturating(self, x):
        self._on_device("x", x, torch.float32)
        out = self.empty(x.shape, torch.int32)
        self._check(self.lib.sanic_store_u32_saturating(self.h, _ptr(x), x.numel(), _ptr(out), self.stream()), "store_u32")
        return out

    def w4_unpack(self, packed, n_elems):
        self._on_device("packed", packed, torch.uint8)
        out = self.empty((n_elems,), torch.float32)
        self._check(self.lib.sanic_w4_unpack(self.h, _ptr(packed), n_elems, _ptr(out), self.stream()), "w4_unpack")
        return out


def make_carrier(kinds, refs=None, leaf_dtype=abi.F32, in_body_contraction=False, deferred_div=False):
    c = abi.CarrierDesc()
    c.n_slots = len(kinds)
    for i, k in enumerate(kinds):
        c.kind[i] = k
        c.ref[i] = (refs or [0] * len(kinds))[i]
    c.leaf_dtype = leaf_dtype
    c.in_body_contraction = int(in_body_contraction)
    c.deferred_div = int(deferred_div)
    return c


# The four derived carriers of the hot path, as the reference's deriver reports them
# (tests/laws.rs:107-126,620-646; tests/compile.rs:139-171; tests/metal.rs:1224-1236).
def carrier_online_softmax(leaf_dtype=abi.BF16):
    return make_carrier([abi.SLOT_PLAIN_MAX, abi.SLOT_EXP_SHIFTED, abi.SLOT_EXP_SHIFTED], [0, 0, 0], leaf_dtype, True)


def carrier_deferred_norm(leaf_dtype=abi.BF16):
    return make_carrier([abi.SLOT_PLAIN_ADD, abi.SLOT_PLAIN_ADD], [0, 0], leaf_dtype, False, True)


def carrier_contraction(leaf_dtype=abi.BF16):
    return make_carrier([abi.SLOT_PLAIN_ADD], [0], leaf_dtype)


def carrier_extremum_index():
    return make_carrier([abi.SLOT_PLAIN_MAX, abi.SLOT_AT_EXTREMUM], [0, 0], abi.F32)
