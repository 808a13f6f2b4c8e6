"""Llama-3.2-1B-architecture decode step as a captured launch list.

Mirrors the stateful-stepping API of the reference (`Graph::compile_for` ->
`StepProgram::instantiate` -> `Machine::step`, src/graph.rs:231-356 of the reference project)
for the decode graph of examples/llama3_2.rs:112-253, with a leading batch axis and a shared
scalar position. The emitter's product is an ordered stage list (Fused / Elementwise / Gather,
src/partition.rs:44-98); state (KV caches, position, token) lives in device buffers owned by
the machine, and a step is one CUDA-graph replay with no host writes.

Storage declarations (the graph's, not the kernels'): weights bf16 or int4+bf16 scales; caches
bf16; the residual stream is pinned f32; every activation a projection reads, and q, are
stored bf16 (a bf16 boundary policy).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _abi as abi
from .backend import (CompileError, CudaDevice, RunError, carrier_contraction, carrier_extremum_index,
                      carrier_online_softmax)

LLAMA_3_2_1B = dict(vocab=128256, layers=16, hidden=2048, q_heads=32, kv_heads=8, head_dim=64, ffn=8192)

ROPE_THETA = 500000.0


def llama3_inv_freq(n_freq: int):
    """examples/llama3_2.rs:95-107 (factor 32, original context 8192, low/high 1/4)."""
    out = []
    for i in range(n_freq):
        inv = math.exp(i * (-math.log(ROPE_THETA) / n_freq))
        wave = 2.0 * math.pi / inv
        smooth = (8192.0 / wave - 1.0) / (4.0 - 1.0)
        scaled = inv / 32.0
        blended = (1.0 - smooth) * scaled + smooth * inv
        out.append(scaled if 8192.0 / 1.0 < wave else (inv if wave < 8192.0 / 4.0 else blended))
    return out


def random_weights(cfg: dict, seed: int, device, w4: bool = False, w4_head: bool | None = None):
    """Random-init weights of the architecture: N(0, 0.02) bf16, norms N(1, 0.1); the int4 variant draws
    integers uniform in [-8, 7] with a positive bf16 scale per 64 inputs. `w4_head` (default: as `w4`) quantises
    the tied embedding / lm_head table the same way ('embed' packed, 'sembed' scales); False keeps it bf16."""
    if w4_head is None:
        w4_head = w4
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    H, F, V = cfg["hidden"], cfg["ffn"], cfg["vocab"]
    Hq, Hkv, D = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]

    def dense(rows, cols):
        return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def norm():
        return (1.0 + 0.1 * torch.randn(H, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)

    def quant(rows, cols):
        q = torch.randint(-8, 8, (rows, cols), generator=g, device=device, dtype=torch.int32)
        u = (q + 8).to(torch.uint8)
        packed = (u[:, 0::2] | (u[:, 1::2] << 4)).contiguous()  # low nibble = even element
        s = 0.02 / 4.6 * (1.0 + 0.25 * torch.rand(rows, cols // 64, generator=g, device=device, dtype=torch.float32))
        return packed, s.to(torch.bfloat16).contiguous()

    w = dict(final_norm=norm(), attn_norm=[], mlp_norm=[])
    if w4_head:
        w["embed"], w["sembed"] = quant(V, H)
    else:
        w["embed"] = dense(V, H)
    shapes = dict(wq=(Hq * D, H), wk=(Hkv * D, H), wv=(Hkv * D, H), wo=(H, Hq * D), wgate=(F, H), wup=(F, H), wdown=(H, F))
    for name in shapes:
        w[name] = []
        if w4:
            w["s" + name[1:]] = []
    for _ in range(cfg["layers"]):
        w["attn_norm"].append(norm())
        w["mlp_norm"].append(norm())
        for name, (r, c) in shapes.items():
            if w4:
                pk, sc = quant(r, c)
                w[name].append(pk)
                w["s" + name[1:]].append(sc)
            else:
                w[name].append(dense(r, c))
    return w


class LlamaMachine:
    """The instantiated step program: owns state buffers, replays one captured graph per step."""

    def __init__(self, dev: CudaDevice, cfg: dict, weights: dict, ctx: int, batch: int, w4: bool = False,
                 capture: bool = True, fused: bool = True, persistent: bool = False):
        self.dev, self.cfg, self.ctx, self.batch, self.w4, self.fused = dev, dict(cfg), ctx, batch, w4, fused
        H, F, V, L = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["layers"]
        Hq, Hkv, D = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
        if H != Hq * D or Hq % Hkv or D not in (64, 128):
            raise CompileError("invalid graph: hidden must equal q_heads*head_dim and head_dim must be 64 or 128")
        if ctx % 8:
            raise CompileError("invalid input declaration: the cache sequence extent must be a multiple of 8")
        td, B = dev.torch_device, batch
        z = lambda shape, dt: torch.zeros(shape, dtype=dt, device=td)
        self.w = weights
        self.tokens = z((B,), torch.int32)
        self.position = z((1,), torch.int32)
        self.x = z((B, H), torch.float32)
        self.xn = z((B, H), torch.bfloat16)
        self.q = z((B, Hq * D), torch.float32)
        self.k = z((B, Hkv * D), torch.float32)
        self.v = z((B, Hkv * D), torch.float32)
        self.qb = z((B, Hq, D), torch.bfloat16)
        self.att = z((B, Hq, D), torch.bfloat16)
        self.h = z((B, F), torch.bfloat16)
        self.logits = z((B, V), torch.float32)
        self.kcache = [z((B, Hkv, ctx, D), torch.bfloat16) for _ in range(L)]   # [kv, seq, hd]
        self.vcache = [z((B, Hkv, D, ctx), torch.bfloat16) for _ in range(L)]   # [kv, hd, seq]
        self.table = dev.rope_table(llama3_inv_freq(D // 2) if cfg.get("llama3_rope", 1) else
                                    [math.exp(i * (-math.log(cfg.get("theta", ROPE_THETA)) / (D // 2))) for i in range(D // 2)],
                                    ctx)
        tiles = (ctx + 63) // 64
        # chunks of the key axis per (batch, kv head): about 64 CTAs in all, and two chunks while the (batch, kv head)
        # pairs alone do not fill the SMs (measured at ctx ~1k: 8 chunks best at batch 1; at batch 16 two chunks give
        # 1.251 ms/step against 1.298 with one and 1.303 with four); at least 2 tiles of 64 keys per chunk
        want = max(-(-64 // (B * Hkv)), 2 if B * Hkv <= 148 else 1)
        self.n_splits = max(1, min(max(1, tiles // 2), want))
        # the machine owns its scratch: two machines stepping on different streams must not share one
        self.partials = z((dev.lib.sanic_attn_decode_scratch_bytes(B, Hq, D, self.n_splits) // 4,), torch.float32)
        self.amax_scratch = z((B * 2 * 256,), torch.float32)
        self.stream = torch.cuda.Stream(device=td)
        self._host_position = 0
        self.persistent = persistent
        self._build()
        self.captured = False
        if capture:
            self.capture()

    # ── stage list ──
    def _gemv(self, x, names, layer, outs, epilogue=abi.EPI_STORE, residual=None, out_dtype=abi.F32, norm=None,
              rope_layer=None):
        ws = [self.w[n][layer] if layer is not None else self.w[n] for n in names]
        if layer is not None:
            sc = [self.w["s" + n[1:]][layer] for n in names] if self.w4 else None
        else:       # the tied table: quantised when it came with scales
            sc = [self.w["s" + n] for n in names] if ws[0].dtype == torch.uint8 else None
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_GEMV
        s.carrier = carrier_contraction(abi.I4 if sc is not None else abi.BF16)
        g = self.dev.gemv_params(x, ws, outs, sc, epilogue, residual, out_dtype)
        if norm is not None:      # the RMSNorm cone of the residual stream is inlined into the fold's leaf
            g.norm_x, g.norm_gamma, g.norm_eps = self.x.data_ptr(), norm.data_ptr(), float(self.cfg.get("eps", 1e-5))
        if rope_layer is not None:
            cfg = self.cfg
            g.rope_table, g.rope_position = self.table.data_ptr(), self.position.data_ptr()
            g.rope_q_out = self.qb.data_ptr()
            g.rope_k_cache, g.rope_v_cache = self.kcache[rope_layer].data_ptr(), self.vcache[rope_layer].data_ptr()
            g.rope_q_heads, g.rope_kv_heads, g.rope_head_dim, g.rope_ctx = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], self.ctx
        s.u.gemv = g
        return s

    def _rmsnorm(self, gamma):
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_RMSNORM
        s.u.rmsnorm.x, s.u.rmsnorm.gamma = self.x.data_ptr(), gamma.data_ptr()
        s.u.rmsnorm.rows, s.u.rmsnorm.n, s.u.rmsnorm.eps = self.batch, self.cfg["hidden"], float(self.cfg.get("eps", 1e-5))
        s.u.rmsnorm.out = self.xn.data_ptr()
        return s

    def _build(self):
        """The launch list. fused=True: 5 launches per layer (norm and RoPE/cache write ride the projections);
        fused=False: one stage per graph cone (9 per layer), kept for comparison and tests."""
        cfg, B = self.cfg, self.batch
        Hq, Hkv, D = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
        fused = self.fused
        # as separate launches, every CTA re-deriving the normalised rows costs more than a launch at larger batch;
        # the single-kernel step derives them once per stage, so it inlines the norm at any batch
        inline_norm = fused and (B <= 4 or self.persistent)
        st = []
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_GATHER, abi.OP_EMBED
        s.u.embed.table, s.u.embed.tokens = self.w["embed"].data_ptr(), self.tokens.data_ptr()
        s.u.embed.batch, s.u.embed.hidden, s.u.embed.vocab = B, cfg["hidden"], cfg["vocab"]
        s.u.embed.out = self.x.data_ptr()
        if self.w["embed"].dtype == torch.uint8:
            s.u.embed.scales, s.u.embed.table_dtype, s.u.embed.group = self.w["sembed"].data_ptr(), abi.I4, 64
        st.append(s)
        for l in range(cfg["layers"]):
            if fused:
                if not inline_norm:
                    st.append(self._rmsnorm(self.w["attn_norm"][l]))
                st.append(self._gemv(self.xn, ["wq", "wk", "wv"], l, [], abi.EPI_ROPE_CACHE,
                                     norm=self.w["attn_norm"][l] if inline_norm else None, rope_layer=l))
            else:
                st.append(self._rmsnorm(self.w["attn_norm"][l]))
                st.append(self._gemv(self.xn, ["wq", "wk", "wv"], l, [self.q, self.k, self.v]))
                s = abi.StageDesc()
                s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_ROPE_CACHE
                r = s.u.rope_cache
                r.q, r.k, r.v = self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr()
                r.q_out, r.k_cache, r.v_cache = self.qb.data_ptr(), self.kcache[l].data_ptr(), self.vcache[l].data_ptr()
                r.table, r.position = self.table.data_ptr(), self.position.data_ptr()
                r.batch, r.q_heads, r.kv_heads, r.head_dim, r.ctx = B, Hq, Hkv, D, self.ctx
                st.append(s)
            s = abi.StageDesc()
            s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_DECODE_ATTN
            s.carrier = carrier_online_softmax(abi.BF16)
            s.u.decode, _ = self.dev.decode_params(self.qb, self.kcache[l], self.vcache[l], 1, v_transposed=True,
                                                   n_splits=self.n_splits, kv_len_dev=self.position, out=self.att,
                                                   partials=self.partials, out_dtype=abi.BF16)
            st.append(s)
            st.append(self._gemv(self.att.view(B, Hq * D), ["wo"], l, [self.x], abi.EPI_RESIDUAL_ADD, self.x))
            if inline_norm:
                st.append(self._gemv(self.xn, ["wgate", "wup"], l, [self.h], abi.EPI_SILU_MUL, None, abi.BF16,
                                     norm=self.w["mlp_norm"][l]))
            else:
                st.append(self._rmsnorm(self.w["mlp_norm"][l]))
                st.append(self._gemv(self.xn, ["wgate", "wup"], l, [self.h], abi.EPI_SILU_MUL, None, abi.BF16))
            st.append(self._gemv(self.h, ["wdown"], l, [self.x], abi.EPI_RESIDUAL_ADD, self.x))
        if inline_norm:
            st.append(self._gemv(self.xn, ["embed"], None, [self.logits], norm=self.w["final_norm"]))
        else:
            st.append(self._rmsnorm(self.w["final_norm"]))
            st.append(self._gemv(self.xn, ["embed"], None, [self.logits]))
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_ARGMAX
        s.carrier = carrier_extremum_index()
        s.u.argmax.x, s.u.argmax.rows, s.u.argmax.n = self.logits.data_ptr(), B, cfg["vocab"]
        s.u.argmax.out, s.u.argmax.scratch = self.tokens.data_ptr(), self.amax_scratch.data_ptr()
        st.append(s)
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_ADVANCE
        s.u.advance.position = self.position.data_ptr()
        st.append(s)
        arr = (abi.StageDesc * len(st))(*st)
        h = C.c_void_p()
        self.dev._check(self.dev.lib.sanic_program_create(self.dev.h, arr, len(st), C.byref(h)), "program_create")
        self.prog = h
        self.n_stages = len(st)
        self.kernel_count = int(self.dev.lib.sanic_program_kernel_count(h))

    def capture(self):
        torch.cuda.synchronize(self.dev.torch_device)
        fn = self.dev.lib.sanic_program_capture_persistent if self.persistent else self.dev.lib.sanic_program_capture
        rc = fn(self.prog, C.c_void_p(self.stream.cuda_stream))
        self.dev._check(rc, "program_capture")
        self.captured = True
        self.kernel_count = int(self.dev.lib.sanic_program_kernel_count(self.prog))   # kernels one replay starts

    # ── Machine::step ──
    def set_state(self, tokens, position: int):
        if position < 0 or position >= self.ctx:
            raise RunError(f"position {position} is outside the cache extent {self.ctx}")
        # steps are asynchronous on the machine's own stream: a step still in flight would write its token and its
        # advanced position AFTER the values set here
        self.sync()
        self.tokens.copy_(torch.as_tensor(tokens, dtype=torch.int32).to(self.dev.torch_device))
        self.position.fill_(position)
        self._host_position = int(position)
        torch.cuda.synchronize(self.dev.torch_device)

    def step(self, timed: bool = False):
        """One decode step: token <- argmax(logits(token, position)); position += 1. Returns device seconds if timed."""
        # the position lives on the device; the host keeps its own count so that a step whose cache row would fall
        # outside the cache is refused here instead of being clamped (and reported) by the kernels
        if self._host_position >= self.ctx:
            raise RunError(f"step: position {self._host_position} is outside the cache extent {self.ctx}")
        self._host_position += 1
        st = C.c_void_p(self.stream.cuda_stream)
        if self.captured:
            sec = C.c_double(0.0)
            rc = self.dev.lib.sanic_program_step(self.prog, st, C.byref(sec) if timed else None)
            self.dev._check(rc, "program_step")
            return sec.value if timed else None
        self.dev._check(self.dev.lib.sanic_program_run(self.prog, st), "program_run")
        return None

    def step_stage_times(self):
        """One decode step with a device time per stage (MetalDevice::run_kernel_timed): list of seconds."""
        if self._host_position >= self.ctx:
            raise RunError(f"step: position {self._host_position} is outside the cache extent {self.ctx}")
        self._host_position += 1
        st = C.c_void_p(self.stream.cuda_stream)
        cap = 4 * self.n_stages + 8
        buf = (C.c_double * cap)()
        n = C.c_int32(0)
        self.dev._check(self.dev.lib.sanic_program_stage_times(self.prog, st, buf, cap, C.byref(n)), "program_stage_times")
        return [buf[i] for i in range(n.value)]

    def generate(self, prompts, new_tokens: int):
        """Greedy decoding (the loop of examples/llama3_2.rs:577-664): `prompts` is one equal-length list of token ids per
        batch row. The prompt is consumed one position per step through the same decode step (decode equals prefill,
        tests/decode.rs:121-204: the model's prediction is simply replaced by the next prompt token), then `new_tokens`
        steps run back to back on the device, each feeding its argmax to the next with no host round trip.
        Returns an int array [batch, new_tokens]."""
        import numpy as np
        prompts = np.asarray(prompts, dtype=np.int32)
        if prompts.ndim != 2 or prompts.shape[0] != self.batch or prompts.shape[1] < 1:
            raise RunError("generate: one equal-length, non-empty prompt per batch row")
        n = prompts.shape[1]
        if n + new_tokens > self.ctx:
            raise RunError(f"generate: {n} prompt + {new_tokens} new tokens exceed the cache extent {self.ctx}")
        for pos in range(n - 1):
            self.set_state(prompts[:, pos], pos)
            self.step()
        self.set_state(prompts[:, n - 1], n - 1)
        out = np.zeros((self.batch, new_tokens), dtype=np.int32)
        history = torch.empty(new_tokens, self.batch, dtype=torch.int32, device=self.dev.torch_device)
        with torch.cuda.stream(self.stream):
            for i in range(new_tokens):
                self.step()
                history[i].copy_(self.tokens, non_blocking=True)      # same stream: ordered after the step that wrote it
        self.sync()
        out[:] = history.cpu().numpy().T
        return out

    def sync(self):
        """Wait for the steps in flight and surface the device status word: a step whose bounded wait ran out, or
        whose position ran past the cache, left partial writes, and a decode loop must not continue on them
        (src/metal.rs:686-705 returns Err for the same reason). Raises RunError."""
        self.dev._check(self.dev.lib.sanic_sync(self.dev.h, C.c_void_p(self.stream.cuda_stream)), "machine sync")

    def read_tokens(self):
        self.sync()
        return self.tokens.cpu().numpy().copy()

    def load_caches(self, k_list, v_list):
        self.sync()      # a step in flight still writes its cache row
        for l in range(self.cfg["layers"]):
            self.kcache[l].copy_(k_list[l])
            self.vcache[l].copy_(v_list[l])
        torch.cuda.synchronize(self.dev.torch_device)

    def weight_bytes(self) -> int:
        n = 0
        for key, val in self.w.items():
            for t in (val if isinstance(val, list) else [val]):
                n += t.numel() * t.element_size()
        return n

    def __del__(self):
        try:
            self.dev.lib.sanic_program_destroy(self.prog)
        except Exception:
            pass
