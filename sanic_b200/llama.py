"""Llama-3.2-1B-architecture decode step as a schedule over named buffers, instantiated as a machine.

The decode graph of examples/llama3_2.rs:112-253 of the reference project, with a leading batch axis and a
shared scalar position, is written down the way the reference's emitter hands a step to its runtime: a buffer
table (weights under their checkpoint names, states, intermediates), an ordered stage list (Fused / Elementwise /
Gather, src/partition.rs:44-98) whose pointer fields name table buffers, the roots (state successors first,
src/graph.rs:164-177) and which roots were compiled in place. `Graph::compile_for` -> `StepProgram::instantiate`
-> `Machine::step` (src/graph.rs:231-356) are then the generic `sanic_b200.schedule` calls: the machine
allocates the states (KV caches, token, position) zero-filled, binds the weights by name, wires every state's
successor to the next step's input, and a step is one CUDA-graph replay with no host writes.

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
from .checkpoint import _LAYER
from .schedule import ScheduleBuilder, view_tensor

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


def weight_bindings(cfg: dict, w: dict) -> dict:
    """The weight dictionary under the graph's input names (the checkpoint's tensor names; int4 scales under
    `<name>.scales`)."""
    out = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["final_norm"]}
    if "sembed" in w:
        out["model.embed_tokens.weight.scales"] = w["sembed"]
    for l in range(cfg["layers"]):
        for key, suffix in _LAYER.items():
            out[f"model.layers.{l}.{suffix}"] = w[key][l]
            if key.startswith("w") and ("s" + key[1:]) in w:
                out[f"model.layers.{l}.{suffix}.scales"] = w["s" + key[1:]][l]
    return out


class LlamaMachine:
    """The decode step as a machine: owns the state buffers, replays one captured step per call."""

    def __init__(self, dev: CudaDevice, cfg: dict, weights: dict, ctx: int, batch: int, w4: bool = False,
                 capture: bool = True, fused: bool = True, persistent: bool = False, deferred_norm: bool | None = None):
        self.dev, self.cfg, self.ctx, self.batch, self.w4, self.fused = dev, dict(cfg), ctx, batch, w4, fused
        # deferred normaliser (fused stage lists only): every RMSNorm whose input a residual-add produces is split into
        # what that epilogue can do (multiply by gamma, per-tile sums of squares) and one multiply in the next contraction's
        # epilogue; stored(bf16) then sits on x * gamma (the defer-div carrier of the reference's laws) instead of on the
        # normalised value. Layer 0's attention norm, fed by the gather, is unchanged. Default: on for the launch list (at
        # batch > 4 the norm would otherwise be a launch of its own: 86 launches per step instead of 118, 1.10 against 1.23 ms
        # at batch 16; at batch 1, where it would be inlined into the contractions' activation loads, 0.872 against 0.945 ms
        # with bf16 weights and 0.710 against 0.738 with int4); the single-kernel step keeps the norm inlined into its
        # staging pass, which measured faster there (0.875 against 0.935 ms: the scale's loads would sit in front of the
        # staging loads).
        if deferred_norm is None:
            deferred_norm = fused and not persistent
        self.deferred_norm = bool(deferred_norm and fused)
        H, Hq, Hkv, D = cfg["hidden"], cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
        if H != Hq * D or Hq % Hkv or D not in (64, 128):
            raise CompileError("invalid graph: hidden must equal q_heads*head_dim and head_dim must be 64 or 128")
        if ctx % 8:
            raise CompileError("invalid input declaration: the cache sequence extent must be a multiple of 8")
        self.w = weights
        self.table = dev.rope_table(llama3_inv_freq(D // 2) if cfg.get("llama3_rope", 1) else
                                    [math.exp(i * (-math.log(cfg.get("theta", ROPE_THETA)) / (D // 2))) for i in range(D // 2)],
                                    ctx)
        tiles = (ctx + 63) // 64
        # chunks of the key axis per (batch, kv head): about 64 CTAs in all, and two chunks while the (batch, kv head)
        # pairs alone do not fill the SMs (measured at ctx ~1k: 8 chunks best at batch 1; at batch 16 two chunks give
        # 1.251 ms/step against 1.298 with one and 1.303 with four); at least 2 tiles of 64 keys per chunk
        want = max(-(-64 // (batch * Hkv)), 2 if batch * Hkv <= 148 else 1)
        self.n_splits = max(1, min(max(1, tiles // 2), want))
        self.stream = torch.cuda.Stream(device=dev.torch_device)
        self._host_position = 0
        self.persistent = persistent
        self.captured = bool(capture)
        self._build()
        self._instantiate()

    # ── the schedule: buffer table, stages, roots ──
    def _names(self, l, key):
        name = f"model.layers.{l}.{_LAYER[key]}" if l is not None else {"embed": "model.embed_tokens.weight"}[key]
        return name

    def _gemv(self, b, x, keys, layer, outs, K, rows, epilogue=abi.EPI_STORE, residual=None, out_dtype=abi.F32, norm=None,
              rope_layer=None, next_norm=None, scaled=False):
        """One contraction stage: activations `x` against the weight matrices `keys` of `layer` (None: the tied table).
        `next_norm` (a residual-add stage): also write bf16(y * gamma) and the per-tile sums of y^2 for the next normed
        contraction; `scaled`: this stage's activations are such a bf16(y * gamma) and its outputs take the deferred
        1/sqrt(mean + eps)."""
        names = [self._names(layer, k) for k in keys]
        quant = self.w[keys[0]][layer].dtype == torch.uint8 if layer is not None else self.w["embed"].dtype == torch.uint8
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_GEMV
        s.carrier = carrier_contraction(abi.I4 if quant else abi.BF16)
        g = s.u.gemv
        g.batch, g.K, g.weight_dtype, g.group, g.n_segments = self.batch, K, (abi.I4 if quant else abi.BF16), 64, len(keys)
        refs = {}
        for i, n in enumerate(names):
            g.rows[i] = rows[i]
            refs[f"gemv.w[{i}]"] = n
            if quant:
                refs[f"gemv.scales[{i}]"] = n + ".scales"
        for i, o in enumerate(outs):
            refs[f"gemv.out[{i}]"] = o
        g.out_dtype, g.epilogue = out_dtype, epilogue
        if residual is not None:
            refs["gemv.residual"] = residual
        if norm is not None:      # the RMSNorm cone of the residual stream is inlined into the fold's leaf
            refs["gemv.norm_x"], refs["gemv.norm_gamma"] = "x", norm
            g.norm_eps = float(self.cfg.get("eps", 1e-5))
        else:
            refs["gemv.x"] = x
        if next_norm is not None:
            refs["gemv.nx_out"], refs["gemv.nx_gamma"], refs["gemv.nx_partial"] = "xn", next_norm, "xn.partial"
        if scaled:
            refs["gemv.ds_partial"] = "xn.partial"
            g.ds_tiles, g.ds_eps = K // 16, float(self.cfg.get("eps", 1e-5))
        if rope_layer is not None:
            cfg = self.cfg
            refs["gemv.rope_table"], refs["gemv.rope_position"], refs["gemv.rope_q_out"] = "rope_table", "position", "q_rope"
            refs["gemv.rope_k_cache"], refs["gemv.rope_v_cache"] = f"cache.{rope_layer}.key.next", f"cache.{rope_layer}.value.next"
            g.rope_q_heads, g.rope_kv_heads, g.rope_head_dim, g.rope_ctx = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], self.ctx
        b.stage(s, refs)

    def _rmsnorm(self, b, gamma):
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_RMSNORM
        s.u.rmsnorm.rows, s.u.rmsnorm.n, s.u.rmsnorm.eps = self.batch, self.cfg["hidden"], float(self.cfg.get("eps", 1e-5))
        b.stage(s, {"rmsnorm.x": "x", "rmsnorm.gamma": gamma, "rmsnorm.out": "xn"})

    def _build(self):
        """fused=True: 5 stages per layer (norm and RoPE/cache write ride the projections); fused=False: one stage per
        graph cone (8 per layer), kept for comparison and tests."""
        cfg, B, dev = self.cfg, self.batch, self.dev
        H, F, V, L = cfg["hidden"], cfg["ffn"], cfg["vocab"], cfg["layers"]
        Hq, Hkv, D, ctx = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], self.ctx
        fused = self.fused
        # as separate launches, every CTA re-deriving the normalised rows costs more than a launch at larger batch;
        # the single-kernel step derives them once per stage, so it inlines the norm at any batch
        inline_norm = fused and (B <= 4 or self.persistent)
        b = ScheduleBuilder()
        # inputs: the weights under their checkpoint names, the RoPE table, and the states
        self.bindings = weight_bindings(cfg, self.w)
        for name, t in self.bindings.items():
            shape = tuple(t.shape)
            if t.dtype == torch.uint8:
                shape = shape[:-1] + (shape[-1] * 2,)      # declared in elements, stored two per byte
            b.input(name, abi.dtype_of_torch(t.dtype), shape)
        b.input("rope_table", abi.F32, tuple(self.table.shape))
        self.bindings["rope_table"] = self.table
        b.input("tokens", abi.U32, (B,))
        b.input("position", abi.U32, (1,))
        for l in range(L):
            b.input(f"cache.{l}.key", abi.BF16, (B, Hkv, ctx, D))      # [kv, seq, hd]
            b.input(f"cache.{l}.value", abi.BF16, (B, Hkv, D, ctx))    # [kv, hd, seq]
        # state successors: every one of them overwrites its predecessor (the cache row write is the conditional store
        # of where(coord == position, new, cache); token and position are read before they are written within a step)
        for l in range(L):
            b.scratch(f"cache.{l}.key.next", abi.BF16, (B, Hkv, ctx, D))
            b.scratch(f"cache.{l}.value.next", abi.BF16, (B, Hkv, D, ctx))
        b.scratch("tokens.next", abi.U32, (B,))
        b.scratch("position.next", abi.U32, (1,))
        # intermediates
        b.scratch("x", abi.F32, (B, H))
        b.scratch("xn", abi.BF16, (B, H))
        b.scratch("xn.partial", abi.F32, (B, H // 16))
        if not fused:
            b.scratch("q", abi.F32, (B, Hq * D)); b.scratch("k", abi.F32, (B, Hkv * D)); b.scratch("v", abi.F32, (B, Hkv * D))
        b.scratch("q_rope", abi.BF16, (B, Hq, D))
        b.scratch("attended", abi.BF16, (B, Hq, D))
        b.scratch("h", abi.BF16, (B, F))
        b.scratch("logits", abi.F32, (B, V))
        b.scratch("attn.partials", abi.F32, (dev.lib.sanic_attn_decode_scratch_bytes(B, Hq, D, self.n_splits) // 4,))
        b.scratch("argmax.scratch", abi.F32, (B * 2 * 256,))

        quant_table = self.w["embed"].dtype == torch.uint8
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_GATHER, abi.OP_EMBED
        s.u.embed.batch, s.u.embed.hidden, s.u.embed.vocab = B, H, V
        refs = {"embed.table": "model.embed_tokens.weight", "embed.tokens": "tokens", "embed.out": "x"}
        if quant_table:
            s.u.embed.table_dtype, s.u.embed.group = abi.I4, 64
            refs["embed.scales"] = "model.embed_tokens.weight.scales"
        b.stage(s, refs)
        qkv_rows = [Hq * D, Hkv * D, Hkv * D]
        for l in range(L):
            attn_norm, mlp_norm = self._names(l, "attn_norm"), self._names(l, "mlp_norm")
            defer = self.deferred_norm
            if fused and defer and l > 0:
                self._gemv(b, "xn", ["wq", "wk", "wv"], l, [], H, qkv_rows, abi.EPI_ROPE_CACHE, rope_layer=l, scaled=True)
            elif fused:
                if not inline_norm:
                    self._rmsnorm(b, attn_norm)
                self._gemv(b, "xn", ["wq", "wk", "wv"], l, [], H, qkv_rows, abi.EPI_ROPE_CACHE,
                           norm=attn_norm if inline_norm else None, rope_layer=l)
            else:
                self._rmsnorm(b, attn_norm)
                self._gemv(b, "xn", ["wq", "wk", "wv"], l, ["q", "k", "v"], H, qkv_rows)
                s = abi.StageDesc()
                s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_ROPE_CACHE
                r = s.u.rope_cache
                r.batch, r.q_heads, r.kv_heads, r.head_dim, r.ctx = B, Hq, Hkv, D, ctx
                b.stage(s, {"rope_cache.q": "q", "rope_cache.k": "k", "rope_cache.v": "v", "rope_cache.q_out": "q_rope",
                            "rope_cache.k_cache": f"cache.{l}.key.next", "rope_cache.v_cache": f"cache.{l}.value.next",
                            "rope_cache.table": "rope_table", "rope_cache.position": "position"})
            s = abi.StageDesc()
            s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_DECODE_ATTN
            s.carrier = carrier_online_softmax(abi.BF16)
            p = s.u.decode
            p.k_batch_stride, p.k_head_stride, p.k_seq_stride = Hkv * ctx * D, ctx * D, D
            p.v_batch_stride, p.v_head_stride, p.v_row_stride = Hkv * D * ctx, D * ctx, ctx
            p.v_transposed, p.batch, p.q_heads, p.kv_heads, p.head_dim = 1, B, Hq, Hkv, D
            p.kv_len, p.window, p.n_splits, p.scale = 1, 0, self.n_splits, 1.0 / math.sqrt(D)
            p.out_dtype, p.kv_cap = abi.BF16, ctx
            b.stage(s, {"decode.q": "q_rope", "decode.k": f"cache.{l}.key.next", "decode.v": f"cache.{l}.value.next",
                        "decode.kv_len_dev": "position", "decode.partials": "attn.partials", "decode.out": "attended"})
            if defer:
                after = self._names(l + 1, "attn_norm") if l + 1 < L else "model.norm.weight"
                self._gemv(b, "attended", ["wo"], l, ["x"], Hq * D, [H], abi.EPI_RESIDUAL_ADD, "x", next_norm=mlp_norm)
                self._gemv(b, "xn", ["wgate", "wup"], l, ["h"], H, [F, F], abi.EPI_SILU_MUL, None, abi.BF16, scaled=True)
                self._gemv(b, "h", ["wdown"], l, ["x"], F, [H], abi.EPI_RESIDUAL_ADD, "x", next_norm=after)
                continue
            self._gemv(b, "attended", ["wo"], l, ["x"], Hq * D, [H], abi.EPI_RESIDUAL_ADD, "x")
            if inline_norm:
                self._gemv(b, "xn", ["wgate", "wup"], l, ["h"], H, [F, F], abi.EPI_SILU_MUL, None, abi.BF16, norm=mlp_norm)
            else:
                self._rmsnorm(b, mlp_norm)
                self._gemv(b, "xn", ["wgate", "wup"], l, ["h"], H, [F, F], abi.EPI_SILU_MUL, None, abi.BF16)
            self._gemv(b, "h", ["wdown"], l, ["x"], F, [H], abi.EPI_RESIDUAL_ADD, "x")
        if self.deferred_norm:
            self._gemv(b, "xn", ["embed"], None, ["logits"], H, [V], scaled=True)
        elif inline_norm:
            self._gemv(b, "xn", ["embed"], None, ["logits"], H, [V], norm="model.norm.weight")
        else:
            self._rmsnorm(b, "model.norm.weight")
            self._gemv(b, "xn", ["embed"], None, ["logits"], H, [V])
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_ARGMAX
        s.carrier = carrier_extremum_index()
        s.u.argmax.rows, s.u.argmax.n = B, V
        b.stage(s, {"argmax.x": "logits", "argmax.out": "tokens.next", "argmax.scratch": "argmax.scratch"})
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_ELEMENTWISE, abi.OP_ADVANCE
        b.stage(s, {"advance.position": "position.next"})
        # roots: state successors first (src/graph.rs:164-177), then the outputs
        self.state_roots = []
        for l in range(L):
            self.state_roots.append((f"cache.{l}.key", b.root(f"cache.{l}.key.next", in_place_of=f"cache.{l}.key")))
            self.state_roots.append((f"cache.{l}.value", b.root(f"cache.{l}.value.next", in_place_of=f"cache.{l}.value")))
        self.token_root = b.root("tokens.next", in_place_of="tokens")
        self.state_roots.append(("tokens", self.token_root, 1))          # indices are exact or wrong: pinned at u32
        self.state_roots.append(("position", b.root("position.next", in_place_of="position"), 1))
        self.logits_root = b.root("logits")
        self.n_stages = len(b.stages)
        self.prog = b.compile(dev)

    def _instantiate(self):
        td, L = self.dev.torch_device, self.cfg["layers"]
        torch.cuda.synchronize(td)
        st = C.c_void_p(self.stream.cuda_stream)
        if self.captured:
            self.machine = self.prog.instantiate(self.state_roots, self.bindings, abi.BF16,
                                                 outputs=[("token", self.token_root), ("logits", self.logits_root)],
                                                 persistent=self.persistent, stream=st)
            state = lambda name: view_tensor(self.machine.state(name), td)
            self.kernel_count = self.machine.kernel_count       # kernels one replay starts
            self.logits = view_tensor(self.machine.output("logits"), td)
            self._states = None
        else:
            # no frozen step: every step is a run of the schedule with the states bound like any other input
            # (Program::try_run); the in-place roots still write their predecessors' buffers
            z = lambda d: torch.zeros(d[3], dtype={abi.BF16: torch.bfloat16, abi.U32: torch.int32}[d[2]], device=td)
            decl = {d[0]: d for d in self.prog.buffer_decls}
            self._states = {name: z(decl[name]) for name, *_ in self.state_roots}
            state = lambda name: self._states[name]
            self.machine = None
            self.kernel_count = self.n_stages + 1
            outs = self.prog.try_run(dict(self.bindings, **self._states), stream=st)     # also allocates the scratch
            self.stream.synchronize()
            for t in self._states.values():
                t.zero_()
            self.logits = view_tensor(outs[self.logits_root], td)
        self.kcache = [state(f"cache.{l}.key") for l in range(L)]
        self.vcache = [state(f"cache.{l}.value") for l in range(L)]
        self.tokens, self.position = state("tokens"), state("position")

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

    def _guard(self):
        # the position lives on the device; the host keeps its own count so that a step whose cache row would fall
        # outside the cache is refused here instead of being clamped (and reported) by the kernels
        if self._host_position >= self.ctx:
            raise RunError(f"step: position {self._host_position} is outside the cache extent {self.ctx}")
        self._host_position += 1

    def step(self, timed: bool = False):
        """One decode step: token <- argmax(logits(token, position)); position += 1. Returns device seconds if timed."""
        self._guard()
        st = C.c_void_p(self.stream.cuda_stream)
        if self.machine is not None:
            return self.machine.step(stream=st, timed=timed)
        self.prog.try_run(dict(self.bindings, **self._states), stream=st)
        return None

    def step_stage_times(self):
        """One decode step with a device time per stage (MetalDevice::run_kernel_timed): list of seconds."""
        if self.machine is None:
            raise RunError("step_stage_times needs a captured machine")
        self._guard()
        return self.machine.stage_times(stream=C.c_void_p(self.stream.cuda_stream), cap=4 * self.n_stages + 8)

    def step_phase_profile(self):
        """One decode step of the single-kernel form with four clock stamps per phase (see Replay.phase_profile)."""
        if self.machine is None or not self.persistent:
            raise RunError("step_phase_profile needs a machine captured in its single-kernel form")
        self._guard()
        return self.machine.phase_profile(stream=C.c_void_p(self.stream.cuda_stream), cap=4 * self.n_stages + 8)

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

    def close(self):
        if getattr(self, "machine", None) is not None:
            self.machine.close()
            self.machine = None
        if getattr(self, "prog", None) is not None:
            self.prog.close()
            self.prog = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
