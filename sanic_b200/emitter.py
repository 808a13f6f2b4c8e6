"""Host side of the generic emitter: carriers as expression programs -> generated CUDA kernels.

A carrier here is the reference's own (src/derive.rs:262-287 of the reference project): `leaves` (the
per-element inputs of the fold), `into` (lift one element), `combine` (the associative merge over two
accumulators), `identity`, `project`. Expressions are trees over the closed scalar basis
(src/scalar.rs:45-69; Expr, src/derive.rs:96-118), built with the operators and functions of this
module and flattened to the postfix programs of the C ABI. The generated kernel is the fallback for
carriers no specialised kernel matches (scalar fold / cooperative fold) and the pointwise kernel for
elementwise cones (src/emit_metal.rs:626-1178).

Nothing here computes: `Description` only packs a descriptor, `source` and `compiles` render and compile
without a device, `GenericKernel` compiles, loads and launches through libsanic_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Sequence

from . import _abi as abi


class E:
    """An expression node. Build with the helpers below; Python operators map onto the scalar basis."""
    __slots__ = ("op", "arg", "value", "kids")

    def __init__(self, op, arg=0, value=0.0, kids=()):
        self.op, self.arg, self.value, self.kids = op, arg, float(value), tuple(kids)

    @staticmethod
    def of(x) -> "E":
        return x if isinstance(x, E) else const(x)

    def __add__(self, o): return E(abi.X_ADD, kids=(self, E.of(o)))
    def __radd__(self, o): return E(abi.X_ADD, kids=(E.of(o), self))
    def __sub__(self, o): return E(abi.X_SUB, kids=(self, E.of(o)))
    def __rsub__(self, o): return E(abi.X_SUB, kids=(E.of(o), self))
    def __mul__(self, o): return E(abi.X_MUL, kids=(self, E.of(o)))
    def __rmul__(self, o): return E(abi.X_MUL, kids=(E.of(o), self))
    def __truediv__(self, o): return E(abi.X_DIV, kids=(self, E.of(o)))
    def __rtruediv__(self, o): return E(abi.X_DIV, kids=(E.of(o), self))
    def __neg__(self): return E(abi.X_NEG, kids=(self,))
    def __lt__(self, o): return E(abi.X_LT, kids=(self, E.of(o)))      # 1.0 / 0.0
    def __gt__(self, o): return E(abi.X_LT, kids=(E.of(o), self))

    def flatten(self, out: list):
        for k in self.kids:
            k.flatten(out)
        out.append((self.op, self.arg, self.value))


def const(v) -> E: return E(abi.X_CONST, value=v)
def load(operand: int) -> E: return E(abi.X_LOAD, arg=operand)
def coord(axis: int) -> E: return E(abi.X_COORD, arg=axis)
def gather(operand: int, index) -> E: return E(abi.X_GATHER, arg=operand, kids=(E.of(index),))
def gather_pad(operand: int, index) -> E: return E(abi.X_GATHER_PAD, arg=operand, kids=(E.of(index),))   # out of range reads 0
def item(i: int) -> E: return E(abi.X_ITEM, arg=i)
def A(i: int) -> E: return E(abi.X_A, arg=i)
def B(i: int) -> E: return E(abi.X_B, arg=i)
def F(i: int) -> E: return E(abi.X_F, arg=i)
def result() -> E: return E(abi.X_RESULT)
def maximum(a, b) -> E: return E(abi.X_MAX, kids=(E.of(a), E.of(b)))
def minimum(a, b) -> E: return E(abi.X_MIN, kids=(E.of(a), E.of(b)))
def recip(a) -> E: return E(abi.X_RECIP, kids=(E.of(a),))
def exp(a) -> E: return E(abi.X_EXP, kids=(E.of(a),))
def log(a) -> E: return E(abi.X_LOG, kids=(E.of(a),))
def sqrt(a) -> E: return E(abi.X_SQRT, kids=(E.of(a),))
def tanh(a) -> E: return E(abi.X_TANH, kids=(E.of(a),))
def sin(a) -> E: return E(abi.X_SIN, kids=(E.of(a),))
def cos(a) -> E: return E(abi.X_COS, kids=(E.of(a),))
def where(c, a, b) -> E: return E(abi.X_WHERE, kids=(E.of(c), E.of(a), E.of(b)))
def round_to(a, dtype: int) -> E: return E(abi.X_ROUND, arg=dtype, kids=(E.of(a),))


@dataclass
class Operand:
    """A typed, strided view of one bound buffer: element index = offset + sum(coord * stride) + s * stream_stride."""
    buffer: int
    dtype: int
    strides: Sequence[int]
    stream_stride: int = 0
    offset: int = 0
    inner_stride: int = 0      # for a contracted leaf: elements per step of its inner axis
    gather_stride: int = 0     # for `gather`: elements per step of the gathered index, and the number of valid indices
    gather_extent: int = 0
    stream_strides: Sequence[int] = ()   # with a streamed window of several axes: elements per step of each window axis


@dataclass
class Carrier:
    """leaves / into / combine / identity / project, as in the reference's `Carrier`."""
    leaves: Sequence[E]
    into: Sequence[E]
    combine: Sequence[E]
    identity: Sequence[float]
    project: E
    leaf_inner: Sequence[int] = ()     # per leaf: an extent R > 1 makes the leaf the sum over r < R of its expression


# ── the carriers the reference's laws pin (tests/laws.rs:107-126,620-646; tests/compile.rs:139-171) ──
def carrier_sum(leaf: E) -> Carrier:
    return Carrier([leaf], [item(0)], [A(0) + B(0)], [0.0], F(0))


def carrier_max(leaf: E) -> Carrier:
    return Carrier([leaf], [item(0)], [maximum(A(0), B(0))], [float("-inf")], F(0))


def _shift(side, m):
    """exp(side - m), forced to 0 when the side's maximum is -inf (src/derive.rs:1700-1713)."""
    return where(const(float("-inf")) < side, exp(side - m), 0.0)


def carrier_online_softmax(score: E, value: E, contraction: int = 0, post: "callable | None" = None) -> Carrier:
    """(m, l, o): Plain(Max), ExpShifted{0}, ExpShifted{0}; project o / l. With `contraction` = E > 1 the score leaf is
    the sum of `score` over an inner axis of that extent, computed in the fold body; `post` maps the contracted leaf to
    the score that is lifted (scale, additive mask)."""
    m = maximum(A(0), B(0))
    s = item(0) if post is None else post(item(0))
    return Carrier([score, value], [s, const(1.0), item(1)],
                   [m, A(1) * _shift(A(0), m) + B(1) * _shift(B(0), m), A(2) * _shift(A(0), m) + B(2) * _shift(B(0), m)],
                   [float("-inf"), 0.0, 0.0], F(2) / F(1), leaf_inner=(contraction, 0) if contraction > 1 else ())


def carrier_logsumexp(leaf: E) -> Carrier:
    m = maximum(A(0), B(0))
    return Carrier([leaf], [item(0), const(1.0)], [m, A(1) * _shift(A(0), m) + B(1) * _shift(B(0), m)],
                   [float("-inf"), 0.0], F(0) + log(F(1)))


def carrier_deferred_norm(x: E, gamma_w: E, n: int, eps: float) -> Carrier:
    """2 x Plain(Add): sum x^2 and sum x*gamma*w; project dot / sqrt(sum x^2 / n + eps) (defer-div)."""
    return Carrier([x, gamma_w], [item(0) * item(0), item(0) * item(1)], [A(0) + B(0), A(1) + B(1)], [0.0, 0.0],
                   F(1) / sqrt(F(0) * (1.0 / n) + eps))


def carrier_first_argmax(leaf: E, index: E) -> Carrier:
    """(Plain(Max), AtExtremum{key 0, Max, ties Min}): the first maximal index (src/ir.rs:1415-1433)."""
    key = maximum(A(0), B(0))
    idx = where(A(0) < B(0), B(1), where(B(0) < A(0), A(1), minimum(A(1), B(1))))
    return Carrier([leaf, index], [item(0), item(1)], [key, idx], [float("-inf"), float("inf")], F(1))


def attention(batch, q_heads, kv_heads, q_len, kv_len, head_dim, v_dim, scale, dtype=abi.F32, causal=False):
    """softmax(Q K^T * scale [+ causal mask]) V as ONE fused stage that reads only Q, K and V (the shape the reference's
    partitioner pins, src/partition.rs:2491-2513): grid (batch, kv head, repeat, query, value feature), stream = key, the
    QK^T contraction over head_dim computed in the fold body. Grouped-query attention is the reindex-expand of the kv
    heads: the repeat axis has stride 0 in K and V (src/nn.rs:107-151). The computed mask is where(i < j, -1e30, 0)
    (src/ir.rs:1511-1526). Returns (grid, stream, operands, carrier); buffers are Q [B,Hq,L,E], K [B,Hkv,S,E], V [B,Hkv,S,Ev]."""
    rep = q_heads // kv_heads
    L, S, E, Ev = q_len, kv_len, head_dim, v_dim
    q = Operand(0, dtype, [q_heads * L * E, rep * L * E, L * E, E, 0], 0, inner_stride=1)
    k = Operand(1, dtype, [kv_heads * S * E, S * E, 0, 0, 0], E, inner_stride=1)
    v = Operand(2, dtype, [kv_heads * S * Ev, S * Ev, 0, 0, 1], Ev)

    def post(x):
        x = x * scale
        return x + where(coord(3) < coord(5), -1e30, 0.0) if causal else x
    car = carrier_online_softmax(load(0) * load(1), load(2), contraction=E, post=post)
    return (batch, kv_heads, rep, L, Ev), S, [q, k, v], car


def conv2d(batch, channels, height, width, out_channels, kh, kw, stride=1, dilation=1, padding=0, dtype=abi.F32):
    """y[n, co, oy, ox] = sum over (ci, ky, kx) of x[n, ci, oy*stride + ky*dilation - padding, ox*stride + kx*dilation - padding]
    * w[co, ci, ky, kx], taps outside the input reading 0: the convolution as the reference states it, a (padded) window view of
    x times a broadcast view of w reduced over three axes at once (no patch matrix is materialised: an implicit GEMM whose K axis
    is the window). Returns (grid, window, operands, carrier); buffers are x [N,C,H,W] and w [CO,C,KH,KW]."""
    oh = (height + 2 * padding - dilation * (kh - 1) - 1) // stride + 1
    ow = (width + 2 * padding - dilation * (kw - 1) - 1) // stride + 1
    if oh <= 0 or ow <= 0:
        raise ValueError("the window does not fit the input")
    w = Operand(1, dtype, [0, channels * kh * kw, 0, 0], stream_strides=[kh * kw, kw, 1])
    grid, window = (batch, out_channels, oh, ow), (channels, kh, kw)
    if padding == 0:
        x = Operand(0, dtype, [channels * height * width, 0, stride * width, stride],
                    stream_strides=[height * width, dilation * width, dilation])
        return grid, window, [x, w], carrier_sum(load(0) * load(1))
    # padded: the tap's position inside the image plane is computed from the output and window coordinates and read through
    # a padded gather; a tap whose row or column falls outside reads 0 whatever element its flat index happens to name
    x = Operand(0, dtype, [channels * height * width, 0, 0, 0], stream_strides=[height * width, 0, 0],
                gather_stride=1, gather_extent=height * width)
    iy = coord(2) * float(stride) + coord(len(grid) + 3) * float(dilation) - float(padding)
    ix = coord(3) * float(stride) + coord(len(grid) + 4) * float(dilation) - float(padding)
    inside = (const(-1.0) < iy) * (iy < float(height)) * (const(-1.0) < ix) * (ix < float(width))
    tap = where(inside, gather_pad(0, iy * float(width) + ix), 0.0)
    return grid, window, [x, w], carrier_sum(tap * load(1))


def pool2d(batch, channels, height, width, kh, kw, stride=None, kind="max", dtype=abi.F32):
    """Max or mean over (kh, kw) windows stepping by `stride` (default: the window): a reduce over two window axes."""
    sh, sw = (kh, kw) if stride is None else (stride, stride)
    oh, ow = (height - kh) // sh + 1, (width - kw) // sw + 1
    if oh <= 0 or ow <= 0:
        raise ValueError("the window does not fit the input")
    x = Operand(0, dtype, [channels * height * width, height * width, sh * width, sw], stream_strides=[width, 1])
    if kind == "max":
        car = carrier_max(load(0))
    elif kind == "mean":
        car = Carrier([load(0)], [item(0)], [A(0) + B(0)], [0.0], F(0) * (1.0 / (kh * kw)))
    else:
        raise ValueError("kind is 'max' or 'mean'")
    return (batch, channels, oh, ow), (kh, kw), [x], car


class Description:
    """A packed sanic_generic_desc with the ctypes arrays it points into kept alive."""

    def __init__(self, grid: Sequence[int], operands: Sequence[Operand], *, carrier: Carrier | None = None, stream: int = 0,
                 value: E | None = None, epilogue: E | None = None, store_if: E | None = None, out_dtype: int = abi.F32,
                 lanes: int = 1, warps: int = 1, interleave: bool = False, lane_axis: bool = False):
        if len(grid) > abi.MAX_AXES:
            raise ValueError(f"at most {abi.MAX_AXES} grid axes")
        if (carrier is None) == (value is None):
            raise ValueError("give a carrier (a fold) or a value (a pointwise kernel), not both")
        window = ()
        if carrier is not None and not isinstance(stream, int):      # a window of several axes, reduced at once
            window = tuple(int(e) for e in stream)
            if not 2 <= len(window) <= 3:
                raise ValueError("a streamed window has 2 or 3 axes (one axis: give its extent)")
            stream = 1
            for e in window:
                stream *= e
        if carrier is not None and stream <= 0:
            raise ValueError("a fold needs a positive streamed extent")
        ops: list = []

        def prog(e: E) -> abi.Expr:
            first = len(ops)
            e.flatten(ops)
            return abi.Expr(first, len(ops) - first)

        d = abi.GenericDesc()
        d.n_axes = len(grid)
        for i, g in enumerate(grid):
            d.extent[i] = int(g)
        d.stream = int(stream) if carrier is not None else 0
        d.stream_dims = len(window)
        for j, e in enumerate(window):
            d.stream_extent[j] = e
        d.lanes, d.warps, d.interleave = int(lanes), int(warps), int(bool(interleave))
        d.lane_axis = int(bool(lane_axis))
        self._operands = (abi.Operand * max(1, len(operands)))()
        for i, o in enumerate(operands):
            if len(o.strides) != len(grid):
                raise ValueError("an operand needs one stride per grid axis")
            self._operands[i].dtype, self._operands[i].buffer = int(o.dtype), int(o.buffer)
            self._operands[i].offset, self._operands[i].stream_stride = int(o.offset), int(o.stream_stride)
            self._operands[i].gather_stride, self._operands[i].gather_extent = int(o.gather_stride), int(o.gather_extent)
            self._operands[i].inner_stride = int(o.inner_stride)
            if window:
                if len(o.stream_strides) != len(window):
                    raise ValueError("with a streamed window an operand needs one stream stride per window axis")
                for j, st in enumerate(o.stream_strides):
                    self._operands[i].stream_sub_stride[j] = int(st)
            for a, s in enumerate(o.strides):
                self._operands[i].stride[a] = int(s)
        d.n_operands, d.operands = len(operands), self._operands
        if carrier is not None:
            n = len(carrier.into)
            if not (len(carrier.combine) == len(carrier.identity) == n):
                raise ValueError("into, combine and identity must have one entry per slot")
            self._leaves = (abi.Expr * max(1, len(carrier.leaves)))(*[prog(e) for e in carrier.leaves])
            self._into = (abi.Expr * n)(*[prog(e) for e in carrier.into])
            self._combine = (abi.Expr * n)(*[prog(e) for e in carrier.combine])
            self._identity = (C.c_double * n)(*[float(v) for v in carrier.identity])
            d.n_leaves, d.leaves, d.n_slots = len(carrier.leaves), self._leaves, n
            if carrier.leaf_inner:
                if len(carrier.leaf_inner) != len(carrier.leaves):
                    raise ValueError("leaf_inner needs one extent per leaf")
                self._inner = (abi.i64 * len(carrier.leaves))(*[int(r) for r in carrier.leaf_inner])
                d.leaf_inner = self._inner
            d.identity, d.into, d.combine = self._identity, self._into, self._combine
            d.project = prog(carrier.project)
        else:
            d.project = prog(value)
        d.epilogue = prog(epilogue) if epilogue is not None else abi.Expr(0, 0)
        d.store_if = prog(store_if) if store_if is not None else abi.Expr(0, 0)
        d.out_dtype = int(out_dtype)
        self._ops = (abi.ExprOp * max(1, len(ops)))(*[abi.ExprOp(o, a, v) for o, a, v in ops])
        d.n_ops, d.ops = len(ops), self._ops
        self.desc = d
        self.points = 1
        for g in grid:
            self.points *= int(g)
        self.n_buffers = 1 + max((o.buffer for o in operands), default=-1)


def source(desc: Description) -> str:
    """The generated CUDA C text. Needs the library, not a device."""
    lib = abi.load()
    need = C.c_size_t()
    rc = lib.sanic_generic_source(None, C.byref(desc.desc), None, 0, C.byref(need))
    if rc != abi.OK:
        raise ValueError(f"the descriptor does not render (status {rc})")
    buf = C.create_string_buffer(need.value)
    lib.sanic_generic_source(None, C.byref(desc.desc), buf, need.value, None)
    return buf.value.decode()


def compiles(desc: Description) -> int:
    """Compiles the generated text for sm_100a without loading it; returns the cubin size. Needs no device."""
    lib = abi.load()
    n = C.c_size_t()
    rc = lib.sanic_generic_cubin_size(None, C.byref(desc.desc), C.byref(n))
    if rc != abi.OK:
        raise RuntimeError(f"the generated kernel does not compile (status {rc})")
    return n.value


def cache_stats(lib=None):
    """(texts compiled, compilations answered from the cache) of this process: isomorphic stages compile once."""
    lib = lib or abi.load()
    a, b = abi.i64(0), abi.i64(0)
    lib.sanic_generic_cache_stats(C.byref(a), C.byref(b))
    return a.value, b.value


class GenericKernel:
    """A compiled and loaded generic kernel on one device (the Executable of one stage)."""

    def __init__(self, device, desc: Description):
        self.device, self.desc = device, desc
        h = C.c_void_p()
        device._check(device.lib.sanic_generic_compile(device.h, C.byref(desc.desc), C.byref(h)), "generic_compile")
        self.h = h

    @property
    def name(self) -> str:
        """Kind, grid, streamed extent, schedule and output width, e.g. 'fold1_g8x4_s16_lanes_f32'."""
        return self.device.lib.sanic_generic_kernel_name(self.h).decode()

    def __call__(self, buffers, out):
        """buffers: torch tensors on the device, in buffer-index order; out: a tensor of grid size at the output dtype."""
        if out.numel() != self.desc.points:
            raise ValueError("the output must hold one element per grid point")
        arr = (C.c_void_p * max(1, len(buffers)))(*[C.c_void_p(b.data_ptr()) for b in buffers])
        self.device._check(self.device.lib.sanic_generic_launch(self.device.h, self.h, arr, len(buffers), C.c_void_p(out.data_ptr()),
                                                                self.device.stream()), "generic_launch")
        return out

    def close(self):
        if getattr(self, "h", None):
            self.device.lib.sanic_generic_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
