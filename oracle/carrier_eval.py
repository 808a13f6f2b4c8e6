"""CPU oracle for carriers given as expression programs (numpy, f64).

TEST INFRASTRUCTURE ONLY: imported by tests/ and by __graft_entry__.smoke(). The product package never
imports it.

Restates, in dense f64:
  * the scalar-expression evaluator of the reference, src/derive.rs:219-253 (Lt gives 1.0 / 0.0, Where tests
    `!= 0`, max / min as f64::max / f64::min);
  * Carrier::fold_acc / lift / merge / project, src/derive.rs:292-352: a left fold from the identity in index
    order, every slot of a merge computed from the OLD accumulators;
  * run_carrier_split, src/interp.rs:597-640: partials over the contiguous chunks [b*n/B, (b+1)*n/B), merged
    left to right starting from the first partial, projected once.
A program is a postfix list of (name, arg, value) triples. All grid points are evaluated at once (arrays of
grid shape); the streamed axis is a Python loop, so keep stream * ops small.
"""
from __future__ import annotations

import numpy as np


def _bf16_round(x: np.ndarray) -> np.ndarray:
    """RNE to bf16 and back, quiet NaN (src/scalar.rs:128-135)."""
    f = np.asarray(x, np.float64).astype(np.float32)
    b = f.view(np.uint32)
    r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint32) << 16
    nan = np.isnan(f)
    r = np.where(nan, (b & 0xFFFF0000) | 0x00400000, r).astype(np.uint32)
    return r.view(np.float32).astype(np.float64)


def _run(prog, env):
    st = []
    for name, arg, value in prog:
        if name == "const": st.append(np.float64(value))
        elif name == "load": st.append(env["load"](arg))
        elif name == "coord": st.append(env["coord"](arg))
        elif name == "gather": st.append(env["gather"](arg, st.pop()))
        elif name in ("item", "a", "b", "f"): st.append(env[name][arg])
        elif name == "result": st.append(env["result"])
        elif name in ("neg", "recip", "exp", "log", "sqrt", "tanh", "sin", "cos", "round_bf16", "round_f32"):
            x = st.pop()
            with np.errstate(all="ignore"):
                st.append({"neg": lambda v: -v, "recip": lambda v: 1.0 / v, "exp": np.exp, "log": np.log, "sqrt": np.sqrt,
                           "tanh": np.tanh, "sin": np.sin, "cos": np.cos, "round_bf16": _bf16_round,
                           "round_f32": lambda v: np.asarray(v, np.float64).astype(np.float32).astype(np.float64)}[name](x))
        elif name == "where":
            b, a, c = st.pop(), st.pop(), st.pop()
            st.append(np.where(np.asarray(c) != 0.0, a, b))
        else:
            y, x = st.pop(), st.pop()
            with np.errstate(all="ignore"):
                if name == "add": st.append(x + y)
                elif name == "sub": st.append(x - y)
                elif name == "mul": st.append(x * y)
                elif name == "div": st.append(np.asarray(x, np.float64) / y)
                elif name == "max": st.append(np.fmax(x, y))      # f64::max ignores a NaN side
                elif name == "min": st.append(np.fmin(x, y))
                elif name == "lt": st.append(np.where(np.asarray(x) < y, 1.0, 0.0))
                else: raise ValueError(f"unknown op {name}")
    if len(st) != 1:
        raise ValueError("a program must leave exactly one value")
    return st[0]


class _Point:
    """Loads and coordinates at every grid point, for one value of the streamed coordinate."""

    def __init__(self, grid, operands, buffers):
        self.grid = tuple(int(g) for g in grid)
        self.coords = np.indices(self.grid) if self.grid else np.zeros((0,))
        self.operands, self.buffers = operands, [np.asarray(b, np.float64).reshape(-1) for b in buffers]
        self.base = []
        for o in operands:
            idx = np.full(self.grid, int(o["offset"]), np.int64)
            for a, s in enumerate(o["strides"]):
                idx = idx + self.coords[a] * int(s)
            self.base.append(idx)

    def env(self, s, r=None):
        def load(k):
            idx = self.base[k] + (0 if s is None else s * int(self.operands[k]["stream_stride"]))
            if r is not None:
                idx = idx + r * int(self.operands[k].get("inner_stride", 0))
            return self.buffers[int(self.operands[k]["buffer"])][idx]

        def coord(a):
            if a == len(self.grid):
                if s is None:
                    raise ValueError("stream coordinate outside the fold body")
                return np.full(self.grid, float(s))
            if a == len(self.grid) + 1:
                if r is None:
                    raise ValueError("inner coordinate outside a contracted leaf")
                return np.full(self.grid, float(r))
            return self.coords[a].astype(np.float64)
        def gather(k, index):
            # index = round() (half away from zero), then a bounds check (src/interp.rs:378-379)
            o = self.operands[k]
            gi = np.broadcast_to(np.trunc(np.asarray(index, np.float64) + np.copysign(0.5, index)), self.grid).astype(np.int64)
            if np.any(gi < 0) or np.any(gi >= int(o["gather_extent"])):
                raise IndexError("gather index out of range")
            idx = self.base[k] + (0 if s is None else s * int(o["stream_stride"])) + gi * int(o["gather_stride"])
            return self.buffers[int(o["buffer"])][idx]
        return {"load": load, "coord": coord, "gather": gather}


def pointwise(grid, operands, buffers, value, epilogue=None) -> np.ndarray:
    """out[point] = value (an elementwise cone, evaluated densely as interp::eval does)."""
    pt = _Point(grid, operands, buffers)
    env = pt.env(None)
    r = np.broadcast_to(_run(value, env), pt.grid).astype(np.float64)
    if epilogue is not None:
        env["result"] = r
        r = np.broadcast_to(_run(epilogue, env), pt.grid).astype(np.float64)
    return r


def carrier_fold(grid, stream, operands, buffers, leaves, into, combine, identity, project, epilogue=None, blocks=1,
                 leaf_inner=()) -> np.ndarray:
    """run_carrier (blocks == 1) / run_carrier_split (blocks > 1) of one carrier over every grid point. leaf_inner[l] = R > 1
    makes leaf l a Reduce(Add) over an inner axis: a left fold from 0.0 in index order (src/interp.rs:355-363)."""
    pt = _Point(grid, operands, buffers)
    n, nb = int(stream), int(blocks)
    if not (1 <= nb <= n):
        raise ValueError("blocks must be in 1..=extent")

    def merge(acc, other):
        env = {"a": acc, "b": other}
        return [np.broadcast_to(_run(c, env), pt.grid).astype(np.float64) for c in combine]

    def fold(lo, hi):
        acc = [np.full(pt.grid, float(v)) for v in identity]
        for s in range(lo, hi):
            env = pt.env(s)
            items = []
            for li, l in enumerate(leaves):
                R = int(leaf_inner[li]) if li < len(leaf_inner) else 0
                if R > 1:
                    tot = np.zeros(pt.grid)
                    for r in range(R):
                        tot = tot + np.broadcast_to(_run(l, pt.env(s, r)), pt.grid)
                    items.append(tot)
                else:
                    items.append(np.broadcast_to(_run(l, env), pt.grid))
            env["item"] = items
            el = [np.broadcast_to(_run(e, env), pt.grid).astype(np.float64) for e in into]
            acc = merge(acc, el)
        return acc

    parts = [fold(b * n // nb, (b + 1) * n // nb) for b in range(nb)]
    acc = parts[0]
    for p in parts[1:]:
        acc = merge(acc, p)
    env = pt.env(None)
    env["f"] = acc
    r = np.broadcast_to(_run(project, env), pt.grid).astype(np.float64)
    if epilogue is not None:
        env["result"] = r
        r = np.broadcast_to(_run(epilogue, env), pt.grid).astype(np.float64)
    return r
