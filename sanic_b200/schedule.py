"""Schedules over a buffer table: bind-by-name runs, replays with state feedback, machines.

Host-side mirror of `Program` (`try_run`, `capture`), `MetalReplay` and `Graph` / `StepProgram` / `Machine` of
the reference (src/compile.rs:122-229,800-1035 and src/graph.rs:31-360 of the reference project) over the C
ABI's `sanic_schedule_*`, `sanic_replay_*` and `sanic_machine_*` entry points. A `ScheduleBuilder` collects what
the reference's emitter produces for its runtime: a buffer table, stages whose pointer fields refer to table
buffers, the roots, and which roots were compiled in place.

`compile(dev=None)` gives a program without a device: every binding and feedback refusal can be exercised
anywhere; only running needs the GPU.
"""
from __future__ import annotations

import ctypes as C

from . import _abi as abi
from .backend import CompileError, RunError

_ERR_TEXT = {abi.ERR_MISSING_INPUT: "MissingInput", abi.ERR_UNKNOWN_INPUT: "UnknownInput",
             abi.ERR_DUPLICATE_INPUT: "DuplicateInput", abi.ERR_SHAPE: "Shape", abi.ERR_DTYPE: "Dtype",
             abi.ERR_FEEDBACK: "Feedback", abi.ERR_CUDA: "Backend", abi.ERR_TIMEOUT: "Backend", abi.ERR_INVALID: "Invalid"}


class ProgramError(RunError):
    """A RunError that carries its kind (src/compile.rs:41-76): MissingInput, UnknownInput, DuplicateInput, Shape,
    Dtype, Feedback or Backend."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


def _field_offset(path: str) -> int:
    """Byte offset inside sanic_stage_desc of a pointer field given as a dotted path into the stage union, e.g.
    'gemv.w[1]', 'decode.k', 'embed.table', 'generic.buffers[3]'."""
    off = abi.StageDesc.u.offset
    cls = abi._StageUnion
    for part in path.split("."):
        name, idx = part, None
        if "[" in part:
            name, idx = part[:part.index("[")], int(part[part.index("[") + 1:-1])
        f = getattr(cls, name)
        off += f.offset
        ftype = dict((n, t) for n, t, *_ in cls._fields_)[name]
        if idx is not None:
            off += idx * C.sizeof(ftype._type_)
            ftype = ftype._type_
        cls = ftype
    return off


class ScheduleBuilder:
    def __init__(self):
        self.buffers = []          # (name, kind, dtype, shape)
        self.index = {}
        self.stages = []           # abi.StageDesc
        self.relocs = []           # (stage, field offset, buffer, byte offset)
        self.outputs = []          # buffer index per root
        self.in_place = []         # (root index, input buffer index)

    def _add(self, name, kind, dtype, shape):
        if name in self.index:
            raise CompileError(f"InvalidGraph: buffer `{name}` is declared twice")
        self.index[name] = len(self.buffers)
        self.buffers.append((name, kind, dtype, tuple(int(e) for e in shape)))
        return self.index[name]

    def input(self, name, dtype, shape):
        return self._add(name, abi.BUF_INPUT, dtype, shape)

    def scratch(self, name, dtype, shape):
        return self._add(name, abi.BUF_SCRATCH, dtype, shape)

    def stage(self, desc, refs: dict):
        """Append a stage; `refs` maps a pointer-field path ('gemv.x', 'gemv.w[0]', ...) to a buffer name or a
        (buffer name, byte offset) pair."""
        idx = len(self.stages)
        self.stages.append(desc)
        for path, target in refs.items():
            name, byte_off = (target, 0) if isinstance(target, str) else target
            if name not in self.index:
                raise CompileError(f"InvalidGraph: stage {idx} refers to an undeclared buffer `{name}`")
            self.relocs.append((idx, _field_offset(path), self.index[name], int(byte_off)))
        return idx

    def root(self, name, in_place_of=None):
        """Declare the next output root; `in_place_of` names the input whose buffer this root overwrites."""
        self.outputs.append(self.index[name])
        if in_place_of is not None:
            self.in_place.append((len(self.outputs) - 1, self.index[in_place_of]))
        return len(self.outputs) - 1

    def compile(self, dev=None):
        return Program(self, dev)


def _binding_array(bindings):
    """bindings: iterable of (name, tensor-like). A tensor-like has data_ptr(), shape and a torch dtype, or is a
    tuple (address, abi dtype, shape) for tests without a device."""
    items = list(bindings.items()) if isinstance(bindings, dict) else list(bindings)
    arr = (abi.Binding * max(1, len(items)))()
    keep = []
    for i, (name, t) in enumerate(items):
        nb = name.encode()
        keep.append(nb)
        arr[i].name = nb
        if isinstance(t, tuple):
            ptr, dt, shape = t
        else:
            ptr, dt, shape = t.data_ptr(), abi.dtype_of_torch(t.dtype), tuple(t.shape)
            if dt == abi.I4 and shape:      # packed two elements per byte: the declared shape counts elements
                shape = shape[:-1] + (shape[-1] * 2,)
        arr[i].dptr, arr[i].dtype, arr[i].rank = ptr, dt, len(shape)
        for a, e in enumerate(shape[:abi.MAX_AXES]):
            arr[i].shape[a] = int(e)
    return arr, len(items), keep


class Program:
    """A compiled schedule: `Program<B>` of the reference. Outputs come back in root order."""

    def __init__(self, b: ScheduleBuilder, dev=None):
        self.dev = dev
        self.lib = dev.lib if dev is not None else abi.load()
        self._keep = []
        self.n_stages = len(b.stages)
        n_b = len(b.buffers)
        decls = (abi.BufferDecl * max(1, n_b))()
        for i, (name, kind, dtype, shape) in enumerate(b.buffers):
            nb = name.encode()
            self._keep.append(nb)
            decls[i].name, decls[i].kind, decls[i].dtype, decls[i].rank = nb, kind, dtype, len(shape)
            if len(shape) > abi.MAX_AXES:
                raise CompileError(f"InvalidInput: buffer `{name}` has more than {abi.MAX_AXES} axes")
            for a, e in enumerate(shape):
                decls[i].shape[a] = e
        stages = (abi.StageDesc * max(1, len(b.stages)))(*b.stages)
        relocs = (abi.Reloc * max(1, len(b.relocs)))()
        for i, (st, off, buf, boff) in enumerate(b.relocs):
            relocs[i].stage, relocs[i].field_offset, relocs[i].buffer, relocs[i].byte_offset = st, off, buf, boff
        outs = (C.c_int32 * max(1, len(b.outputs)))(*b.outputs)
        ipr = (C.c_int32 * max(1, len(b.in_place)))(*[r for r, _ in b.in_place])
        ipi = (C.c_int32 * max(1, len(b.in_place)))(*[i for _, i in b.in_place])
        d = abi.ScheduleDesc()
        d.stages, d.n_stages = C.cast(stages, C.c_void_p), len(b.stages)
        d.buffers, d.n_buffers = C.cast(decls, C.c_void_p), n_b
        d.relocs, d.n_relocs = C.cast(relocs, C.c_void_p), len(b.relocs)
        d.outputs, d.n_outputs = C.cast(outs, C.c_void_p), len(b.outputs)
        d.in_place_root, d.in_place_input, d.n_in_place = C.cast(ipr, C.c_void_p), C.cast(ipi, C.c_void_p), len(b.in_place)
        self._keep += [decls, stages, relocs, outs, ipr, ipi]
        h = C.c_void_p()
        rc = self.lib.sanic_schedule_compile(dev.h if dev is not None else None, C.byref(d), C.byref(h))
        if rc != abi.OK:
            msg = self.lib.sanic_schedule_last_error(None).decode()
            raise CompileError(f"schedule_compile: {msg}")
        self.h = h
        self.n_outputs = len(b.outputs)
        self.buffer_decls = list(b.buffers)

    def _raise(self, rc, what):
        msg = self.lib.sanic_schedule_last_error(self.h).decode()
        if rc == abi.ERR_UNSUPPORTED:
            raise CompileError(f"Backend: {msg}")
        raise ProgramError(_ERR_TEXT.get(rc, f"status {rc}"), f"{what}: {msg}")

    def input_names(self):
        n = self.lib.sanic_schedule_input_count(self.h)
        return [self.lib.sanic_schedule_input_name(self.h, i).decode() for i in range(n)]

    def check_bindings(self, bindings):
        arr, n, _keep = _binding_array(bindings)
        rc = self.lib.sanic_schedule_check_bindings(self.h, arr, n)
        if rc != abi.OK:
            self._raise(rc, "bindings")

    def try_run(self, bindings, stream=None):
        """Program::try_run: returns one BufferView per root (address, dtype, shape), in root order."""
        arr, n, _keep = _binding_array(bindings)
        outs = (abi.BufferView * self.n_outputs)()
        st = stream if stream is not None else (self.dev.stream() if self.dev is not None else None)
        rc = self.lib.sanic_schedule_execute(self.h, arr, n, st, outs, self.n_outputs)
        if rc != abi.OK:
            self._raise(rc, "run")
        return list(outs)

    run = try_run

    def capture(self, bindings, feedback=(), persistent=False, stream=None):
        """Program::capture: `feedback` is a list of (root index, input name)."""
        arr, n, _keep = _binding_array(bindings)
        fo = (C.c_int32 * max(1, len(feedback)))(*[int(o) for o, _ in feedback])
        names = [nm.encode() for _, nm in feedback]
        fi = (C.c_char_p * max(1, len(feedback)))(*names)
        h = C.c_void_p()
        st = stream if stream is not None else (self.dev.stream() if self.dev is not None else None)
        rc = self.lib.sanic_schedule_capture(self.h, arr, n, fo, fi, len(feedback), int(persistent), st, C.byref(h))
        if rc != abi.OK:
            self._raise(rc, "capture")
        return Replay(self, h)

    def instantiate(self, states, bindings, boundary_dtype, outputs=(), persistent=False, stream=None):
        """Graph::compile_for + StepProgram::instantiate: `states` is a list of (input name, root index[, pinned]);
        `outputs` a list of (name, root index). State buffers are allocated by the machine, zero-filled."""
        arr, n, _keep = _binding_array(bindings)
        sd = (abi.StateDecl * max(1, len(states)))()
        keep = []
        for i, st_ in enumerate(states):
            nb = st_[0].encode()
            keep.append(nb)
            sd[i].input_name, sd[i].root, sd[i].pinned = nb, int(st_[1]), int(st_[2]) if len(st_) > 2 else 0
        onames = [nm.encode() for nm, _ in outputs]
        on = (C.c_char_p * max(1, len(outputs)))(*onames)
        oroots = (C.c_int32 * max(1, len(outputs)))(*[int(r) for _, r in outputs])
        h = C.c_void_p()
        st = stream if stream is not None else (self.dev.stream() if self.dev is not None else None)
        rc = self.lib.sanic_machine_instantiate(self.h, sd, len(states), boundary_dtype, arr, n, on, oroots, len(outputs),
                                                int(persistent), st, C.byref(h))
        if rc != abi.OK:
            self._raise(rc, "instantiate")
        return Replay(self, h)

    def close(self):
        if getattr(self, "h", None):
            self.lib.sanic_schedule_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Replay:
    """`MetalReplay` / `Machine`: frozen steps over bound buffers; state advances inside."""

    def __init__(self, program: Program, h):
        self.program, self.h, self.lib = program, h, program.lib

    def step(self, stream=None, timed=False):
        sec = C.c_double(0.0)
        st = stream if stream is not None else self.program.dev.stream()
        rc = self.lib.sanic_replay_step(self.h, st, C.byref(sec) if timed else None)
        if rc != abi.OK:
            self.program._raise(rc, "step")
        return sec.value if timed else None

    def stage_times(self, stream=None, cap=4096):
        buf = (C.c_double * cap)()
        n = C.c_int32(0)
        st = stream if stream is not None else self.program.dev.stream()
        rc = self.lib.sanic_replay_stage_times(self.h, st, buf, cap, C.byref(n))
        if rc != abi.OK:
            self.program._raise(rc, "stage_times")
        return [buf[i] for i in range(n.value)]

    def phase_profile(self, stream=None, cap=4096):
        """One step of a single-kernel replay, per phase: [staged, contracted, finished, barrier released] seconds."""
        buf = (C.c_double * (4 * cap))()
        n = C.c_int32(0)
        st = stream if stream is not None else self.program.dev.stream()
        rc = self.lib.sanic_replay_phase_profile(self.h, st, buf, cap, C.byref(n))
        if rc != abi.OK:
            self.program._raise(rc, "phase_profile")
        return [[buf[4 * i + k] for k in range(4)] for i in range(n.value)]

    def last_output(self, root: int):
        v = abi.BufferView()
        rc = self.lib.sanic_replay_output(self.h, root, C.byref(v))
        if rc != abi.OK:
            self.program._raise(rc, "output")
        return v

    def output(self, name: str):
        v = abi.BufferView()
        rc = self.lib.sanic_machine_output(self.h, name.encode(), C.byref(v))
        if rc != abi.OK:
            self.program._raise(rc, "output")
        return v

    def state(self, name: str):
        v = abi.BufferView()
        rc = self.lib.sanic_machine_state(self.h, name.encode(), C.byref(v))
        if rc != abi.OK:
            self.program._raise(rc, "state")
        return v

    @property
    def kernel_count(self):
        return int(self.lib.sanic_replay_kernel_count(self.h))

    @property
    def parities(self):
        return int(self.lib.sanic_replay_parities(self.h))

    def close(self):
        if getattr(self, "h", None):
            self.lib.sanic_replay_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def view_tensor(view, device):
    """A torch tensor over the device memory a BufferView names (no copy). int4 views come back as packed bytes."""
    import torch
    dt = {abi.F32: torch.float32, abi.BF16: torch.bfloat16, abi.F16: torch.float16, abi.U32: torch.int32, abi.I4: torch.uint8}[view.dtype]
    shape = tuple(view.shape[i] for i in range(view.rank))
    n = 1
    for e in shape:
        n *= e
    if view.dtype == abi.I4:
        shape, n = (view.bytes,), view.bytes

    class _Mem:       # the CUDA array interface lets torch wrap foreign device memory
        pass
    m = _Mem()
    typestr = {torch.float32: "<f4", torch.bfloat16: "<u2", torch.float16: "<f2", torch.int32: "<i4", torch.uint8: "|u1"}[dt]
    m.__cuda_array_interface__ = dict(shape=(max(n, 1),), typestr=typestr, data=(int(view.dptr), False), version=2)
    t = torch.as_tensor(m, device=device)
    if dt == torch.bfloat16:
        t = t.view(torch.int16).view(torch.bfloat16)
    return t[:n].view(shape if shape else ())
