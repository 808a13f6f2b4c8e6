"""The binding surface without a device: every refusal of `Program::try_run`, `Program::capture` and
`Graph::compile_for` / `StepProgram::instantiate` (reference src/compile.rs:41-76,190-229,820-890 and
src/graph.rs:231-245; the reference's own tests of them are tests/graph.rs and tests/compile.rs) is decided on
the host before any CUDA call, so a schedule compiled with no context exercises them here."""
import ctypes as C

import pytest

from sanic_b200 import _abi as abi
from sanic_b200.backend import CompileError, carrier_contraction
from sanic_b200.schedule import ProgramError, ScheduleBuilder, _field_offset

P = 0x1000          # stand-in addresses: nothing is dereferenced without a device


def gemv_stage(K, rows, batch=1):
    s = abi.StageDesc()
    s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_GEMV
    s.carrier = carrier_contraction(abi.BF16)
    g = s.u.gemv
    g.batch, g.K, g.weight_dtype, g.group, g.n_segments = batch, K, abi.BF16, 64, 1
    g.rows[0] = rows
    g.out_dtype, g.epilogue = abi.F32, abi.EPI_STORE
    return s


def step_schedule():
    """y = W x; state' = y (a plain root fed back: ping-pong); cache' = where(coord == pos, y, cache) compiled in place."""
    b = ScheduleBuilder()
    b.input("w", abi.BF16, (64, 128))
    b.input("x", abi.BF16, (1, 128))
    b.input("state", abi.F32, (1, 64))
    b.input("cache", abi.F32, (1, 64))
    b.scratch("y", abi.F32, (1, 64))
    b.scratch("cache_next", abi.F32, (1, 64))
    b.stage(gemv_stage(128, 64), {"gemv.x": "x", "gemv.w[0]": "w", "gemv.out[0]": "y"})
    b.stage(gemv_stage(128, 64), {"gemv.x": "x", "gemv.w[0]": "w", "gemv.out[0]": "cache_next"})
    b.root("y")
    b.root("cache_next", in_place_of="cache")
    return b


GOOD = {"w": (P, abi.BF16, (64, 128)), "x": (P, abi.BF16, (1, 128)), "state": (P, abi.F32, (1, 64)), "cache": (P, abi.F32, (1, 64))}


def kind_of(fn):
    with pytest.raises(ProgramError) as e:
        fn()
    return e.value.kind


def test_field_offsets_follow_the_header_layout():
    base = abi.StageDesc.u.offset
    assert _field_offset("gemv.x") == base + abi.GemvParams.x.offset
    assert _field_offset("gemv.w[2]") == base + abi.GemvParams.w.offset + 16
    assert _field_offset("decode.partials") == base + abi.DecodeParams.partials.offset
    assert _field_offset("generic.buffers[5]") == base + abi._GenericStage.buffers.offset + 40
    assert _field_offset("embed.scales") % 8 == 0


def test_input_names_and_counts():
    prog = step_schedule().compile()
    assert prog.input_names() == ["w", "x", "state", "cache"]
    assert prog.n_outputs == 2
    prog.check_bindings(GOOD)          # a complete, well-typed set passes


def test_binding_refusals_in_the_reference_order():
    prog = step_schedule().compile()
    assert kind_of(lambda: prog.check_bindings(dict(GOOD, nope=(P, abi.F32, (1,))))) == "UnknownInput"
    assert kind_of(lambda: prog.check_bindings(list(GOOD.items()) + [("x", GOOD["x"])])) == "DuplicateInput"
    assert kind_of(lambda: prog.check_bindings({k: v for k, v in GOOD.items() if k != "state"})) == "MissingInput"
    assert kind_of(lambda: prog.check_bindings(dict(GOOD, x=(P, abi.BF16, (128,))))) == "Shape"
    assert kind_of(lambda: prog.check_bindings(dict(GOOD, x=(P, abi.BF16, (2, 128))))) == "Shape"
    assert kind_of(lambda: prog.check_bindings(dict(GOOD, x=(P, abi.F32, (1, 128))))) == "Dtype"
    # an unknown name is reported before a missing one, a shape before a dtype (src/compile.rs:196-226)
    assert kind_of(lambda: prog.check_bindings({"nope": (P, abi.F32, (1,))})) == "UnknownInput"
    assert kind_of(lambda: prog.check_bindings(dict(GOOD, x=(P, abi.F32, (3, 128))))) == "Shape"
    with pytest.raises(ProgramError, match=r"`x` has shape \[2, 128\]; expected \[1, 128\]"):
        prog.check_bindings(dict(GOOD, x=(P, abi.BF16, (2, 128))))
    # running needs the device; the checks come first either way
    assert kind_of(lambda: prog.try_run({k: v for k, v in GOOD.items() if k != "w"})) == "MissingInput"
    assert kind_of(lambda: prog.try_run(GOOD)) == "Backend"


def test_feedback_refusals():
    prog = step_schedule().compile()
    cap = lambda fb, bind=GOOD: prog.capture(bind, fb)
    with pytest.raises(ProgramError, match="output index 7 is out of range \\(2 outputs\\)"):
        cap([(7, "state")])
    with pytest.raises(ProgramError, match="no input named `ghost`"):
        cap([(0, "ghost")])
    with pytest.raises(ProgramError, match="output 0 has shape \\[1, 64\\]; input `x` expects \\[1, 128\\]"):
        cap([(0, "x")])
    with pytest.raises(ProgramError, match="fed back more than once"):
        cap([(0, "state"), (0, "cache")])
    with pytest.raises(ProgramError, match="`state` is fed more than once"):
        cap([(0, "state"), (1, "state")])
    for fb in ([(7, "state")], [(0, "ghost")], [(0, "x")]):
        assert kind_of(lambda: cap(fb)) == "Feedback"
    # binding errors come before feedback errors, as in Program::capture
    assert kind_of(lambda: cap([(7, "state")], {k: v for k, v in GOOD.items() if k != "w"})) == "MissingInput"
    # a valid wiring passes every check and stops only at the missing device
    assert kind_of(lambda: cap([(0, "state"), (1, "cache")])) == "Backend"


def test_feedback_storage_mismatch():
    b = step_schedule()
    b.input("state16", abi.BF16, (1, 64))
    prog = b.compile()
    bind = dict(GOOD, state16=(P, abi.BF16, (1, 64)))
    with pytest.raises(ProgramError, match="input `state16` is bf16; output 0 is stored f32"):
        prog.capture(bind, [(0, "state16")])


def test_machine_refusals():
    prog = step_schedule().compile()
    user = {"w": GOOD["w"], "x": GOOD["x"]}
    states = [("state", 0), ("cache", 1)]
    # a state declared at another width than the compilation's boundary policy (src/graph.rs:236-245)
    with pytest.raises(CompileError, match="state `state` is declared f32 but the compilation's policy stores step boundaries as bf16"):
        prog.instantiate(states, user, abi.BF16)
    # the machine owns its states: binding one is a duplicate
    assert kind_of(lambda: prog.instantiate(states, dict(user, cache=GOOD["cache"]), abi.F32)) == "DuplicateInput"
    assert kind_of(lambda: prog.instantiate(states, {"w": GOOD["w"]}, abi.F32)) == "MissingInput"
    assert kind_of(lambda: prog.instantiate([("ghost", 0)], user, abi.F32)) == "Feedback"
    assert kind_of(lambda: prog.instantiate(states, user, abi.F32, outputs=[("y", 5)])) == "Invalid"
    # pinned states may keep their own width (Graph::output_at, src/graph.rs:113-125)
    assert kind_of(lambda: prog.instantiate([("state", 0, 1), ("cache", 1, 1)], user, abi.BF16)) == "Backend"


def test_schedule_compile_refusals():
    def build(mut):
        b = step_schedule()
        mut(b)
        return b.compile()
    with pytest.raises(CompileError):
        build(lambda b: b.outputs.clear())                                     # CompileError::EmptyOutputs
    with pytest.raises(CompileError):
        build(lambda b: b.stages.clear() or b.relocs.clear())                  # an empty stage list
    with pytest.raises(CompileError):
        build(lambda b: b.relocs.append((9, 8, 0, 0)))                         # a relocation into a stage that is not there
    with pytest.raises(CompileError):
        build(lambda b: b.relocs.append((0, 8, 0, 1 << 20)))                   # ... or past the end of its buffer
    with pytest.raises(CompileError):
        build(lambda b: b.buffers.__setitem__(1, ("x", abi.BUF_INPUT, abi.BF16, (1, 0))))    # dynamic / empty extent
    with pytest.raises(CompileError):
        build(lambda b: b.buffers.__setitem__(1, ("w", abi.BUF_INPUT, abi.BF16, (1, 128))))  # a name declared twice
    with pytest.raises(CompileError):
        build(lambda b: b.buffers.__setitem__(1, ("x", abi.BUF_INPUT, 99, (1, 128))))        # an unknown storage width
    with pytest.raises(CompileError):
        build(lambda b: b.in_place.append((0, b.index["x"])))                  # a root cannot overwrite an input of another shape
    with pytest.raises(CompileError):
        step_schedule().input("w", abi.BF16, (1,))                             # the builder refuses a duplicate name itself


def test_one_shot_schedules_of_the_configurations_check_their_bindings():
    """Attention, the RMSNorm-fused GEMM and split-KV decode as schedules: one fused stage each (plus the RoPE cut in
    front of a fold over rotated operands), inputs bound by name with the reference's refusals."""
    from sanic_b200 import schedules
    assert _field_offset("attn.p.v") == abi.StageDesc.u.offset + abi.AttnParams.v.offset
    assert _field_offset("gemm.w") == abi.StageDesc.u.offset + abi.GemmRmsnormParams.w.offset
    assert _field_offset("rope.table") == abi.StageDesc.u.offset + abi._RopeStage.table.offset

    c1 = schedules.attention(1, 1, 1, 256, 1024, 64, storage=abi.F32).compile()
    assert c1.input_names() == ["q", "k", "v"] and c1.n_stages == 1
    good = {"q": (P, abi.F32, (1, 1, 256, 64)), "k": (P, abi.F32, (1, 1, 1024, 64)), "v": (P, abi.F32, (1, 1, 1024, 64))}
    c1.check_bindings(good)
    assert kind_of(lambda: c1.check_bindings(dict(good, q=(P, abi.BF16, (1, 1, 256, 64))))) == "Dtype"
    assert kind_of(lambda: c1.check_bindings(dict(good, k=(P, abi.F32, (1, 1, 1000, 64))))) == "Shape"
    assert kind_of(lambda: c1.check_bindings({k: v for k, v in good.items() if k != "v"})) == "MissingInput"

    c3 = schedules.attention(8, 32, 8, 4096, 4096, 64, storage=abi.BF16, causal=True, window=1024, rope=True).compile()
    assert c3.input_names() == ["q", "k", "v", "rope_table"] and c3.n_stages == 3      # rotate q, rotate k, fold
    c2 = schedules.rmsnorm_gemm(4096, 2048, 8192, w_is_nk=False).compile()
    assert c2.input_names() == ["x", "gamma", "w"] and c2.n_stages == 1
    assert kind_of(lambda: c2.check_bindings({"x": (P, abi.BF16, (4096, 2048)), "gamma": (P, abi.BF16, (2048,)),
                                              "w": (P, abi.BF16, (8192, 2048))})) == "Shape"       # [K, N] was declared
    c5 = schedules.splitkv_decode(4, 32, 8, 1 << 20, 128, n_splits=74).compile()
    assert c5.input_names() == ["q", "k", "v"] and c5.n_stages == 1

    # a stage whose op does not match its carrier is refused when the schedule is compiled
    b = schedules.rmsnorm_gemm(128, 256, 256)
    b.stages[0].carrier = carrier_contraction(abi.BF16)
    with pytest.raises(CompileError, match="does not match its carrier"):
        b.compile()
    with pytest.raises(ValueError):
        schedules.attention(1, 1, 1, 8, 8, 64, storage=abi.F32, rope=True)
