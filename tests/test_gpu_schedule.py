"""Schedules over a buffer table on the device: bind-by-name runs, rebinding without rebuilding, replays whose
fed-back state is one buffer (a root compiled in place) or two that trade places (ping-pong), and machines
(reference src/compile.rs:132-229,820-1035, src/graph.rs:231-356; its tests: tests/graph.rs, tests/compile.rs).
Every value is checked against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from test_schedule_cpu import gemv_stage

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from sanic_b200 import CudaDevice
    return CudaDevice(0)


def bf16t(a, dev):
    bits = orc.to_bf16_bits(a)
    return torch.tensor(bits.view(np.int16), device=dev.torch_device).view(torch.bfloat16), orc.from_bf16_bits(bits)


def nerr(got, exp):
    got, exp = np.asarray(got, dtype=np.float64), np.asarray(exp, dtype=np.float64)
    assert got.shape == exp.shape and np.all(np.isfinite(got))
    return float(np.max(np.abs(got - exp) / (1.0 + np.abs(exp))))


def accumulate_schedule(in_place):
    """acc' = acc + W x: one contraction with the residual-add epilogue; the root is fed back into `acc`."""
    from sanic_b200 import abi
    from sanic_b200.schedule import ScheduleBuilder
    b = ScheduleBuilder()
    b.input("w", abi.BF16, (64, 128))
    b.input("x", abi.BF16, (2, 128))
    b.input("acc", abi.F32, (2, 64))
    b.scratch("acc.next", abi.F32, (2, 64))
    s = gemv_stage(128, 64, batch=2)
    s.u.gemv.epilogue = abi.EPI_RESIDUAL_ADD
    b.stage(s, {"gemv.x": "x", "gemv.w[0]": "w", "gemv.out[0]": "acc.next", "gemv.residual": "acc"})
    b.root("acc.next", in_place_of="acc" if in_place else None)
    return b


def test_run_binds_by_name_and_rebinding_does_not_rebuild(dev):
    from sanic_b200.schedule import view_tensor
    rng = orc.Xorshift(0x5C4ED)
    prog = accumulate_schedule(in_place=False).compile(dev)
    w1, w1v = bf16t(0.1 * rng.normal(64, 128), dev)
    w2, w2v = bf16t(0.1 * rng.normal(64, 128), dev)
    x, xv = bf16t(rng.normal(2, 128), dev)
    acc = torch.tensor(rng.normal(2, 64), dtype=torch.float32, device=dev.torch_device)
    accv = acc.cpu().numpy().astype(np.float64)
    for w, wv in ((w1, w1v), (w2, w2v), (w1, w1v)):       # other buffers under the same names: no recompilation
        (out,) = prog.try_run({"x": x, "acc": acc, "w": w})      # any order: binding is by name
        dev.sync()
        got = view_tensor(out, dev.torch_device).cpu().numpy()
        assert nerr(got, accv + orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)) <= 1e-5
        assert tuple(out.shape[i] for i in range(out.rank)) == (2, 64)
    assert torch.equal(acc.cpu(), torch.tensor(accv, dtype=torch.float32))      # a plain run never writes its inputs


@pytest.mark.parametrize("in_place", [True, False])
@pytest.mark.parametrize("persistent", [False])
def test_replay_feedback_in_place_and_ping_pong(dev, in_place, persistent):
    from sanic_b200.schedule import view_tensor
    rng = orc.Xorshift(0xFEED)
    prog = accumulate_schedule(in_place).compile(dev)
    w, wv = bf16t(0.1 * rng.normal(64, 128), dev)
    x, xv = bf16t(rng.normal(2, 128), dev)
    acc = torch.zeros(2, 64, dtype=torch.float32, device=dev.torch_device)
    st = torch.cuda.Stream(device=dev.torch_device)
    import ctypes as C
    rep = prog.capture({"w": w, "x": x, "acc": acc}, [(0, "acc")], persistent=persistent, stream=C.c_void_p(st.cuda_stream))
    # one buffer when the root overwrites its predecessor, two frozen steps trading buffers otherwise
    assert rep.parities == (1 if in_place else 2)
    step_val = orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)
    exp = np.zeros((2, 64))
    for n in range(1, 6):
        sec = rep.step(stream=C.c_void_p(st.cuda_stream), timed=True)
        assert sec > 0.0
        exp = (exp.astype(np.float32) + step_val.astype(np.float32)).astype(np.float64)     # f32 accumulation, as the device stores it
        got = view_tensor(rep.last_output(0), dev.torch_device).cpu().numpy()
        assert nerr(got, exp) <= 1e-5, n
    if in_place:
        assert view_tensor(rep.last_output(0), dev.torch_device).data_ptr() == acc.data_ptr()
    rep.close()


def test_machine_allocates_zeroed_states_and_names_outputs(dev):
    from sanic_b200 import abi
    from sanic_b200.schedule import ProgramError, view_tensor
    import ctypes as C
    rng = orc.Xorshift(0x3AC)
    prog = accumulate_schedule(in_place=True).compile(dev)
    w, wv = bf16t(0.1 * rng.normal(64, 128), dev)
    x, xv = bf16t(rng.normal(2, 128), dev)
    st = torch.cuda.Stream(device=dev.torch_device)
    sp = C.c_void_p(st.cuda_stream)
    m = prog.instantiate([("acc", 0)], {"w": w, "x": x}, abi.F32, outputs=[("total", 0)], stream=sp)
    state = view_tensor(m.state("acc"), dev.torch_device)
    assert torch.count_nonzero(state) == 0                       # StepProgram::instantiate zero-fills the states
    for _ in range(3):
        m.step(stream=sp)
    st.synchronize()
    exp = 3.0 * orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)
    assert nerr(view_tensor(m.output("total"), dev.torch_device).cpu().numpy(), exp) <= 1e-5
    with pytest.raises(ProgramError, match="no output named `nope`"):
        m.output("nope")
    # host-written inputs are read by the next replay: change x in place, the frozen step sees it
    x.zero_()
    torch.cuda.synchronize()
    m.step(stream=sp)
    st.synchronize()
    assert nerr(view_tensor(m.output("total"), dev.torch_device).cpu().numpy(), exp) <= 1e-5
    m.close()


def test_generated_kernel_as_a_schedule_stage(dev):
    """A carrier no specialised kernel matches runs as a generated stage whose operands are table buffers:
    row sums of x (the reference's `[3, 7]` pin, tests/compile.rs:13-40, at another size) feeding a second
    generated stage that adds a bias: two stages, one intermediate, all through the buffer table."""
    from sanic_b200 import abi, emitter as em
    from sanic_b200.schedule import ScheduleBuilder, view_tensor
    rows, n = 5, 300
    rng = orc.Xorshift(0x6E4)
    xv = orc.round_to(orc.DT_F32, rng.normal(rows, n))
    bv = orc.round_to(orc.DT_F32, rng.normal(rows))
    x = torch.tensor(xv, dtype=torch.float32, device=dev.torch_device)
    bias = torch.tensor(bv, dtype=torch.float32, device=dev.torch_device)
    d1 = em.Description((rows,), [em.Operand(0, abi.F32, [n], 1)], carrier=em.carrier_sum(em.load(0)), stream=n, lanes=32)
    d2 = em.Description((rows,), [em.Operand(0, abi.F32, [1]), em.Operand(1, abi.F32, [1])], value=em.load(0) + em.load(1))
    k1, k2 = em.GenericKernel(dev, d1), em.GenericKernel(dev, d2)
    b = ScheduleBuilder()
    b.input("x", abi.F32, (rows, n))
    b.input("bias", abi.F32, (rows,))
    b.scratch("sums", abi.F32, (rows,))
    b.scratch("y", abi.F32, (rows,))
    for kern, refs in ((k1, {"generic.buffers[0]": "x", "generic.out": "sums"}),
                       (k2, {"generic.buffers[0]": "sums", "generic.buffers[1]": "bias", "generic.out": "y"})):
        s = abi.StageDesc()
        s.stage_kind, s.op = abi.STAGE_FUSED, abi.OP_GENERIC
        s.u.generic.kernel, s.u.generic.n_buffers = kern.h, len(refs) - 1
        b.stage(s, refs)
    b.root("y")
    prog = b.compile(dev)
    (out,) = prog.try_run({"x": x, "bias": bias})
    dev.sync()
    exp = orc.round_to(orc.DT_F32, np.array([np.sum(xv[r]) for r in range(rows)])) + bv
    assert nerr(view_tensor(out, dev.torch_device).cpu().numpy(), exp) <= 1e-5
    prog.close(); k1.close(); k2.close()


def test_nan_scan_names_the_buffer_and_debug_levels_print(dev):
    """SANIC_NANSCAN and SANIC_DEBUG are read once per process, so the run happens in a child process."""
    import os
    import subprocess
    import sys
    import ctypes as C
    from sanic_b200 import abi
    bad = torch.tensor([1.0, float("nan"), float("inf"), 2.0, -float("inf")], device=dev.torch_device)
    n = C.c_uint32(0)
    dev._check(dev.lib.sanic_count_nonfinite(dev.h, C.c_void_p(bad.data_ptr()), bad.numel(), abi.F32, dev.stream(), C.byref(n)), "count")
    assert n.value == 3
    dev._check(dev.lib.sanic_count_nonfinite(dev.h, C.c_void_p(bad.to(torch.bfloat16).data_ptr()), bad.numel(), abi.BF16, dev.stream(), C.byref(n)), "count")
    assert n.value == 3
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r'''
import sys, ctypes as C
sys.path.insert(0, %r); sys.path.insert(0, %r + "/tests")
import torch
from sanic_b200 import CudaDevice
from sanic_b200.schedule import ProgramError
from test_gpu_schedule import accumulate_schedule
dev = CudaDevice(0)
prog = accumulate_schedule(in_place=False).compile(dev)
w = torch.full((64, 128), 0.01, dtype=torch.bfloat16, device=dev.torch_device)
x = torch.ones(2, 128, dtype=torch.bfloat16, device=dev.torch_device)
acc = torch.zeros(2, 64, dtype=torch.float32, device=dev.torch_device)
st = torch.cuda.Stream(device=dev.torch_device)
rep = prog.capture({"w": w, "x": x, "acc": acc}, [(0, "acc")], stream=C.c_void_p(st.cuda_stream))
rep.step(stream=C.c_void_p(st.cuda_stream))
w[3, 5] = float("nan")
torch.cuda.synchronize()
try:
    rep.step(stream=C.c_void_p(st.cuda_stream))
    print("NO ERROR")
except ProgramError as e:
    print("ERROR:", e)
''' % (root, root)
    env = dict(os.environ, SANIC_NANSCAN="1", SANIC_DEBUG="3")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
    assert "ERROR:" in r.stdout and "non-finite" in r.stdout and "`acc" in r.stdout, r.stdout + r.stderr
    assert "sanic: captured 1 stage(s)" in r.stderr and "2 frozen step(s)" in r.stderr
    assert "sanic: step 1" in r.stderr and "ms on the device" in r.stderr
    assert "stage   0  contraction" in r.stderr


def test_one_shot_configurations_run_as_schedules(dev):
    """The graphs of the one-shot configurations compiled to schedules (one fused stage each; a fold over rotated operands
    has the RoPE cut in front) and run with inputs bound by name. Each result is checked against the oracle and is
    bit-identical to the direct kernel call."""
    from sanic_b200 import abi, schedules
    from sanic_b200.schedule import view_tensor
    td = dev.torch_device

    def run(builder, binds):
        prog = builder.compile(dev)
        (out,) = prog.try_run(binds)
        dev.sync()
        got = view_tensor(out, td).clone()
        prog.close()
        return got

    # configuration 1 at its own size: f32 attention, Q [256,64], K and V [1024,64], scale 1/8, no mask
    rng = orc.Xorshift(0xC1)
    qv, kv, vv = (orc.round_to(orc.DT_F32, rng.normal(1, 1, n, 64)) for n in (256, 1024, 1024))
    f32 = lambda a: torch.tensor(a, dtype=torch.float32, device=td)
    q, k, v = f32(qv), f32(kv), f32(vv)
    got = run(schedules.attention(1, 1, 1, 256, 1024, 64, storage=abi.F32), {"v": v, "q": q, "k": k})
    assert nerr(got.cpu().numpy(), orc.sdpa(qv, kv, vv)) <= 1e-5
    assert torch.equal(got, dev.attn_fwd_f32(q, k, v))

    # configuration 2's graph at a small size, both weight layouts
    for nk in (True, False):
        x, xv = bf16t(rng.normal(256, 512), dev)
        g, gv = bf16t(1.0 + 0.1 * rng.normal(512), dev)
        w, wv = bf16t(0.02 * rng.normal(*((768, 512) if nk else (512, 768))), dev)
        got = run(schedules.rmsnorm_gemm(256, 512, 768, w_is_nk=nk), {"x": x, "gamma": g, "w": w})
        assert nerr(got.float().cpu().numpy(), orc.rmsnorm_gemm(xv, gv, wv, eps=1e-5, w_is_nk=nk)) <= 2e-2
        assert torch.equal(got, dev.gemm_rmsnorm(x, g, w, w_is_nk=nk))

    # configuration 3's graph at a small size: RoPE on q and k, then the causal fold with a window, grouped heads
    B, Hq, Hkv, S, D = 1, 4, 2, 384, 64
    qb, qbv = bf16t(rng.normal(B, Hq, S, D), dev)
    kb, kbv = bf16t(rng.normal(B, Hkv, S, D), dev)
    vb, vbv = bf16t(rng.normal(B, Hkv, S, D), dev)
    inv = orc.rope_inv_freq(500000.0, D // 2)
    table = dev.rope_table(list(inv), S)
    got = run(schedules.attention(B, Hq, Hkv, S, S, D, storage=abi.BF16, causal=True, window=100, rope=True),
              {"q": qb, "k": kb, "v": vb, "rope_table": table})
    pos = np.arange(float(S))[None, None, :]
    qr = orc.round_to(orc.DT_BF16, orc.rope(qbv, pos, inv))
    kr = orc.round_to(orc.DT_BF16, orc.rope(kbv, pos, inv))
    rep = Hq // Hkv
    exp = orc.sdpa_window(qr, np.repeat(kr, rep, axis=1), np.repeat(vbv, rep, axis=1), 100)
    assert nerr(got.float().cpu().numpy(), exp) <= 2e-2
    assert torch.equal(got, dev.attn_fwd_bf16(dev.rope_bf16(qb, table), dev.rope_bf16(kb, table), vb, causal=True, window=100))

    # configuration 5's graph on one device at a small size: chunked fold + derived merge
    B, Hq, Hkv, S, D, splits = 2, 8, 2, 4096, 128, 5
    q1, q1v = bf16t(rng.normal(B, Hq, D), dev)
    k1, k1v = bf16t(rng.normal(B, Hkv, S, D), dev)
    v1, v1v = bf16t(rng.normal(B, Hkv, S, D), dev)
    got = run(schedules.splitkv_decode(B, Hq, Hkv, S, D, n_splits=splits), {"q": q1, "k": k1, "v": v1})
    rep = Hq // Hkv
    exp = orc.sdpa(q1v[:, :, None, :], np.repeat(k1v, rep, axis=1), np.repeat(v1v, rep, axis=1))[:, :, 0, :]
    assert nerr(got.cpu().numpy(), exp) <= 2e-2
