"""The generic emitter: carriers as expression programs -> generated CUDA kernels.

CPU part (no device): the numpy carrier oracle is pinned to the reference's known answers and to the C++ oracle;
every descriptor renders to CUDA C and the text compiles for sm_100a with the run-time compiler; malformed
programs are refused with a status. GPU part: the generated kernels, launched through the C ABI, against the
oracle on the same seeded inputs.

Tolerances: f32 storage 1e-5, bf16 storage 2e-2, of max |g - e| / (1 + |e|) against the f64 oracle; indices,
u32 stores and bf16 stores of exactly representable values bit-exact.
"""
import math

import numpy as np
import pytest

from oracle import carrier_eval as ce
from oracle import oracle as orc
from sanic_b200 import _abi as abi
from sanic_b200 import emitter as em

F32_TOL = 1e-5
BF16_TOL = 2e-2

_NAMES = {abi.X_CONST: "const", abi.X_LOAD: "load", abi.X_COORD: "coord", abi.X_ITEM: "item", abi.X_A: "a", abi.X_B: "b",
          abi.X_F: "f", abi.X_RESULT: "result", abi.X_ADD: "add", abi.X_SUB: "sub", abi.X_MUL: "mul", abi.X_DIV: "div",
          abi.X_MAX: "max", abi.X_MIN: "min", abi.X_LT: "lt", abi.X_NEG: "neg", abi.X_RECIP: "recip", abi.X_EXP: "exp",
          abi.X_LOG: "log", abi.X_SQRT: "sqrt", abi.X_TANH: "tanh", abi.X_SIN: "sin", abi.X_COS: "cos", abi.X_WHERE: "where",
          abi.X_GATHER: "gather", abi.X_GATHER_PAD: "gather_pad"}


def prog(e):
    """An expression tree as the oracle's postfix triples."""
    flat = []
    e.flatten(flat)
    out = []
    for op, arg, value in flat:
        if op == abi.X_ROUND:
            out.append(("round_bf16" if arg == abi.BF16 else "round_f32", 0, 0.0))
        else:
            out.append((_NAMES[op], arg, value))
    return out


def _ops(operands):
    return [dict(buffer=o.buffer, strides=list(o.strides), stream_stride=o.stream_stride, offset=o.offset,
                 inner_stride=o.inner_stride, gather_stride=o.gather_stride, gather_extent=o.gather_extent) for o in operands]


def oracle_fold(grid, stream, operands, buffers, carrier, epilogue=None, blocks=1):
    ops = _ops(operands)
    return ce.carrier_fold(grid, stream, ops, buffers, [prog(l) for l in carrier.leaves], [prog(e) for e in carrier.into],
                           [prog(e) for e in carrier.combine], list(carrier.identity), prog(carrier.project),
                           prog(epilogue) if epilogue is not None else None, blocks, list(carrier.leaf_inner))


def oracle_map(grid, operands, buffers, value):
    ops = _ops(operands)
    return ce.pointwise(grid, ops, buffers, prog(value))


def matmul_case(m, k, n, dtype=abi.F32):
    """c[i, j] = sum_s a[i, s] * b[s, j]: matmul = Reduce(Add, Map(Mul, view(a), view(b))) (src/ir.rs:1171-1223)."""
    operands = [em.Operand(0, dtype, [k, 0], 1), em.Operand(1, dtype, [0, 1], n)]
    return (m, n), k, operands, em.carrier_sum(em.load(0) * em.load(1))


def attention_case(L, S, E, Ev, scale, dtype=abi.F32, causal=False):
    """grid (query, value feature), stream = key; the score contraction is its own (inner) fold in the reference
    (in-body contraction); here the score leaf is given precomputed by a first kernel, or E == 1."""
    assert E == 1
    operands = [em.Operand(0, dtype, [1, 0], 0), em.Operand(1, dtype, [0, 0], 1), em.Operand(2, dtype, [0, 1], Ev)]
    score = em.load(0) * em.load(1) * scale
    if causal:   # where(i < j, -1e30, 0) added to the score (src/ir.rs:1511-1526)
        score = score + em.where(em.coord(0) < em.coord(2), -1e30, 0.0)
    return (L, Ev), S, operands, em.carrier_online_softmax(score, em.load(2))


def full_attention_case(B, Hq, Hkv, L, S, E, Ev, scale, dtype=abi.F32, causal=False):
    return em.attention(B, Hq, Hkv, L, S, E, Ev, scale, dtype, causal)


# ───────────────────────── CPU: oracle pins ─────────────────────────
def test_oracle_row_sums_and_matmul_known_answers():
    # tests/compile.rs:13-60, src/lib.rs:11-23
    x = np.array([[1.0, 2.0], [3.0, 4.0]])
    ops = [em.Operand(0, abi.F32, [2], 1)]
    assert list(oracle_fold((2,), 2, ops, [x], em.carrier_sum(em.load(0)))) == [3.0, 7.0]
    a, b = np.array([[1.0, 2.0], [3.0, 4.0]]), np.array([[5.0, 6.0], [7.0, 8.0]])
    grid, k, ops, car = matmul_case(2, 2, 2)
    assert oracle_fold(grid, k, ops, [a, b], car).ravel().tolist() == [19.0, 22.0, 43.0, 50.0]


def test_oracle_first_argmax_known_answer():
    # tests/compile.rs:139-171: argmax of [2,5,5,1,5,2,0,5] is 1 (first maximum), at every split
    x = np.array([2.0, 5.0, 5.0, 1.0, 5.0, 2.0, 0.0, 5.0])
    ops = [em.Operand(0, abi.F32, [], 1)]
    car = em.carrier_first_argmax(em.load(0), em.coord(0))
    for blocks in (1, 2, 3, 7, 8):
        assert float(oracle_fold((), 8, ops, [x], car, blocks=blocks)) == 1.0


def test_oracle_direct_attention_known_answer():
    # tests/compile.rs:236-261: Q = K = I, V = [[2,3],[5,7]], default scale; via two folds: scores, then (m, l, o)
    q = k = np.eye(2)
    v = np.array([[2.0, 3.0], [5.0, 7.0]])
    s_ops = [em.Operand(0, abi.F32, [2, 0], 1), em.Operand(1, abi.F32, [0, 2], 1)]
    scores = oracle_fold((2, 2), 2, s_ops, [q, k], em.carrier_sum(em.load(0) * em.load(1)))
    a_ops = [em.Operand(0, abi.F32, [2, 0], 1), em.Operand(1, abi.F32, [0, 1], 2)]
    car = em.carrier_online_softmax(em.load(0) * (1.0 / math.sqrt(2.0)), em.load(1))
    out = oracle_fold((2, 2), 2, a_ops, [scores, v], car).ravel()
    literal = np.array([2.990715, 4.3209534, 4.009285, 5.6790466])
    assert np.all(np.abs(out - literal) < 1e-6)
    assert np.allclose(out, orc.sdpa(q, k, v).ravel(), rtol=0, atol=1e-14)


def test_oracle_split_law_and_cpp_oracle_agree():
    # tests/group.rs:48-116: the split fold equals the straight fold for blocks {1,2,3,7,9}; and the numpy
    # evaluator equals the C++ oracle's attention on the same seeded tensors
    L, S, Ev = 5, 9, 4
    g = orc.Xorshift(0xA11CE)
    q, k, v = g.normal(L, 1), g.normal(S, 1), g.normal(S, Ev)
    grid, n, ops, car = attention_case(L, S, 1, Ev, 0.7)
    ref = oracle_fold(grid, n, ops, [q, k, v], car)
    assert np.allclose(ref, orc.sdpa(q, k, v, scale=0.7), rtol=0, atol=1e-13)
    for blocks in (2, 3, 7, 9):
        assert np.allclose(oracle_fold(grid, n, ops, [q, k, v], car, blocks=blocks), ref, rtol=0, atol=1e-13)
    grid, n, ops, car = attention_case(L, S, 1, Ev, 0.7, causal=True)
    assert np.allclose(oracle_fold(grid, n, ops, [q, k, v], car), orc.sdpa(q, k, v, scale=0.7, is_causal=True), rtol=0, atol=1e-13)


def test_oracle_fused_attention_reads_only_qkv():
    # tests/oracle.rs:90-151 shapes (2,3,5,7,4,6) seed 0xA11CE, and the GQA 4/2 known answer of tests/nn.rs:108-137
    g = orc.Xorshift(0xA11CE)
    B, H, L, S, E, Ev = 2, 3, 5, 7, 4, 6
    q, k, v = g.normal(B, H, L, E), g.normal(B, H, S, E), g.normal(B, H, S, Ev)
    for causal in (False, True):
        grid, n, ops, car = full_attention_case(B, H, H, L, S, E, Ev, 0.5, causal=causal)
        got = oracle_fold(grid, n, ops, [q, k, v], car, blocks=3).reshape(B, H, L, Ev)
        assert np.allclose(got, orc.sdpa(q, k, v, scale=0.5, is_causal=causal), rtol=0, atol=1e-13)
    q = np.ones((1, 4, 1, 1)); k = np.ones((1, 2, 1, 1)); v = np.array([10.0, 20.0]).reshape(1, 2, 1, 1)
    grid, n, ops, car = full_attention_case(1, 4, 2, 1, 1, 1, 1, 1.0)
    assert oracle_fold(grid, n, ops, [q, k, v], car).ravel().tolist() == [10.0, 10.0, 20.0, 20.0]


def test_oracle_overflow_magnitude_carriers_stay_finite():
    # tests/laws.rs:444-505: scores centred far outside exp's range fold to the same answer as centred ones
    g = orc.Xorshift(0x0F10)
    base, v = g.normal(12), g.normal(12, 3)
    ops = [em.Operand(0, abi.F32, [0], 1), em.Operand(1, abi.F32, [1], 3)]
    car = em.carrier_online_softmax(em.load(0), em.load(1))
    want = oracle_fold((3,), 12, ops, [base, v], car)
    for centre in (50.0, 300.0, 710.0, -710.0):
        got = oracle_fold((3,), 12, ops, [base + centre, v], car, blocks=3)
        assert np.all(np.isfinite(got)) and np.allclose(got, want, rtol=0, atol=1e-9)


# ───────────────────────── CPU: rendering and compiling ─────────────────────────
def all_descriptions():
    out = {}
    grid, k, ops, car = matmul_case(8, 16, 4, abi.BF16)
    out["scalar fold"] = em.Description(grid, ops, carrier=car, stream=k, out_dtype=abi.BF16)
    out["cooperative fold"] = em.Description(grid, ops, carrier=car, stream=k, lanes=32)
    out["interleaved fold"] = em.Description(grid, ops, carrier=car, stream=k, lanes=32, interleave=True)
    g5, n5, o5, c5 = full_attention_case(2, 4, 2, 8, 24, 16, 8, 0.25, abi.BF16, causal=True)
    out["fused attention"] = em.Description(g5, o5, carrier=c5, stream=n5, lanes=32, out_dtype=abi.BF16)
    out["lane-distributed output axis"] = em.Description(g5, o5, carrier=c5, stream=n5, lanes=32, lane_axis=True)
    out["lane axis, stream over 4 warps"] = em.Description(g5, o5, carrier=c5, stream=n5, lanes=32, warps=4, lane_axis=True)
    out["four warps per point"] = em.Description(grid, ops, carrier=car, stream=k, lanes=32, warps=4)
    grid, n, ops, car = attention_case(6, 40, 1, 8, 0.5, causal=True)
    out["online softmax"] = em.Description(grid, ops, carrier=car, stream=n, lanes=32)
    ops = [em.Operand(0, abi.F32, [1], 0), em.Operand(1, abi.BF16, [1], 0)]
    silu = em.load(0) * em.recip(1.0 + em.exp(-em.load(0)))      # silu(x) = x * 1/(1+exp(-x)), src/ir.rs:1500-1509
    out["pointwise"] = em.Description((64,), ops, value=silu * em.load(1), out_dtype=abi.BF16)
    ops = [em.Operand(0, abi.F32, [], 1)]
    out["argmax"] = em.Description((), ops, carrier=em.carrier_first_argmax(em.load(0), em.coord(0)), stream=100, out_dtype=abi.U32)
    ops = [em.Operand(0, abi.I4, [128], 1), em.Operand(1, abi.BF16, [2], 0), em.Operand(2, abi.BF16, [0], 1)]
    out["int4 leaf"] = em.Description((4,), ops, carrier=em.carrier_sum(em.load(0) * em.load(1) * em.load(2)), stream=128)
    ops = [em.Operand(0, abi.BF16, [0, 1], gather_stride=32, gather_extent=100), em.Operand(1, abi.F32, [1, 0])]
    out["gather"] = em.Description((4, 32), ops, value=em.gather(0, em.load(1)))
    ops = [em.Operand(0, abi.F32, [0, 1]), em.Operand(1, abi.F32, [0, 0])]
    hit = (em.coord(0) < em.load(1) + 1.0) * (em.load(1) < em.coord(0) + 1.0)
    out["in-place row write"] = em.Description((16, 8), ops, value=em.load(0), store_if=hit, out_dtype=abi.BF16)
    g, win, ops, car = em.conv2d(2, 3, 9, 8, 4, 3, 3, dtype=abi.BF16)
    out["convolution over a three-axis window"] = em.Description(g, ops, carrier=car, stream=win, lanes=32)
    g, win, ops, car = em.pool2d(2, 3, 8, 8, 2, 2)
    out["pooling over a two-axis window"] = em.Description(g, ops, carrier=car, stream=win)
    g, win, ops, car = em.conv2d(1, 2, 6, 6, 3, 3, 3, padding=1)
    out["padded convolution"] = em.Description(g, ops, carrier=car, stream=win, lanes=32)
    return out


def test_oracle_gather_rounds_then_checks_bounds():
    # src/interp.rs:378-379: the index is round()ed (half away from zero), then bounds-checked
    table = np.arange(12.0).reshape(4, 3)
    idx = np.array([0.4, 2.5, 1.49, 3.0])
    ops = [em.Operand(0, abi.F32, [0, 1], gather_stride=3, gather_extent=4), em.Operand(1, abi.F32, [1, 0])]
    got = oracle_map((4, 3), ops, [table, idx], em.gather(0, em.load(1)))
    assert got.tolist() == [[0, 1, 2], [9, 10, 11], [3, 4, 5], [9, 10, 11]]
    with pytest.raises(IndexError):
        oracle_map((4, 3), ops, [table, np.array([0.0, 3.5, 0.0, 0.0])], em.gather(0, em.load(1)))


def test_every_description_renders():
    for name, d in all_descriptions().items():
        text = em.source(d)
        assert 'extern "C" __global__' in text and "sanic_generic" in text, name
        if d.desc.stream > 0:
            assert "for (long long s" in text, name
        if d.desc.lanes == 32 and d.desc.lane_axis:
            assert "__shfl_xor_sync" in text and "const bool active" in text, name    # the shared score, summed over lanes
        elif d.desc.lanes == 32:
            assert "__shfl_down_sync" in text, name
        else:
            assert "__shfl" not in text.split("sanic_generic(")[1], name


def test_every_generated_kernel_compiles_for_sm_100a():
    for name, d in all_descriptions().items():
        assert em.compiles(d) > 0, name


def test_malformed_programs_are_refused():
    ops = [em.Operand(0, abi.F32, [1], 1)]
    # A(0) outside a combine; an operand that does not exist; the stream coordinate in a projection
    bad = [em.Carrier([em.load(0)], [em.A(0)], [em.A(0) + em.B(0)], [0.0], em.F(0)),
           em.Carrier([em.load(3)], [em.item(0)], [em.A(0) + em.B(0)], [0.0], em.F(0)),
           em.Carrier([em.load(0)], [em.item(0)], [em.A(0) + em.B(0)], [0.0], em.F(0) + em.coord(1))]
    for car in bad:
        with pytest.raises(ValueError):
            em.source(em.Description((4,), ops, carrier=car, stream=8))
    with pytest.raises(ValueError):
        em.Description((4,), ops, carrier=bad[0], stream=0)
    d = em.Description((4,), ops, carrier=em.carrier_sum(em.load(0)), stream=8, lanes=7)
    with pytest.raises(ValueError):
        em.source(d)
    # a streamed window: one stride per window axis on every operand, 2 or 3 axes, and a coordinate that exists
    with pytest.raises(ValueError):
        em.Description((4,), ops, carrier=em.carrier_sum(em.load(0)), stream=(2, 4))
    with pytest.raises(ValueError):
        em.Description((4,), [em.Operand(0, abi.F32, [1], stream_strides=[4, 1])], carrier=em.carrier_sum(em.load(0)), stream=(2, 2, 2, 2))
    wops = [em.Operand(0, abi.F32, [8], stream_strides=[4, 1])]
    assert "% 4LL" in em.source(em.Description((4,), wops, carrier=em.carrier_sum(em.load(0) * em.coord(3)), stream=(2, 4)))
    with pytest.raises(ValueError):
        em.source(em.Description((4,), wops, carrier=em.carrier_sum(em.load(0) * em.coord(5)), stream=(2, 4)))


# ───────────────────────── GPU parity ─────────────────────────
@pytest.fixture(scope="module")
def dev():
    from sanic_b200 import CudaDevice
    return CudaDevice(0)


def nerr(got, exp):
    got, exp = np.asarray(got, np.float64), np.asarray(exp, np.float64)
    assert got.shape == exp.shape, (got.shape, exp.shape)
    assert np.all(np.isfinite(got)), "non-finite values in the GPU result"
    return float(np.max(np.abs(got - exp) / (1.0 + np.abs(exp))))


def on_device(dev, x, dtype):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float64)).to(dev.torch_device)
    return t.to({abi.F32: torch.float32, abi.BF16: torch.bfloat16}[dtype]).contiguous()


def run_kernel(dev, desc, buffers, grid, out_dtype=abi.F32):
    import torch
    out = torch.empty(max(1, int(np.prod(grid, dtype=np.int64))), device=dev.torch_device,
                      dtype={abi.F32: torch.float32, abi.BF16: torch.bfloat16, abi.U32: torch.int32}[out_dtype])
    k = em.GenericKernel(dev, desc)
    k(buffers, out)
    dev.sync()
    k.close()
    if out_dtype == abi.U32:
        return out.cpu().numpy().view(np.uint32).reshape(grid)
    return out.float().cpu().numpy().astype(np.float64).reshape(grid)


@pytest.mark.gpu
@pytest.mark.parametrize("lanes,interleave", [(1, False), (32, False), (32, True)])
@pytest.mark.parametrize("dtype", [abi.F32, abi.BF16])
def test_generic_matmul_fold(dev, lanes, interleave, dtype):
    m, k, n = 37, 300, 19
    g = orc.Xorshift(0x9E0)
    a, b = g.normal(m, k), g.normal(k, n)
    if dtype == abi.BF16:
        a, b = orc.round_to(orc.DT_BF16, a), orc.round_to(orc.DT_BF16, b)
    else:
        a, b = orc.round_to(orc.DT_F32, a), orc.round_to(orc.DT_F32, b)
    grid, stream, ops, car = matmul_case(m, k, n, dtype)
    want = oracle_fold(grid, stream, ops, [a, b], car)
    d = em.Description(grid, ops, carrier=car, stream=stream, lanes=lanes, interleave=interleave)
    got = run_kernel(dev, d, [on_device(dev, a, dtype), on_device(dev, b, dtype)], grid)
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("lanes,interleave", [(1, False), (32, False), (32, True)])
@pytest.mark.parametrize("stream", [1, 7, 33, 500])
def test_generic_online_softmax_fold(dev, lanes, interleave, stream):
    L, Ev = 21, 16
    g = orc.Xorshift(0xF1A5)
    q, k, v = (orc.round_to(orc.DT_F32, x) for x in (g.normal(L, 1), g.normal(stream, 1) * 3.0, g.normal(stream, Ev)))
    grid, n, ops, car = attention_case(L, stream, 1, Ev, 0.9, causal=True)
    want = oracle_fold(grid, n, ops, [q, k, v], car)
    d = em.Description(grid, ops, carrier=car, stream=n, lanes=lanes, interleave=interleave)
    got = run_kernel(dev, d, [on_device(dev, x, abi.F32) for x in (q, k, v)], grid)
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("warps,interleave", [(2, False), (8, False), (4, True)])
@pytest.mark.parametrize("stream", [5, 40, 257, 3000])
def test_generic_block_level_split(dev, warps, interleave, stream):
    # the streamed axis split over the threads of a block: lanes, then warps (src/plan.rs:434-488); the answer is the
    # straight fold's, for the online-softmax carrier and for the first-argmax carrier (bit-exact)
    L, Ev = 7, 8
    g = orc.Xorshift(0x5B17)
    q, k, v = (orc.round_to(orc.DT_F32, x) for x in (g.normal(L, 1), g.normal(stream, 1) * 2.0, g.normal(stream, Ev)))
    grid, n, ops, car = attention_case(L, stream, 1, Ev, 0.8, causal=True)
    want = oracle_fold(grid, n, ops, [q, k, v], car)
    d = em.Description(grid, ops, carrier=car, stream=n, lanes=32, warps=warps, interleave=interleave)
    got = run_kernel(dev, d, [on_device(dev, x, abi.F32) for x in (q, k, v)], grid)
    assert nerr(got, want) <= F32_TOL
    x = np.round(g.normal(3, stream) * 2.0) / 2.0
    ops = [em.Operand(0, abi.F32, [stream], 1)]
    car = em.carrier_first_argmax(em.load(0), em.coord(1))
    d = em.Description((3,), ops, carrier=car, stream=stream, lanes=32, warps=warps, interleave=interleave, out_dtype=abi.U32)
    got = run_kernel(dev, d, [on_device(dev, x, abi.F32)], (3,), abi.U32)
    assert got.tolist() == np.argmax(x, axis=1).tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("lanes,warps", [(1, 1), (32, 1), (32, 4)])
def test_generic_fused_attention_reads_only_qkv(dev, causal, lanes, warps):
    # one generated kernel for softmax(QK^T * scale + mask) V with grouped-query heads, against the C++ oracle
    B, Hq, Hkv, L, S, E, Ev = 2, 4, 2, 9, 70, 16, 8
    g = orc.Xorshift(0xF1A5)
    q, k, v = (orc.round_to(orc.DT_F32, t) for t in (g.normal(B, Hq, L, E), g.normal(B, Hkv, S, E), g.normal(B, Hkv, S, Ev)))
    grid, n, ops, car = full_attention_case(B, Hq, Hkv, L, S, E, Ev, 0.25, causal=causal)
    want = orc.sdpa(q, k, v, scale=0.25, is_causal=causal, enable_gqa=True)
    d = em.Description(grid, ops, carrier=car, stream=n, lanes=lanes, warps=warps)
    got = run_kernel(dev, d, [on_device(dev, t, abi.F32) for t in (q, k, v)], grid).reshape(B, Hq, L, Ev)
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("warps", [1, 3, 8])
@pytest.mark.parametrize("Ev,S", [(8, 70), (40, 5), (64, 200)])
def test_generic_lane_distributed_output_axis(dev, warps, Ev, S):
    # the value-feature axis over the lanes: the score is computed once per warp, each lane owns o[e]
    B, Hq, Hkv, L, E = 1, 4, 2, 6, 48
    g = orc.Xorshift(0x1A2E)
    q, k, v = (orc.round_to(orc.DT_F32, t) for t in (g.normal(B, Hq, L, E), g.normal(B, Hkv, S, E), g.normal(B, Hkv, S, Ev)))
    grid, n, ops, car = full_attention_case(B, Hq, Hkv, L, S, E, Ev, 0.2, causal=True)
    want = orc.sdpa(q, k, v, scale=0.2, is_causal=True, enable_gqa=True)
    d = em.Description(grid, ops, carrier=car, stream=n, lanes=32, warps=warps, lane_axis=True)
    got = run_kernel(dev, d, [on_device(dev, t, abi.F32) for t in (q, k, v)], grid).reshape(B, Hq, L, Ev)
    assert nerr(got, want) <= F32_TOL
    # a carrier without a contracted leaf on the same schedule: row-wise matmul, the output column over the lanes
    m, kk = 5, 90
    a, b = (orc.round_to(orc.DT_F32, t) for t in (g.normal(m, kk), g.normal(kk, Ev)))
    grid, stream, ops, car = matmul_case(m, kk, Ev)
    d = em.Description(grid, ops, carrier=car, stream=stream, lanes=32, warps=warps, lane_axis=True)
    got = run_kernel(dev, d, [on_device(dev, a, abi.F32), on_device(dev, b, abi.F32)], grid)
    assert nerr(got, oracle_fold(grid, stream, ops, [a, b], car)) <= F32_TOL


@pytest.mark.gpu
def test_generic_attention_at_the_first_config_matches_the_specialised_kernel(dev):
    # Q[256, 64], K, V[1024, 64] f32, scale 1/8, no mask: the generated kernel, the hand-written f32 fold and the oracle
    import torch
    g = orc.Xorshift(0xC1)
    q, k, v = (orc.round_to(orc.DT_F32, t) for t in (g.normal(1, 1, 256, 64), g.normal(1, 1, 1024, 64), g.normal(1, 1, 1024, 64)))
    grid, n, ops, car = full_attention_case(1, 1, 1, 256, 1024, 64, 64, 0.125)
    want = orc.sdpa(q, k, v, scale=0.125)
    tq, tk, tv = (on_device(dev, t, abi.F32) for t in (q, k, v))
    for kw in (dict(interleave=True), dict(lane_axis=True, warps=4)):
        got = run_kernel(dev, em.Description(grid, ops, carrier=car, stream=n, lanes=32, **kw), [tq, tk, tv], grid)
        assert nerr(got.reshape(1, 1, 256, 64), want) <= F32_TOL
    hand = dev.attn_fwd_f32(tq, tk, tv, scale=0.125).cpu().numpy().astype(np.float64)
    assert nerr(hand, want) <= F32_TOL


@pytest.mark.gpu
def test_generic_overflow_magnitude_scores(dev):
    # tests/laws.rs:444-505 at f32 range: exp(centre) alone overflows f32 from 89 on; the carrier does not
    g = orc.Xorshift(0x0F10)
    base, v = g.normal(64), orc.round_to(orc.DT_F32, g.normal(64, 3))
    ops = [em.Operand(0, abi.F32, [0], 1), em.Operand(1, abi.F32, [1], 3)]
    car = em.carrier_online_softmax(em.load(0), em.load(1))
    for centre in (50.0, 300.0, -3000.0):
        s = orc.round_to(orc.DT_F32, base + centre)
        want = oracle_fold((3,), 64, ops, [s, v], car)
        d = em.Description((3,), ops, carrier=car, stream=64, lanes=32)
        got = run_kernel(dev, d, [on_device(dev, s, abi.F32), on_device(dev, v, abi.F32)], (3,))
        assert nerr(got, want) <= 2e-5     # the scores themselves carry an f32 rounding of 2^-24 * |centre|... absorbed by the shift


@pytest.mark.gpu
@pytest.mark.parametrize("lanes", [1, 32])
def test_generic_logsumexp_and_deferred_norm(dev, lanes):
    rows, n, outs = 9, 200, 5
    g = orc.Xorshift(0x524D53)
    x = orc.round_to(orc.DT_BF16, g.normal(rows, n))
    gamma = orc.round_to(orc.DT_BF16, 1.0 + 0.1 * g.normal(n))
    w = orc.round_to(orc.DT_BF16, 0.05 * g.normal(n, outs))
    ops = [em.Operand(0, abi.BF16, [n], 1)]
    car = em.carrier_logsumexp(em.load(0))
    want = oracle_fold((rows,), n, ops, [x], car)
    got = run_kernel(dev, em.Description((rows,), ops, carrier=car, stream=n, lanes=lanes), [on_device(dev, x, abi.BF16)], (rows,))
    assert nerr(got, want) <= F32_TOL
    # RMSNorm folded into the projection: (sum x^2, sum x*gamma*w), one division at the end (tests/laws.rs:620-646)
    ops = [em.Operand(0, abi.BF16, [n, 0], 1), em.Operand(1, abi.BF16, [0, 0], 1), em.Operand(2, abi.BF16, [0, 1], outs)]
    car = em.carrier_deferred_norm(em.load(0), em.load(1) * em.load(2), n, 1e-5)
    want = oracle_fold((rows, outs), n, ops, [x, gamma, w], car)
    assert np.allclose(want, orc.rmsnorm_gemm(x, gamma, w, 1e-5), rtol=0, atol=1e-12)
    d = em.Description((rows, outs), ops, carrier=car, stream=n, lanes=lanes)
    got = run_kernel(dev, d, [on_device(dev, t, abi.BF16) for t in (x, gamma, w)], (rows, outs))
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("lanes,interleave", [(1, False), (32, False), (32, True)])
def test_generic_first_argmax_is_bit_exact(dev, lanes, interleave):
    import torch
    rows, n = 6, 1000
    g = orc.Xorshift(0xA46)
    x = np.round(g.normal(rows, n) * 4.0) / 4.0            # many exact ties
    x[0, :] = 1.0                                          # all tied: index 0
    x[1, 999] = 100.0                                      # the last element
    ops = [em.Operand(0, abi.F32, [n], 1)]
    car = em.carrier_first_argmax(em.load(0), em.coord(1))
    d = em.Description((rows,), ops, carrier=car, stream=n, lanes=lanes, interleave=interleave, out_dtype=abi.U32)
    got = run_kernel(dev, d, [on_device(dev, x, abi.F32)], (rows,), abi.U32)
    assert got.tolist() == np.argmax(x, axis=1).tolist()
    assert got.tolist() == orc.argmax(x).astype(np.int64).tolist()


@pytest.mark.gpu
def test_generic_int4_leaf_contraction(dev):
    # tests/metal.rs:1178-1269: unsigned q+8 nibbles, low nibble = even element, one scale per 64 along k
    import torch
    outs, k, group = 12, 256, 64
    g = orc.Xorshift(0x144A16)
    q = np.floor(g.uniform(outs * k).reshape(outs, k) * 8.0).clip(-8, 7)
    scales = orc.round_to(orc.DT_BF16, 0.01 + 0.02 * np.abs(g.normal(outs, k // group)))
    x = orc.round_to(orc.DT_BF16, g.normal(k))
    packed = orc.w4_pack(q.reshape(-1))
    # operand 1 steps one scale per 64 stream steps: express the group index through a widened scale view instead
    wide = np.repeat(scales, group, axis=1)
    ops = [em.Operand(0, abi.I4, [k], 1), em.Operand(1, abi.BF16, [k], 1), em.Operand(2, abi.BF16, [0], 1)]
    car = em.carrier_sum(em.load(0) * em.load(1) * em.load(2))
    want = oracle_fold((outs,), k, ops, [q, wide, x], car)
    assert np.allclose(want, orc.w4_gemv(packed, scales, x, outs, group), rtol=0, atol=1e-12)
    d = em.Description((outs,), ops, carrier=car, stream=k, lanes=32, interleave=True)
    bufs = [torch.from_numpy(packed).to(dev.torch_device), on_device(dev, wide, abi.BF16), on_device(dev, x, abi.BF16)]
    got = run_kernel(dev, d, bufs, (outs,))
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
def test_generic_pointwise_cone_and_stores(dev):
    import torch
    n = 4096
    g = orc.Xorshift(0x51D3)
    gate = orc.round_to(orc.DT_F32, g.normal(n) * 3.0)
    up = orc.round_to(orc.DT_BF16, g.normal(n))
    ops = [em.Operand(0, abi.F32, [1], 0), em.Operand(1, abi.BF16, [1], 0)]
    silu = em.load(0) * em.recip(1.0 + em.exp(-em.load(0)))
    value = silu * em.load(1)
    want = oracle_map((n,), ops, [gate, up], value)
    got = run_kernel(dev, em.Description((n,), ops, value=value), [on_device(dev, gate, abi.F32), on_device(dev, up, abi.BF16)], (n,))
    assert nerr(got, want) <= F32_TOL
    # a bf16 store is the RNE rounding of the f32 value: RoundTo in the graph then an exact store
    value_r = em.round_to(em.load(0) * 0.37, abi.BF16)
    want = orc.round_to(orc.DT_BF16, orc.round_to(orc.DT_F32, gate.astype(np.float32) * np.float32(0.37)))
    got = run_kernel(dev, em.Description((n,), ops, value=value_r, out_dtype=abi.BF16), [on_device(dev, gate, abi.F32), on_device(dev, up, abi.BF16)], (n,), abi.BF16)
    assert np.array_equal(got, want)
    # coordinates, comparison, where, and a transposed broadcast read: out[i, j] = where(j < i + 1, x[j, i], -1e30)
    r = 33
    x = orc.round_to(orc.DT_F32, g.normal(r, r))
    ops = [em.Operand(0, abi.F32, [1, r], 0)]
    value = em.where(em.coord(1) < em.coord(0) + 1.0, em.load(0), -1e30)
    want = oracle_map((r, r), ops, [x], value)
    got = run_kernel(dev, em.Description((r, r), ops, value=value), [on_device(dev, x, abi.F32)], (r, r))
    assert np.array_equal(got, want.astype(np.float32).astype(np.float64))
    # sin / cos / tanh / sqrt / log / max / min / div over the basis
    ops = [em.Operand(0, abi.F32, [1], 0)]
    value = em.sin(em.load(0)) * em.cos(em.load(0)) + em.tanh(em.load(0)) / em.sqrt(em.maximum(em.load(0) * em.load(0), 0.25)) \
        - em.log(1.0 + em.minimum(em.load(0) * em.load(0), 9.0))
    want = oracle_map((n,), ops, [gate], value)
    got = run_kernel(dev, em.Description((n,), ops, value=value), [on_device(dev, gate, abi.F32)], (n,))
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
def test_generic_gather_stage(dev):
    # the embedding: token ids travel as floats, Gather rounds them (src/interp.rs:378-379, examples/llama3_2.rs:112-121)
    import torch
    vocab, hidden, batch = 300, 64, 5
    g = orc.Xorshift(0xE3B)
    table = orc.round_to(orc.DT_BF16, g.normal(vocab, hidden))
    tokens = np.array([0.0, 299.0, 17.4, 17.5, 123.0])          # 17.4 -> 17, 17.5 -> 18
    ops = [em.Operand(0, abi.BF16, [0, 1], gather_stride=hidden, gather_extent=vocab), em.Operand(1, abi.F32, [1, 0])]
    value = em.gather(0, em.load(1))
    want = oracle_map((batch, hidden), ops, [table, tokens], value)
    assert np.array_equal(want, table[[0, 299, 17, 18, 123]])
    d = em.Description((batch, hidden), ops, value=value)
    got = run_kernel(dev, d, [on_device(dev, table, abi.BF16), on_device(dev, tokens, abi.F32)], (batch, hidden))
    assert np.array_equal(got, want)
    # an index out of range reads 0 and the next synchronisation reports it; the context stays usable
    from sanic_b200.backend import RunError
    bad = on_device(dev, np.array([0.0, 300.0, 1.0, 2.0, 3.0]), abi.F32)
    out = torch.empty(batch * hidden, device=dev.torch_device)
    k = em.GenericKernel(dev, d)
    k([on_device(dev, table, abi.BF16), bad], out)
    with pytest.raises(RunError):
        dev.sync()
    assert float(out.view(batch, hidden)[1].abs().max()) == 0.0
    k([on_device(dev, table, abi.BF16), on_device(dev, tokens, abi.F32)], out)
    dev.sync()
    assert np.array_equal(out.cpu().numpy().reshape(batch, hidden).astype(np.float64), want)
    k.close()


@pytest.mark.gpu
def test_generic_in_place_row_write(dev):
    # update_cache = where((idx < pos+1) * (pos < idx+1), current, cache) written into the cache's own buffer: only row
    # `pos` is stored, the rest of the cache is neither loaded nor written (src/nn.rs:208-212, src/emit_metal.rs:1118-1178)
    import torch
    ctx_len, d_head, pos = 40, 16, 23
    g = orc.Xorshift(0xCAC4E)
    cache = orc.round_to(orc.DT_BF16, g.normal(ctx_len, d_head))
    cur = orc.round_to(orc.DT_F32, g.normal(d_head))
    ops = [em.Operand(0, abi.F32, [0, 1]), em.Operand(1, abi.F32, [0, 0])]
    hit = (em.coord(0) < em.load(1) + 1.0) * (em.load(1) < em.coord(0) + 1.0)
    d = em.Description((ctx_len, d_head), ops, value=em.load(0), store_if=hit, out_dtype=abi.BF16)
    t_cache = on_device(dev, cache, abi.BF16).reshape(-1)
    k = em.GenericKernel(dev, d)
    k([on_device(dev, cur, abi.F32), on_device(dev, np.array([float(pos)]), abi.F32)], t_cache)
    dev.sync()
    k.close()
    want = cache.copy()
    want[pos] = orc.round_to(orc.DT_BF16, cur)
    assert np.array_equal(t_cache.float().cpu().numpy().reshape(ctx_len, d_head).astype(np.float64), want)


@pytest.mark.gpu
def test_generic_fold_with_epilogue(dev):
    # a residual add rendered in the fold kernel after the projection (src/partition.rs:2726-2750)
    m, k, n = 10, 64, 12
    g = orc.Xorshift(0xE91)
    a, b, res = (orc.round_to(orc.DT_F32, t) for t in (g.normal(m, k), g.normal(k, n), g.normal(m, n)))
    grid, stream, ops, car = matmul_case(m, k, n)
    ops = ops + [em.Operand(2, abi.F32, [n, 1], 0)]
    epi = em.result() + em.load(2)
    want = oracle_fold(grid, stream, ops, [a, b, res], car, epilogue=epi)
    d = em.Description(grid, ops, carrier=car, stream=stream, epilogue=epi, lanes=32)
    got = run_kernel(dev, d, [on_device(dev, t, abi.F32) for t in (a, b, res)], grid)
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
def test_generic_stage_in_a_program(dev):
    # a stage list whose stages are generated kernels: scores fold, then the (m, l, o) fold; run and replayed
    import ctypes as C
    import torch
    L, S, E, Ev = 16, 48, 8, 8
    g = orc.Xorshift(0xC0FFEE)
    q, k, v = (orc.round_to(orc.DT_F32, t) for t in (g.normal(L, E), g.normal(S, E), g.normal(S, Ev)))
    s_ops = [em.Operand(0, abi.F32, [E, 0], 1), em.Operand(1, abi.F32, [0, E], 1)]
    d1 = em.Description((L, S), s_ops, carrier=em.carrier_sum(em.load(0) * em.load(1)), stream=E)
    a_ops = [em.Operand(0, abi.F32, [S, 0], 1), em.Operand(1, abi.F32, [0, 1], Ev)]
    score = em.load(0) * (1.0 / math.sqrt(E)) + em.where(em.coord(0) < em.coord(2), -1e30, 0.0)
    d2 = em.Description((L, Ev), a_ops, carrier=em.carrier_online_softmax(score, em.load(1)), stream=S, lanes=32)
    k1, k2 = em.GenericKernel(dev, d1), em.GenericKernel(dev, d2)
    tq, tk, tv = (on_device(dev, t, abi.F32) for t in (q, k, v))
    scores = torch.empty(L * S, device=dev.torch_device)
    out = torch.zeros(L * Ev, device=dev.torch_device)
    stages = (abi.StageDesc * 2)()
    for st, kern, bufs, o in ((stages[0], k1, [tq, tk], scores), (stages[1], k2, [scores, tv], out)):
        st.stage_kind, st.op = abi.STAGE_FUSED, abi.OP_GENERIC
        st.u.generic.kernel = kern.h
        for i, b in enumerate(bufs):
            st.u.generic.buffers[i] = b.data_ptr()
        st.u.generic.n_buffers = len(bufs)
        st.u.generic.out = o.data_ptr()
    prog_h = C.c_void_p()
    dev._check(dev.lib.sanic_program_create(dev.h, stages, 2, C.byref(prog_h)), "program_create")
    want = orc.sdpa(q, k, v, is_causal=True)
    dev._check(dev.lib.sanic_program_run(prog_h, dev.stream()), "program_run")
    dev.sync()
    assert nerr(out.cpu().numpy().reshape(L, Ev), want) <= F32_TOL
    out.zero_()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev.torch_device)       # a capture needs a stream of its own
    with torch.cuda.stream(side):
        dev._check(dev.lib.sanic_program_capture(prog_h, dev.stream()), "program_capture")
        dev._check(dev.lib.sanic_program_step(prog_h, dev.stream(), None), "program_step")
        dev.sync()
    assert nerr(out.cpu().numpy().reshape(L, Ev), want) <= F32_TOL
    dev.lib.sanic_program_destroy(prog_h)
    k1.close(); k2.close()


@pytest.mark.gpu
def test_hand_written_merge_equals_the_carriers_own_combine(dev):
    """The (m, l, o) merge the hand-written kernels use (`sanic_carrier_merge`, the stage 2 of every split fold and of the
    multi-device step) against the SAME carrier's combine rendered from its expression programs: the generic emitter folds
    the axis of partial accumulators with into = identity, combine = the derived one (src/derive.rs:1700-1713), project =
    o / l. Equal to f32 rounding, including sides whose maximum is -inf (identity partials)."""
    import torch
    n_parts, rows, D = 7, 24, 16
    g = orc.Xorshift(0x3E26E)
    parts = np.empty((n_parts, rows, D + 2))
    parts[..., 0] = g.uniform(n_parts, rows) * 30.0
    parts[..., 1] = np.abs(g.uniform(n_parts, rows)) * 40.0 + 0.1
    parts[..., 2:] = g.uniform(n_parts, rows, D) * 25.0
    parts[2, :, 0] = -np.inf; parts[2, :, 1] = 0.0; parts[2, :, 2:] = 0.0          # an all-masked part
    parts[0, 5, 0] = -np.inf; parts[0, 5, 1] = 0.0; parts[0, 5, 2:] = 0.0          # ... also as the leftmost one
    parts = orc.round_to(orc.DT_F32, parts)
    tp = on_device(dev, parts, abi.F32)
    hand = dev.carrier_merge(tp.view(n_parts, rows, D + 2)).cpu().numpy()
    # the carrier over partial accumulators: leaves (m, l, o[e]) of part s at row r; lift = the item itself
    W = D + 2
    ops = [em.Operand(0, abi.F32, [W, 0], rows * W, offset=0), em.Operand(0, abi.F32, [W, 0], rows * W, offset=1),
           em.Operand(0, abi.F32, [W, 1], rows * W, offset=2)]
    m = em.maximum(em.A(0), em.B(0))
    car = em.Carrier([em.load(0), em.load(1), em.load(2)], [em.item(0), em.item(1), em.item(2)],
                     [m, em.A(1) * em._shift(em.A(0), m) + em.B(1) * em._shift(em.B(0), m),
                      em.A(2) * em._shift(em.A(0), m) + em.B(2) * em._shift(em.B(0), m)],
                     [float("-inf"), 0.0, 0.0], em.F(2) / em.F(1))
    kern = em.GenericKernel(dev, em.Description((rows, D), ops, carrier=car, stream=n_parts))
    out = torch.empty(rows * D, device=dev.torch_device)
    kern([tp], out)
    dev.sync()
    gen = out.cpu().numpy().reshape(rows, D)
    assert nerr(gen, hand) <= 2e-6
    assert nerr(hand, orc.carrier_merge_mlo(parts)) <= F32_TOL
    kern.close()


# ───────────── reduces over several axes at once, scans and top-k (the reference's tests/movement.rs compositions) ─────────────
def _windows(x, kh, kw, stride, dilation=1):
    """All (kh, kw) windows of the last two axes: [..., OH, OW, kh, kw], dense reference evaluation."""
    span_h, span_w = dilation * (kh - 1) + 1, dilation * (kw - 1) + 1
    v = np.lib.stride_tricks.sliding_window_view(x, (span_h, span_w), axis=(-2, -1))
    return v[..., ::stride, ::stride, ::dilation, ::dilation]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,lanes,stride,dilation", [(abi.F32, 1, 1, 1), (abi.BF16, 32, 1, 1), (abi.F32, 32, 2, 1), (abi.BF16, 1, 1, 2)])
def test_generic_convolution_is_an_implicit_gemm_over_a_window(dev, dtype, lanes, stride, dilation):
    N, C, H, W, CO, KH, KW = 2, 5, 11, 9, 6, 3, 2
    g = orc.Xorshift(0xC0471)
    rd = (lambda a: orc.round_to(orc.DT_BF16, a)) if dtype == abi.BF16 else (lambda a: orc.round_to(orc.DT_F32, a))
    x, w = rd(g.normal(N, C, H, W)), rd(0.2 * g.normal(CO, C, KH, KW))
    grid, win, ops, car = em.conv2d(N, C, H, W, CO, KH, KW, stride=stride, dilation=dilation, dtype=dtype)
    want = np.einsum("nchwyx,ocyx->nohw", _windows(x, KH, KW, stride, dilation), w)
    assert want.shape == grid
    got = run_kernel(dev, em.Description(grid, ops, carrier=car, stream=win, lanes=lanes),
                     [on_device(dev, x, dtype), on_device(dev, w, dtype)], grid)
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("lanes,stride,padding", [(32, 1, 1), (1, 2, 2)])
def test_generic_padded_convolution(dev, lanes, stride, padding):
    """Taps outside the input read 0 through the padded gather (a padded Reindex reads 0.0 in the reference's interpreter),
    and raise no status: the run must leave the context clean."""
    N, C, H, W, CO, KH, KW = 2, 3, 7, 6, 4, 3, 3
    g = orc.Xorshift(0x9AD)
    x, w = orc.round_to(orc.DT_F32, g.normal(N, C, H, W)), orc.round_to(orc.DT_F32, 0.3 * g.normal(CO, C, KH, KW))
    grid, win, ops, car = em.conv2d(N, C, H, W, CO, KH, KW, stride=stride, padding=padding)
    xp = np.pad(x, ((0, 0), (0, 0), (padding, padding), (padding, padding)))
    want = np.einsum("nchwyx,ocyx->nohw", _windows(xp, KH, KW, stride), w)
    assert want.shape == grid
    d = em.Description(grid, ops, carrier=car, stream=win, lanes=lanes)
    assert "atomicCAS(status, 0, 51)" not in em.source(d)
    got = run_kernel(dev, d, [on_device(dev, x, abi.F32), on_device(dev, w, abi.F32)], grid)      # run_kernel syncs: no status raised
    assert nerr(got, want) <= F32_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("kind,k,stride", [("max", 2, None), ("mean", 3, 2), ("max", 3, 1)])
def test_generic_pooling(dev, kind, k, stride):
    N, C, H, W = 2, 3, 10, 12
    x = orc.round_to(orc.DT_F32, orc.Xorshift(0x9001).normal(N, C, H, W))
    grid, win, ops, car = em.pool2d(N, C, H, W, k, k, stride=stride, kind=kind)
    v = _windows(x, k, k, stride if stride else k)
    want = v.max(axis=(-2, -1)) if kind == "max" else v.mean(axis=(-2, -1))
    got = run_kernel(dev, em.Description(grid, ops, carrier=car, stream=win), [on_device(dev, x, abi.F32)], grid)
    assert nerr(got, want) <= (0.0 if kind == "max" else F32_TOL)


@pytest.mark.gpu
@pytest.mark.parametrize("lanes", [1, 32])
def test_generic_inclusive_scan_as_a_masked_fold(dev, lanes):
    """cumsum[i] = sum over j of where(j <= i, x[j], 0): the scan the reference writes as a triangular mask under a reduce."""
    rows, n = 4, 70
    x = orc.round_to(orc.DT_F32, orc.Xorshift(0x5CA4).normal(rows, n))
    ops = [em.Operand(0, abi.F32, [n, 0], 1)]
    car = em.carrier_sum(em.where(em.coord(2) < em.coord(1) + 1.0, em.load(0), 0.0))
    got = run_kernel(dev, em.Description((rows, n), ops, carrier=car, stream=n, lanes=lanes), [on_device(dev, x, abi.F32)], (rows, n))
    assert nerr(got, np.cumsum(x, axis=1)) <= F32_TOL


@pytest.mark.gpu
def test_generic_top_k_as_repeated_first_argmax(dev):
    """top-k as the composition it is in the reference: k rounds of the first-argmax fold, each masking the indices already
    taken. Bit-exact indices, ties to the lowest index."""
    import torch
    rows, n, k = 5, 97, 4
    x = orc.round_to(orc.DT_F32, orc.Xorshift(0x70B4).normal(rows, n))
    x[1, 10] = x[1, 60] = x[1].max() + 1.0                      # a tie for the maximum: the lower index goes first
    xd = on_device(dev, x, abi.F32)
    taken = []
    for r in range(k):
        ops = [em.Operand(0, abi.F32, [n], 1)] + [em.Operand(1 + i, abi.U32, [1], 0) for i in range(r)]
        same = 0.0
        for i in range(r):
            same = same + (em.coord(1) < em.load(1 + i) + 1.0) * (em.load(1 + i) < em.coord(1) + 1.0)
        leaf = em.where(same, float("-inf"), em.load(0)) if r else em.load(0)
        d = em.Description((rows,), ops, carrier=em.carrier_first_argmax(leaf, em.coord(1)), stream=n, lanes=32, out_dtype=abi.U32)
        out = torch.empty(rows, dtype=torch.int32, device=dev.torch_device)
        kern = em.GenericKernel(dev, d)
        kern([xd] + taken, out)
        dev.sync()
        kern.close()
        taken.append(out)
    got = np.stack([t.cpu().numpy() for t in taken], axis=1)
    want = np.argsort(-x, axis=1, kind="stable")[:, :k]
    assert np.array_equal(got, want)
    assert got[1, 0] == 10 and got[1, 1] == 60


def test_isomorphic_stages_compile_once_and_kernels_carry_descriptive_names():
    """Two stages that differ only in the buffers they bind render the same text: one compilation (the reference dedups
    per canonical body, src/emit_metal.rs:1281-1330). Needs NVRTC, not a device."""
    grid, k, ops, car = matmul_case(8, 16, 4, abi.BF16)
    d1 = em.Description(grid, ops, carrier=car, stream=k, lanes=32)
    # the same stage over other buffers of the same layout
    ops2 = [em.Operand(3, abi.BF16, [k, 0], 1), em.Operand(7, abi.BF16, [0, 1], 4)]
    d2 = em.Description(grid, ops2, carrier=car, stream=k, lanes=32)
    assert em.source(d1) != em.source(d2)          # buffer slots are part of the text: positional binding is per kernel
    c0, r0 = em.cache_stats()
    assert em.compiles(d1) > 0
    c1, r1 = em.cache_stats()
    assert em.compiles(d1) > 0 and em.compiles(em.Description(grid, ops, carrier=car, stream=k, lanes=32)) > 0
    c2, r2 = em.cache_stats()
    assert c2 == c1 and r2 == r1 + 2 and c1 - c0 <= 1


@pytest.mark.gpu
def test_generated_kernel_names(dev):
    grid, k, ops, car = matmul_case(8, 16, 4, abi.BF16)
    a = em.GenericKernel(dev, em.Description(grid, ops, carrier=car, stream=k, lanes=32))
    b = em.GenericKernel(dev, em.Description(grid, ops, carrier=car, stream=k, out_dtype=abi.BF16))
    g, win, cops, ccar = em.conv2d(2, 3, 9, 8, 4, 3, 3)
    c = em.GenericKernel(dev, em.Description(g, cops, carrier=ccar, stream=win, lanes=32, warps=4))
    assert a.name == "fold1_g8x4_s16_lanes_f32" and b.name == "fold1_g8x4_s16_thread_bf16"
    assert c.name == "fold1_g2x4x7x6_s3x3x3_lanes_w4_f32"
    for kk in (a, b, c):
        kk.close()
