"""Pins the CPU oracle to the reference's own known answers and seeded laws.

Every case names the reference test it restates (paths within the reference
project). Literal expected vectors come from those tests; the seeded cases use
the reference's xorshift64* generator with the reference's seeds, so the tensors
are the reference's tensors bit for bit.
"""
import math

import numpy as np
import pytest

from oracle import oracle as orc

F64_EPS = np.finfo(np.float64).eps


def rel_tolerance_f64(terms):  # src/verify.rs:35-47
    return 64.0 * F64_EPS * max(terms, 1)


def assert_close(a, e, terms=64):
    a = np.asarray(a, dtype=np.float64).ravel()
    e = np.asarray(e, dtype=np.float64).ravel()
    assert a.shape == e.shape
    tol = rel_tolerance_f64(terms) * (1.0 + np.maximum(np.abs(a), np.abs(e)))
    assert np.all(np.abs(a - e) <= tol), (a, e)


def test_prng_matches_reference_formula():
    # tests/oracle.rs:49-59, recomputed in pure Python integers
    x = 0xA11CE
    want = []
    for _ in range(5):
        x ^= x >> 12
        x = (x ^ (x << 25)) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 27
        want.append(((((x * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF) >> 11) / float(1 << 53)) * 2.0 - 1.0)
    got = orc.Xorshift(0xA11CE).uniform(5)
    assert list(got) == want


def test_direct_attention_known_answer():
    # tests/compile.rs:236-261, examples/direct_attention.rs, tests/nn.rs:15-50
    q = k = np.array([[1.0, 0.0], [0.0, 1.0]])
    v = np.array([[2.0, 3.0], [5.0, 7.0]])
    out = orc.sdpa(q, k, v).ravel()
    high = math.exp(1.0 / math.sqrt(2.0))
    sel = high / (high + 1.0)
    oth = 1.0 - sel
    assert_close(out, [sel * 2 + oth * 5, sel * 3 + oth * 7, oth * 2 + sel * 5, oth * 3 + sel * 7])
    literal = np.array([2.990715, 4.3209534, 4.009285, 5.6790466])
    f32_tol = 64.0 * np.finfo(np.float32).eps * 2 * (1.0 + np.abs(literal))
    assert np.all(np.abs(out - literal) < f32_tol)


def test_additive_mask_and_explicit_scale():
    # tests/nn.rs:52-82
    q = np.array([[1.0], [1.0]])
    k = np.array([[1.0], [2.0], [3.0]])
    v = np.array([[10.0], [20.0], [30.0]])
    mask = np.array([[0.0, -1e30, -1e30], [0.0, 0.0, -1e30]])
    out = orc.sdpa(q, k, v, mask=mask, scale=2.0).ravel()
    w = math.exp(2.0) / (1.0 + math.exp(2.0))
    assert_close(out, [10.0, 10.0 * (1.0 - w) + 20.0 * w])


def test_causal_rectangular_upper_left():
    # tests/nn.rs:84-110
    q = np.zeros((2, 2))
    k = np.zeros((3, 2))
    v = np.array([[10.0], [20.0], [90.0]])
    assert_close(orc.sdpa(q, k, v, is_causal=True, scale=0.5).ravel(), [10.0, 15.0])


def test_gqa_repeats_heads_like_torch():
    # tests/nn.rs:112-137
    q = np.ones((4, 1, 1))
    k = np.array([1.0, 2.0]).reshape(2, 1, 1)
    v = np.array([10.0, 20.0]).reshape(2, 1, 1)
    out = orc.sdpa(q, k, v, enable_gqa=True)
    assert out.shape == (4, 1, 1)
    assert_close(out.ravel(), [10.0, 10.0, 20.0, 20.0])


def test_argmax_first_maximum_wins():
    # tests/compile.rs:139-171
    x = np.array([2.0, 5.0, 5.0, 1.0, 5.0, 2.0, 0.0, 5.0])
    assert orc.argmax(x) == 1.0
    for blocks in (1, 2, 3, 8):
        assert orc.argmax(x, blocks=blocks) == 1.0
    # tests/oracle.rs:259-286
    rng = orc.Xorshift(0xA6A5)
    logits = rng.uniform(5, 20)
    logits[:, 3] = 9.0
    logits[:, 11] = 9.0
    assert list(orc.argmax(logits)) == [3.0] * 5
    assert list(orc.argmax(logits, blocks=7)) == [3.0] * 5


def test_multihead_carrier_equals_eval():
    # tests/oracle.rs:90-122: seed 0xA11CE, (b,h,sq,k,d,e) = (2,3,5,7,4,6), scale 1
    rng = orc.Xorshift(0xA11CE)
    q = rng.uniform(2, 3, 5, 4)
    k = rng.uniform(2, 3, 7, 4)
    v = rng.uniform(2, 3, 7, 6)
    ref = orc.sdpa(q, k, v, scale=1.0)
    got = orc.sdpa_carrier_split(q, k, v, 1, scale=1.0)
    assert_close(got, ref, terms=7)


def test_split_law_any_block_count():
    # tests/group.rs:48-83: seed 0x6408, (s,k,d,e) = (4,9,5,4), blocks 1,2,3,7,9
    rng = orc.Xorshift(0x6408)
    q, k, v = rng.uniform(4, 5), rng.uniform(9, 5), rng.uniform(9, 4)
    ref = orc.sdpa(q, k, v, scale=1.0)
    for blocks in (1, 2, 3, 7, 9):
        assert_close(orc.sdpa_carrier_split(q, k, v, blocks, scale=1.0), ref, terms=64)
    with pytest.raises(ValueError):  # src/interp.rs:570-574: blocks <= extent
        orc.sdpa_carrier_split(q, k, v, 10, scale=1.0)


def test_split_causal_identity_partials():
    # tests/group.rs:85-116: seed 0x640C, 6x6 causal, blocks 2,3,6
    rng = orc.Xorshift(0x640C)
    q, k, v = rng.uniform(6, 4), rng.uniform(6, 4), rng.uniform(6, 3)
    ref = orc.sdpa(q, k, v, is_causal=True, scale=1.0)
    assert np.all(np.isfinite(ref))
    for blocks in (2, 3, 6):
        got = orc.sdpa_carrier_split(q, k, v, blocks, is_causal=True, scale=1.0)
        assert np.all(np.isfinite(got))
        assert_close(got, ref, terms=64)


def test_carrier_merge_matches_split():
    # src/interp.rs:632-639: stage 2 merges the per-chunk partials left to right
    rng = orc.Xorshift(0x6408)
    q, k, v = rng.uniform(4, 5), rng.uniform(9, 5), rng.uniform(9, 4)
    ref = orc.sdpa(q, k, v, scale=1.0)
    parts = []
    for lo, hi in ((0, 3), (3, 6), (6, 9)):
        _, car = orc.sdpa_carrier_split(q, k[lo:hi], v[lo:hi], 1, scale=1.0, return_carriers=True)
        parts.append(car.reshape(4, 2 + 4))
    assert_close(orc.carrier_merge_mlo(np.stack(parts)), ref, terms=64)


def test_rmsnorm_fused_projection():
    # tests/oracle.rs:128-151: seed 0x524D53, (s,dm,f) = (4,16,5), W stored [f, dm]
    rng = orc.Xorshift(0x524D53)
    x, g, w = rng.uniform(4, 16), rng.uniform(16), rng.uniform(5, 16)
    ref = orc.rmsnorm_gemm(x, g, w, eps=1e-5, w_is_nk=True)
    hand = np.empty((4, 5))
    for i in range(4):
        den = math.sqrt(sum(t * t for t in x[i]) * (1.0 / 16.0) + 1e-5)
        for j in range(5):
            acc = 0.0
            for kk in range(16):
                acc = acc + ((x[i, kk] * g[kk]) / den) * w[j, kk]
            hand[i, j] = acc
    assert np.array_equal(ref, hand)
    for blocks in (1, 2, 5, 16):
        assert_close(orc.rmsnorm_gemm(x, g, w, eps=1e-5, w_is_nk=True, blocks=blocks), ref, terms=16)
    # tests/laws.rs:620-646: project = dot / sqrt(ss / n + eps)
    rng = orc.Xorshift(1234)
    assert_close(orc.rmsnorm_gemm(x[:1], g, w[:1], w_is_nk=True, blocks=16), ref[:1, :1], terms=16)


def test_w4_packing_and_grouped_matvec():
    # tests/metal.rs:1178-1269: seed 0x144A16, 16 outputs, 4 groups of 128
    n_out, n_g, n_r = 16, 4, 128
    n_in = n_g * n_r
    rng = orc.Xorshift(0x144A16)
    q = np.clip(np.floor(rng.uniform(n_out * n_in) * 8.0), -8.0, 7.0).astype(np.int8)
    packed = orc.w4_pack(q)
    manual = np.zeros(n_out * n_in // 2, dtype=np.uint8)
    for i, val in enumerate(q):
        manual[i // 2] |= np.uint8((int(val) + 8) << ((i & 1) * 4))
    assert np.array_equal(packed, manual)
    assert np.array_equal(orc.w4_unpack(packed, q.size), q.astype(np.float64))
    scales = (1.0 + np.round(np.abs(rng.uniform(n_out * n_g)) * 15.0)) / 64.0
    x = rng.uniform(n_in)
    y = orc.w4_gemv(packed, scales.reshape(n_out, n_g), x, n_out, group=n_r)
    hand = np.zeros(n_out)
    qf = q.astype(np.float64).reshape(n_out, n_in)
    for o in range(n_out):
        acc = 0.0
        for c in range(n_in):
            acc = acc + (qf[o, c] * x[c]) * scales[o * n_g + c // n_r]
        hand[o] = acc
    assert np.array_equal(y, hand)
    assert_close(orc.w4_gemv(packed, scales.reshape(n_out, n_g), x, n_out, group=n_r, blocks=7), hand, terms=n_in)


def test_quantized_matmul_dequant():
    # tests/oracle.rs:207-233: seed 0x9114A7, per-channel scale (one group spanning K)
    rng = orc.Xorshift(0x9114A7)
    qw = np.round(rng.uniform(6, 12) * 8.0)
    x = rng.uniform(4, 12)
    scale = 0.05 * (rng.uniform(6) + 1.5)
    qi = np.clip(qw, -8, 7).astype(np.int8)
    y = orc.w4_gemv(orc.w4_pack(qi.ravel()), scale.reshape(6, 1), x, 6, group=12)
    want = x @ (qi.astype(np.float64) * scale[:, None]).T
    assert_close(y, want, terms=12)


def test_sliding_window_attention_matches_hand_reference():
    # tests/movement.rs:294-384: seed 0x51D3, ns=10, w=4, d=5, e=6, no scale
    ns, w = 10, 4
    rng = orc.Xorshift(0x51D3)
    q, k, v = rng.uniform(ns, 5), rng.uniform(ns, 5), rng.uniform(ns, 6)
    got = orc.sdpa_window(q, k, v, w, scale=1.0)
    hand = np.zeros((ns, 6))
    for si in range(ns):
        pos = list(range(max(si - (w - 1), 0), si + 1))
        dots = [sum(q[si, d] * k[p, d] for d in range(5)) for p in pos]
        m = max(dots)
        ex = [math.exp(t - m) for t in dots]
        z = sum(ex)
        for e in range(6):
            hand[si, e] = sum((wi / z) * v[p, e] for p, wi in zip(pos, ex))
    assert_close(got, hand, terms=64)


def test_bf16_rounding_value_list():
    # tests/metal.rs:2177-2250 value list; src/scalar.rs:128-135
    torch = pytest.importorskip("torch")
    vals = np.array([0.0, -0.0, 1.0, 1.0 + 1.0 / 512.0, 1.0 + 3.0 / 512.0, -1.0 - 1.0 / 512.0, 65504.0, 3.4e38, -3.4e38,
                     np.inf, -np.inf, 1e-40, math.pi, -math.e, 0.1, 123456789.0])
    got = orc.round_to(orc.DT_BF16, vals)
    want = torch.tensor(vals, dtype=torch.float64).to(torch.float32).to(torch.bfloat16).to(torch.float64).numpy()
    assert np.array_equal(got.view(np.uint64), want.view(np.uint64))
    assert got[3] == 1.0 and got[4] == 1.0 + 1.0 / 128.0 and np.isinf(got[7]) and got[7] > 0
    assert np.signbit(got[1])
    bits = orc.to_bf16_bits(vals)
    assert np.array_equal(orc.from_bf16_bits(bits).view(np.uint64), got.view(np.uint64))
    nan_bits = orc.to_bf16_bits(np.array([np.nan]))
    assert (nan_bits[0] & 0x7FC0) == 0x7FC0  # quiet NaN kept
    h = orc.round_to(orc.DT_F16, vals)
    want_h = torch.tensor(vals, dtype=torch.float64).to(torch.float32).to(torch.float16).to(torch.float64).numpy()
    assert np.array_equal(h.view(np.uint64), want_h.view(np.uint64))


def test_rope_frequencies():
    # examples/llama3_2.rs:689-700
    f = orc.llama3_inv_freq(32)
    assert abs(f[1] - math.exp(-math.log(500000.0) / 32.0)) < 1e-12
    plain = orc.rope_inv_freq(500000.0, 32)
    assert f[0] == plain[0] == 1.0
    assert abs(f[31] - plain[31] / 32.0) < 1e-18  # lowest frequency is scaled by the factor


def test_rope_is_rotate_half():
    # src/nn.rs:176-194: pair-major split, sign (-1, +1)
    x = np.arange(1.0, 9.0).reshape(1, 8)
    f = orc.rope_inv_freq(10000.0, 4)
    out = orc.rope(x, np.array([3.0]), f)[0]
    for i in range(4):
        a = 3.0 * f[i]
        assert abs(out[i] - (x[0, i] * math.cos(a) - x[0, i + 4] * math.sin(a))) < 1e-12
        assert abs(out[i + 4] - (x[0, i + 4] * math.cos(a) + x[0, i] * math.sin(a))) < 1e-12


def _tiny_llama(batch=1, w4=False, seed=7, ctx=6):
    cfg = dict(vocab=16, layers=2, hidden=8, q_heads=4, kv_heads=2, head_dim=2, ffn=16, ctx=ctx, batch=batch,
               w4=int(w4), group=8, round_acts=0, llama3_rope=1)
    rng = orc.Xorshift(seed)

    def bf(*shape):
        return orc.to_bf16_bits(rng.uniform(*shape) * 0.5)

    L = cfg["layers"]
    w = dict(embed=bf(16, 8), final_norm=orc.to_bf16_bits(1.0 + 0.1 * rng.uniform(8)),
             attn_norm=[orc.to_bf16_bits(1.0 + 0.1 * rng.uniform(8)) for _ in range(L)],
             mlp_norm=[orc.to_bf16_bits(1.0 + 0.1 * rng.uniform(8)) for _ in range(L)])
    shapes = dict(wq=(8, 8), wk=(4, 8), wv=(4, 8), wo=(8, 8), wgate=(16, 8), wup=(16, 8), wdown=(8, 16))
    for name, shp in shapes.items():
        w[name] = [bf(*shp) for _ in range(L)]
    return cfg, w


def test_llama_decode_root_shapes_and_prefill_equivalence():
    # examples/llama3_2.rs:702-736 pins the cache layouts; tests/decode.rs:121-204 pins that
    # T incremental steps equal one causal prefill. Here: the stateful oracle's step t must equal
    # an independent numpy evaluation of causal attention over the first t+1 tokens.
    cfg, w = _tiny_llama()
    m = orc.Llama(cfg, w)
    assert m.kcache.shape == (2, 1, 2, 6, 2) and m.vcache.shape == (2, 1, 2, 2, 6)
    toks = [3, 7, 1, 12, 5]
    got = [int(m.step([t], p)[0]) for p, t in enumerate(toks)]
    logits_last = m.logits()[0]

    W = {k: ([orc.from_bf16_bits(a) for a in v] if isinstance(v, list) else orc.from_bf16_bits(v)) for k, v in w.items()}
    inv = orc.llama3_inv_freq(1)
    T = len(toks)
    x = W["embed"][toks]  # [T, 8]
    pos = np.arange(T, dtype=np.float64)
    for l in range(2):
        xn = orc.rms_norm(x, W["attn_norm"][l])
        q = (xn @ W["wq"][l].T).reshape(T, 4, 2).transpose(1, 0, 2)
        k = (xn @ W["wk"][l].T).reshape(T, 2, 2).transpose(1, 0, 2)
        v = (xn @ W["wv"][l].T).reshape(T, 2, 2).transpose(1, 0, 2)
        q = orc.rope(q, pos[None, :], inv)
        k = orc.round_to(orc.DT_BF16, orc.rope(k, pos[None, :], inv))
        v = orc.round_to(orc.DT_BF16, v)
        att = orc.sdpa(q, k, v, is_causal=True, enable_gqa=True)  # [4, T, 2]
        att = att.transpose(1, 0, 2).reshape(T, 8)
        x = x + att @ W["wo"][l].T
        xn = orc.rms_norm(x, W["mlp_norm"][l])
        g, u = xn @ W["wgate"][l].T, xn @ W["wup"][l].T
        x = x + ((g * (1.0 / (1.0 + np.exp(-g)))) * u) @ W["wdown"][l].T
    logits = orc.rms_norm(x, W["final_norm"]) @ W["embed"].T
    assert np.allclose(logits[-1], logits_last, rtol=1e-9, atol=1e-12)
    assert got == [int(t) for t in orc.argmax(logits)]


def test_llama_batch_rows_are_independent():
    cfg, w = _tiny_llama(batch=3)
    m3 = orc.Llama(cfg, w)
    cfg1, _ = _tiny_llama(batch=1)
    singles = [orc.Llama(cfg1, w) for _ in range(3)]
    toks = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]])
    for p in range(3):
        out = m3.step(toks[p], p)
        for b in range(3):
            assert out[b] == singles[b].step([toks[p, b]], p)[0]
