"""GPU parity: every kernel family, called through the C ABI, against the CPU oracle on the same
seeded inputs. Inputs are rounded to their declared storage dtype before either side sees them.

Tolerances (stated once):
  * f32 storage: max |g - e| / (1 + |e|) <= 1e-5 against the f64 oracle
  * bf16 storage: <= 2e-2 of the same normalised error
  * indices, int4 unpacking, bf16 rounding, u32 saturation: bit-exact
"""
import math

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def dev():
    from sanic_b200 import CudaDevice
    return CudaDevice(0)


def nerr(got, exp):
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64)
    assert got.shape == exp.shape, (got.shape, exp.shape)
    assert np.all(np.isfinite(got)), "non-finite values in the GPU result"
    return float(np.max(np.abs(got - exp) / (1.0 + np.abs(exp))))


def normal(seed, *shape):
    return orc.Xorshift(seed).normal(*shape)


def f32t(a, dev):
    return torch.tensor(np.asarray(a, dtype=np.float32), device=dev.torch_device)


def bf16t(a, dev):
    """Round to bf16 with the oracle's rounding and upload; returns (tensor, widened f64 values)."""
    bits = orc.to_bf16_bits(a)
    t = torch.tensor(bits.view(np.int16), device=dev.torch_device).view(torch.bfloat16)
    return t, orc.from_bf16_bits(bits)


# ───────────────────────── f32 online-softmax fold (config 1) ─────────────────────────
def test_attn_f32_known_answers(dev):
    # reference tests/compile.rs:236-261 and tests/nn.rs:15-137
    q = f32t([[1, 0], [0, 1]], dev).view(1, 1, 2, 2)
    v = f32t([[2, 3], [5, 7]], dev).view(1, 1, 2, 2)
    out = dev.attn_fwd_f32(q, q.clone(), v).cpu().numpy().ravel()
    lit = np.array([2.990715, 4.3209534, 4.009285, 5.6790466])
    assert np.all(np.abs(out - lit) < 64 * np.finfo(np.float32).eps * 2 * (1 + np.abs(lit)))
    # additive mask + explicit scale
    q = f32t([[1.0], [1.0]], dev).view(1, 1, 2, 1)
    k = f32t([[1.0], [2.0], [3.0]], dev).view(1, 1, 3, 1)
    v = f32t([[10.0], [20.0], [30.0]], dev).view(1, 1, 3, 1)
    # head_dim 1 is not a multiple of 4: pad the contraction with zeros (adds exact zeros)
    qp = torch.zeros(1, 1, 2, 4, device=dev.torch_device); qp[..., :1] = q
    kp = torch.zeros(1, 1, 3, 4, device=dev.torch_device); kp[..., :1] = k
    mask = f32t([[0.0, -1e30, -1e30], [0.0, 0.0, -1e30]], dev)
    out = dev.attn_fwd_f32(qp, kp, v, scale=2.0, mask=mask).cpu().numpy().ravel()
    w = math.exp(2.0) / (1.0 + math.exp(2.0))
    assert nerr(out, [10.0, 10.0 * (1 - w) + 20.0 * w]) < F32_TOL
    # causal, rectangular: upper-left aligned
    q0 = torch.zeros(1, 1, 2, 4, device=dev.torch_device)
    k0 = torch.zeros(1, 1, 3, 4, device=dev.torch_device)
    v0 = f32t([[10.0], [20.0], [90.0]], dev).view(1, 1, 3, 1)
    assert nerr(dev.attn_fwd_f32(q0, k0, v0, causal=True, scale=0.5).cpu().numpy().ravel(), [10.0, 15.0]) < F32_TOL
    # GQA 4 query heads over 2 kv heads
    q1 = torch.zeros(1, 4, 1, 4, device=dev.torch_device); q1[..., 0] = 1.0
    k1 = torch.zeros(1, 2, 1, 4, device=dev.torch_device); k1[0, 0, 0, 0] = 1.0; k1[0, 1, 0, 0] = 2.0
    v1 = f32t([10.0, 20.0], dev).view(1, 2, 1, 1)
    assert nerr(dev.attn_fwd_f32(q1, k1, v1).cpu().numpy().ravel(), [10.0, 10.0, 20.0, 20.0]) < F32_TOL


def test_attn_f32_config1(dev):
    # Q [256x64], K, V [1024x64] i.i.d. N(0,1), scale 1/8, no mask
    q = orc.round_to(orc.DT_F32, normal(0xC0F1601, 256, 64))
    k = orc.round_to(orc.DT_F32, normal(0xC0F1602, 1024, 64))
    v = orc.round_to(orc.DT_F32, normal(0xC0F1603, 1024, 64))
    exp = orc.sdpa(q, k, v, scale=0.125)
    got = dev.attn_fwd_f32(f32t(q, dev).view(1, 1, 256, 64), f32t(k, dev).view(1, 1, 1024, 64),
                           f32t(v, dev).view(1, 1, 1024, 64), scale=0.125).cpu().numpy()[0, 0]
    assert nerr(got, exp) <= F32_TOL
    rel = np.max(np.abs(got - exp) / np.maximum(np.abs(exp), 1e-2))
    assert rel <= 1e-4  # plain relative error away from zero crossings


@pytest.mark.parametrize("shape", [(2, 3, 3, 5, 7, 4, 6), (1, 4, 2, 33, 70, 8, 32), (1, 2, 2, 7, 130, 64, 128)])
@pytest.mark.parametrize("mode", ["plain", "causal", "window"])
def test_attn_f32_shapes_and_masks(dev, shape, mode):
    B, Hq, Hkv, L, S, E, Ev = shape
    if mode != "plain":
        S = L  # causal / window cases are square
    q = orc.round_to(orc.DT_F32, normal(1 + L, B, Hq, L, E))
    k = orc.round_to(orc.DT_F32, normal(2 + L, B, Hkv, S, E))
    v = orc.round_to(orc.DT_F32, normal(3 + L, B, Hkv, S, Ev))
    scale = 1.0 / math.sqrt(E)
    if mode == "plain":
        exp = orc.sdpa(q, k, v, scale=scale, enable_gqa=True)
        got = dev.attn_fwd_f32(f32t(q, dev), f32t(k, dev), f32t(v, dev), scale=scale)
    elif mode == "causal":
        exp = orc.sdpa(q, k, v, is_causal=True, scale=scale, enable_gqa=True)
        got = dev.attn_fwd_f32(f32t(q, dev), f32t(k, dev), f32t(v, dev), causal=True, scale=scale)
    else:
        w = 4 if L > 4 else 2
        exp = orc.sdpa_window(q, k, v, w, scale=scale)
        got = dev.attn_fwd_f32(f32t(q, dev), f32t(k, dev), f32t(v, dev), window=w, scale=scale)
    assert nerr(got.cpu().numpy(), exp) <= F32_TOL


@pytest.mark.parametrize("mode", ["plain", "causal", "window", "mask"])
@pytest.mark.parametrize("L,S", [(37, 1000), (600, 600), (5, 2100)])
def test_attn_f32_keys_split_over_a_cluster(dev, mode, L, S):
    # few (row block, head) CTAs and several 256-key chunks: the key axis is split over a cluster of up to 8 CTAs and the
    # partial (m, l, o) merge in rank order through distributed shared memory; ragged last chunk, rows whose visible
    # range ends before a CTA's share (its partial is the identity), a window that starts inside a later chunk
    if mode in ("causal", "window"):
        S = L if L > 256 else 600
        L = S
    E, Ev = 24, 40
    q = orc.round_to(orc.DT_F32, normal(11 + L, 1, 2, L, E))
    k = orc.round_to(orc.DT_F32, normal(12 + S, 1, 1, S, E))
    v = orc.round_to(orc.DT_F32, normal(13 + S, 1, 1, S, Ev))
    scale = 0.3
    tq, tk, tv = f32t(q, dev), f32t(k, dev), f32t(v, dev)
    if mode == "plain":
        exp = orc.sdpa(q, k, v, scale=scale, enable_gqa=True)
        got = dev.attn_fwd_f32(tq, tk, tv, scale=scale)
    elif mode == "causal":
        exp = orc.sdpa(q, k, v, is_causal=True, scale=scale, enable_gqa=True)
        got = dev.attn_fwd_f32(tq, tk, tv, causal=True, scale=scale)
    elif mode == "window":
        exp = orc.sdpa_window(q, k, v, 300, scale=scale)
        got = dev.attn_fwd_f32(tq, tk, tv, window=300, scale=scale)
    else:
        m = orc.round_to(orc.DT_F32, normal(14 + S, L, S))
        m[:, S // 2:S // 2 + 300] = -np.inf            # a whole chunk's worth of keys masked out for every row
        exp = orc.sdpa(q, k, v, mask=m, scale=scale, enable_gqa=True)
        got = dev.attn_fwd_f32(tq, tk, tv, mask=f32t(m, dev), scale=scale)
    assert nerr(got.cpu().numpy(), exp) <= F32_TOL


def test_attn_f32_rejects_bad_arguments(dev):
    from sanic_b200 import RunError
    q = torch.zeros(1, 3, 2, 4, device=dev.torch_device)
    k = torch.zeros(1, 2, 2, 4, device=dev.torch_device)
    with pytest.raises(RunError):  # 3 query heads over 2 kv heads
        dev.attn_fwd_f32(q, k, k.clone())
    with pytest.raises(RunError):  # wrong dtype
        dev.attn_fwd_f32(q.to(torch.bfloat16), k, k.clone())


# ───────────────────────── split-KV decode ─────────────────────────
def _decode_case(dev, B, Hq, Hkv, D, S, kv_len, vt, n_splits, window=0, seed=11):
    q, qv = bf16t(normal(seed, B, Hq, D), dev)
    k, kv = bf16t(normal(seed + 1, B, Hkv, S, D), dev)
    v, vv = bf16t(normal(seed + 2, B, Hkv, S, D), dev)
    vdev = v.transpose(2, 3).contiguous() if vt else v
    lo = max(0, kv_len - window) if window else 0
    exp, car = orc.sdpa_carrier_split(qv.reshape(B, Hq, 1, D), kv[:, :, lo:kv_len], vv[:, :, lo:kv_len], 1,
                                      enable_gqa=True, return_carriers=True)
    ref = orc.sdpa(qv.reshape(B, Hq, 1, D), kv[:, :, lo:kv_len], vv[:, :, lo:kv_len], enable_gqa=True)
    assert nerr(exp, ref) < 1e-12
    out, gcar = dev.attn_decode(q, k, vdev, kv_len, v_transposed=vt, n_splits=n_splits, window=window,
                                return_carrier=True, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert nerr(out.cpu().numpy(), exp.reshape(B, Hq, D)) <= BF16_TOL
    gc = gcar.cpu().numpy().astype(np.float64).reshape(B, Hq, D + 2)
    car = car.reshape(B, Hq, D + 2)
    # raw accumulators: same max; l and o agree up to the bf16 rounding of P
    assert np.max(np.abs(gc[..., 0] - car[..., 0])) <= 1e-4 * (1 + np.max(np.abs(car[..., 0])))
    assert nerr(gc[..., 1], car[..., 1]) <= BF16_TOL
    assert nerr(gc[..., 2:] / gc[..., 1:2], car[..., 2:] / car[..., 1:2]) <= BF16_TOL
    return out


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("vt", [False, True])
def test_decode_basic(dev, D, vt):
    _decode_case(dev, B=2, Hq=8, Hkv=2, D=D, S=512, kv_len=512, vt=vt, n_splits=3)


@pytest.mark.parametrize("kv_len,n_splits", [(1, 1), (1, 4), (63, 1), (64, 2), (65, 2), (200, 7), (1000, 16), (1030, 9)])
def test_decode_ragged_lengths_and_splits(dev, kv_len, n_splits):
    _decode_case(dev, B=1, Hq=32, Hkv=8, D=64, S=1056, kv_len=kv_len, vt=True, n_splits=n_splits)
    _decode_case(dev, B=1, Hq=4, Hkv=1, D=128, S=1056, kv_len=kv_len, vt=False, n_splits=n_splits)


@pytest.mark.parametrize("group", [1, 2, 8, 16])
def test_decode_gqa_groups(dev, group):
    _decode_case(dev, B=2, Hq=2 * group, Hkv=2, D=64, S=320, kv_len=300, vt=False, n_splits=2)


def test_decode_window(dev):
    _decode_case(dev, B=1, Hq=8, Hkv=2, D=64, S=1024, kv_len=700, vt=True, n_splits=3, window=256)
    _decode_case(dev, B=1, Hq=8, Hkv=2, D=128, S=1024, kv_len=700, vt=False, n_splits=2, window=100)


def test_decode_position_from_device_scalar(dev):
    B, Hq, Hkv, D, S = 1, 8, 2, 64, 256
    q, qv = bf16t(normal(5, B, Hq, D), dev)
    k, kv = bf16t(normal(6, B, Hkv, S, D), dev)
    v, vv = bf16t(normal(7, B, Hkv, S, D), dev)
    import ctypes as C
    pos = torch.tensor([99], dtype=torch.int32, device=dev.torch_device)
    out = dev.empty((B, Hq, D), torch.float32)
    from sanic_b200 import abi
    p, _keep = dev.decode_params(q, k, v, 1, n_splits=2, kv_len_dev=pos, out=out, out_dtype=abi.F32)
    dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
    exp = orc.sdpa(qv.reshape(B, Hq, 1, D), kv[:, :, :100], vv[:, :, :100], enable_gqa=True).reshape(B, Hq, D)
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL
    # a second launch reuses the scratch (ticket counters were reset by the first)
    pos.fill_(199)
    dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
    exp = orc.sdpa(qv.reshape(B, Hq, 1, D), kv[:, :, :200], vv[:, :, :200], enable_gqa=True).reshape(B, Hq, D)
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL


def test_decode_long_axis_round_trip(dev):
    # size-independent property at a long key axis: any chunking gives the same answer, and
    # folding two halves on their own then merging equals folding the whole.
    B, Hq, Hkv, D, S = 1, 8, 2, 128, 65536
    g = torch.Generator(device=dev.torch_device); g.manual_seed(3)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    outs = [dev.attn_decode(q, k, v, S, n_splits=n, out_dtype=torch.float32).cpu().numpy() for n in (1, 5, 64, 148)]
    for o in outs[1:]:
        assert nerr(o, outs[0]) <= 2e-3
    _, ca = dev.attn_decode(q, k[:, :, :S // 2].contiguous(), v[:, :, :S // 2].contiguous(), S // 2, n_splits=8, return_carrier=True)
    _, cb = dev.attn_decode(q, k[:, :, S // 2:].contiguous(), v[:, :, S // 2:].contiguous(), S // 2, n_splits=8, return_carrier=True)
    merged = dev.carrier_merge(torch.stack([ca, cb])).cpu().numpy().reshape(B, Hq, D)
    assert nerr(merged, outs[0]) <= 2e-3
    # against the oracle on one (batch, kv head)
    qv = q.float().cpu().numpy().astype(np.float64)[:, :4].reshape(1, 4, 1, D)
    exp = orc.sdpa(qv, k[:, :1].float().cpu().numpy().astype(np.float64), v[:, :1].float().cpu().numpy().astype(np.float64),
                   enable_gqa=True).reshape(4, D)
    assert nerr(outs[0][0, :4], exp) <= BF16_TOL


def test_carrier_merge_matches_oracle(dev):
    rng = orc.Xorshift(0x6408)
    n_parts, rows, D = 5, 12, 64
    parts = np.empty((n_parts, rows, D + 2))
    parts[..., 0] = rng.uniform(n_parts, rows) * 20.0
    parts[..., 1] = np.abs(rng.uniform(n_parts, rows)) * 50.0 + 0.1
    parts[..., 2:] = rng.uniform(n_parts, rows, D) * 30.0
    # an identity partial (an all-masked shard): m = -inf, l = 0, o = 0 must be absorbed
    parts[1, :, 0] = -np.inf; parts[1, :, 1] = 0.0; parts[1, :, 2:] = 0.0
    parts = orc.round_to(orc.DT_F32, parts)
    exp = orc.carrier_merge_mlo(parts)
    got, car = dev.carrier_merge(f32t(parts, dev), return_carrier=True)
    assert nerr(got.cpu().numpy(), exp) <= F32_TOL
    c = car.cpu().numpy()
    assert nerr(c[:, 2:] / c[:, 1:2], exp) <= F32_TOL


# ───────────────────────── decode-batch contraction ─────────────────────────
@pytest.mark.parametrize("batch", [1, 3, 8, 16])
@pytest.mark.parametrize("K,rows", [(256, 48), (2048, 512), (8192, 64)])
def test_gemv_bf16(dev, batch, K, rows):
    x, xv = bf16t(normal(21, batch, K), dev)
    w, wv = bf16t(normal(22, rows, K) * 0.02, dev)
    exp = orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)
    got = dev.gemv(x, [w]).cpu().numpy()
    assert nerr(got, exp) <= 1e-4
    got16 = dev.gemv(x, [w], out_dtype=torch.bfloat16).float().cpu().numpy()
    assert nerr(got16, exp) <= BF16_TOL


def _w4(rows, K, seed, dev):
    rng = orc.Xorshift(seed)
    q = np.clip(np.floor(rng.uniform(rows * K) * 8.0), -8, 7).astype(np.int8)
    packed = orc.w4_pack(q)
    scales = 0.02 / 4.6 * (1.0 + 0.25 * np.abs(rng.uniform(rows, K // 64)))
    st, sv = bf16t(scales, dev)
    pt = torch.tensor(packed.reshape(rows, K // 2), device=dev.torch_device)
    return q, packed, pt, st, sv


@pytest.mark.parametrize("batch", [1, 5, 16])
@pytest.mark.parametrize("K,rows", [(128, 16), (2048, 256), (8192, 32)])
def test_gemv_w4(dev, batch, K, rows):
    q, packed, pt, st, sv = _w4(rows, K, 31 + batch, dev)
    x, xv = bf16t(normal(32, batch, K), dev)
    exp = orc.w4_gemv(packed, sv, xv, rows, group=64)
    got = dev.gemv(x, [pt], scales=[st]).cpu().numpy()
    assert nerr(got, exp) <= 2e-4


@pytest.mark.parametrize("batch,K,norm", [(1, 2048, False), (5, 2048, False), (8, 512, False), (3, 2048, True), (12, 2048, False),
                                          (16, 1024, False)])
def test_gemv_w4_many_row_tiles_warp_per_tile(dev, batch, K, norm):
    # An int4 matrix with at least 16 row tiles per SM takes the warp-per-tile kernel (8 or 16 batch columns). Sampled rows (first and
    # last tiles among them) against the oracle; the whole output against the tile-per-block kernel, which sums the same
    # products in another order; bf16 output is the f32 one rounded.
    import os
    rows = 16 * 2400
    gen = torch.Generator(device=dev.torch_device); gen.manual_seed(400 + batch)
    pt = torch.randint(0, 256, (rows, K // 2), device=dev.torch_device, generator=gen, dtype=torch.uint8)
    st = (0.004 * (1.0 + 0.25 * torch.rand(rows, K // 64, device=dev.torch_device, generator=gen))).to(torch.bfloat16)
    if norm:
        x = orc.round_to(orc.DT_F32, normal(401, batch, K) * 3.0)
        g, gv = bf16t(1.0 + 0.1 * normal(402, K), dev)
        xin, kw = f32t(x, dev), dict(norm_gamma=g)
        xv = orc.round_to(orc.DT_BF16, orc.rms_norm(x, gv))
    else:
        xin, xv = bf16t(normal(401, batch, K), dev)
        kw = {}
    got = dev.gemv(xin, [pt], scales=[st], **kw)
    got16 = dev.gemv(xin, [pt], scales=[st], out_dtype=torch.bfloat16, **kw)
    os.environ["SANIC_GEMV_W4_ROWS"] = "0"
    try:
        old = dev.gemv(xin, [pt], scales=[st], **kw)
    finally:
        del os.environ["SANIC_GEMV_W4_ROWS"]
    dev.sync()
    assert nerr(got.cpu().numpy(), old.cpu().numpy()) <= 1e-5
    assert torch.equal(got16, got.to(torch.bfloat16))
    pick = np.concatenate([np.arange(0, 32), np.arange(rows // 2 - 8, rows // 2 + 24), np.arange(rows - 32, rows)])
    packed = pt[torch.tensor(pick, device=dev.torch_device)].cpu().numpy().reshape(-1)
    sv = st[torch.tensor(pick, device=dev.torch_device)].float().cpu().numpy().astype(np.float64)
    exp = orc.w4_gemv(packed, sv, xv, len(pick), group=64)
    assert nerr(got.cpu().numpy()[:, pick], exp) <= (5e-4 if norm else 2e-4)


@pytest.mark.parametrize("batch,K,norm", [(1, 2048, False), (5, 1024, False), (8, 2048, False), (2, 2048, True)])
def test_gemv_w4_silu_mul_team_per_tile(dev, batch, K, norm):
    # silu(gate x) * (up x) with int4 matrices of at least one dual tile per SM takes, up to batch 8, the kernel with a team of
    # four warps per tile. The whole output against the tile-per-block (or ring-fed) form; sampled rows against the oracle.
    import os
    from sanic_b200 import abi
    rows = 16 * 256
    gen = torch.Generator(device=dev.torch_device); gen.manual_seed(500 + batch)
    pts = [torch.randint(0, 256, (rows, K // 2), device=dev.torch_device, generator=gen, dtype=torch.uint8) for _ in range(2)]
    sts = [(0.004 * (1.0 + 0.25 * torch.rand(rows, K // 64, device=dev.torch_device, generator=gen))).to(torch.bfloat16) for _ in range(2)]
    if norm:
        x = orc.round_to(orc.DT_F32, normal(501, batch, K) * 3.0)
        g, gv = bf16t(1.0 + 0.1 * normal(502, K), dev)
        xin, kw = f32t(x, dev), dict(norm_gamma=g)
        xv = orc.round_to(orc.DT_BF16, orc.rms_norm(x, gv))
    else:
        xin, xv = bf16t(normal(501, batch, K), dev)
        kw = {}
    got = dev.gemv(xin, pts, scales=sts, epilogue=abi.EPI_SILU_MUL, **kw)
    os.environ["SANIC_GEMV_W4_ROWS"] = "0"
    try:
        old = dev.gemv(xin, pts, scales=sts, epilogue=abi.EPI_SILU_MUL, **kw)
    finally:
        del os.environ["SANIC_GEMV_W4_ROWS"]
    dev.sync()
    assert got.shape == (batch, rows)
    assert nerr(got.cpu().numpy(), old.cpu().numpy()) <= 2e-5
    pick = np.concatenate([np.arange(0, 32), np.arange(rows // 2 - 8, rows // 2 + 24), np.arange(rows - 32, rows)])
    idx = torch.tensor(pick, device=dev.torch_device)
    ab = [orc.w4_gemv(pt[idx].cpu().numpy().reshape(-1), st[idx].float().cpu().numpy().astype(np.float64), xv, len(pick), group=64)
          for pt, st in zip(pts, sts)]
    exp = ab[0] / (1.0 + np.exp(-ab[0])) * ab[1]
    assert nerr(got.cpu().numpy()[:, pick], exp) <= (1e-3 if norm else 4e-4)


def test_w4_unpack_is_bit_exact(dev):
    q, packed, pt, _, _ = _w4(64, 512, 77, dev)
    got = dev.w4_unpack(pt.reshape(-1), q.size).cpu().numpy()
    assert np.array_equal(got, q.astype(np.float32))
    assert np.array_equal(got.astype(np.float64), orc.w4_unpack(packed, q.size))
    allb = torch.arange(256, dtype=torch.uint8, device=dev.torch_device)
    got = dev.w4_unpack(allb, 512).cpu().numpy().reshape(256, 2)
    assert np.array_equal(got[:, 0], (np.arange(256) & 15) - 8.0) and np.array_equal(got[:, 1], (np.arange(256) >> 4) - 8.0)


def test_gemv_segments_and_epilogues(dev):
    from sanic_b200 import abi
    batch, K = 4, 512
    x, xv = bf16t(normal(41, batch, K), dev)
    ws = [bf16t(normal(42 + i, r, K) * 0.05, dev) for i, r in enumerate((128, 32, 32))]
    outs = dev.gemv(x, [w for w, _ in ws])
    for (w, wv), o in zip(ws, outs):
        assert nerr(o.cpu().numpy(), orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)) <= 1e-4
    # silu(a) * b over a weight pair
    a = orc.gemv_bf16w(orc.to_bf16_bits(ws[1][1]), xv)
    b = orc.gemv_bf16w(orc.to_bf16_bits(ws[2][1]), xv)
    exp = (a * (1.0 / (1.0 + np.exp(-a)))) * b
    got = dev.gemv(x, [ws[1][0], ws[2][0]], epilogue=abi.EPI_SILU_MUL)
    assert nerr(got.cpu().numpy(), exp) <= 1e-4
    # residual add, in place on the f32 residual stream
    res = f32t(normal(49, batch, 128), dev)
    exp = res.cpu().numpy().astype(np.float64) + orc.gemv_bf16w(orc.to_bf16_bits(ws[0][1]), xv)
    import ctypes as C
    p = dev.gemv_params(x, [ws[0][0]], [res], None, abi.EPI_RESIDUAL_ADD, res, abi.F32)
    dev._check(dev.lib.sanic_gemv(dev.h, C.byref(p), dev.stream()), "gemv")
    assert nerr(res.cpu().numpy(), exp) <= 1e-4


@pytest.mark.parametrize("batch", [9, 12, 16])
def test_gemv_wide_batches_ring_fed_and_register_staged(dev, batch):
    """Batches 9-16 run the contraction fed by bulk copies through a shared-memory ring when the shape has a ring geometry
    (a stage of at least 256 inputs that divides K), else the register-staged kernel: both against the oracle, over one to
    four ring stages per tile, more tiles than SMs, three row segments, the silu-mul pair and the residual epilogue."""
    import ctypes as C
    from sanic_b200 import abi
    for K, rows in ((256, 48), (1024, 4752), (4096, 64), (1536, 32), (128, 16)):       # the last two have no ring geometry
        x, xv = bf16t(normal(121, batch, K), dev)
        w, wv = bf16t(normal(122, rows, K) * 0.02, dev)
        assert nerr(dev.gemv(x, [w]).cpu().numpy(), orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)) <= 1e-4, (K, rows)
    for K, rows in ((4096, 48), (8192, 32), (512, 64)):
        q, packed, pt, st, sv = _w4(rows, K, 131 + batch, dev)
        x, xv = bf16t(normal(132, batch, K), dev)
        assert nerr(dev.gemv(x, [pt], scales=[st]).cpu().numpy(), orc.w4_gemv(packed, sv, xv, rows, group=64)) <= 2e-4, (K, rows)
    K = 2048
    x, xv = bf16t(normal(141, batch, K), dev)
    ws = [bf16t(normal(142 + i, r, K) * 0.05, dev) for i, r in enumerate((128, 32, 32))]
    for (w, wv), o in zip(ws, dev.gemv(x, [w for w, _ in ws])):
        assert nerr(o.cpu().numpy(), orc.gemv_bf16w(orc.to_bf16_bits(wv), xv)) <= 1e-4
    a = orc.gemv_bf16w(orc.to_bf16_bits(ws[1][1]), xv)
    b = orc.gemv_bf16w(orc.to_bf16_bits(ws[2][1]), xv)
    got = dev.gemv(x, [ws[1][0], ws[2][0]], epilogue=abi.EPI_SILU_MUL)
    assert nerr(got.cpu().numpy(), (a * (1.0 / (1.0 + np.exp(-a)))) * b) <= 1e-4
    res = f32t(normal(149, batch, 128), dev)
    exp = res.cpu().numpy().astype(np.float64) + orc.gemv_bf16w(orc.to_bf16_bits(ws[0][1]), xv)
    p = dev.gemv_params(x, [ws[0][0]], [res], None, abi.EPI_RESIDUAL_ADD, res, abi.F32)
    dev._check(dev.lib.sanic_gemv(dev.h, C.byref(p), dev.stream()), "gemv")
    assert nerr(res.cpu().numpy(), exp) <= 1e-4


@pytest.mark.parametrize("batch,w4", [(1, False), (16, False), (3, True)])
def test_gemv_with_inlined_rmsnorm(dev, batch, w4):
    K, rows = 2048, 128
    x = orc.round_to(orc.DT_F32, normal(51, batch, K) * 3.0)
    g, gv = bf16t(1.0 + 0.1 * normal(52, K), dev)
    xn = orc.round_to(orc.DT_BF16, orc.rms_norm(x, gv))         # the declared stored(bf16) point
    if w4:
        q, packed, pt, st, sv = _w4(rows, K, 53, dev)
        exp = orc.w4_gemv(packed, sv, xn, rows, group=64)
        got = dev.gemv(f32t(x, dev), [pt], scales=[st], norm_gamma=g).cpu().numpy()
    else:
        w, wv = bf16t(normal(54, rows, K) * 0.02, dev)
        exp = orc.gemv_bf16w(orc.to_bf16_bits(wv), xn)
        got = dev.gemv(f32t(x, dev), [w], norm_gamma=g).cpu().numpy()
    assert nerr(got, exp) <= 5e-4      # a bf16 rounding boundary of xn may fall either way in f32


def test_gemv_rope_cache_epilogue_equals_separate_stages(dev):
    import ctypes as C
    from sanic_b200 import abi
    B, Hq, Hkv, D, ctx, K, pos = 3, 4, 2, 64, 40, 256, 17
    x, _ = bf16t(normal(61, B, K), dev)
    wq, _ = bf16t(normal(62, Hq * D, K) * 0.05, dev)
    wk, _ = bf16t(normal(63, Hkv * D, K) * 0.05, dev)
    wv, _ = bf16t(normal(64, Hkv * D, K) * 0.05, dev)
    table = dev.rope_table(list(orc.llama3_inv_freq(D // 2)), ctx)
    position = torch.tensor([pos], dtype=torch.int32, device=dev.torch_device)
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev.torch_device)
    # separate stages
    q, k, v = dev.gemv(x, [wq, wk, wv])
    qa, ka, va = z(B, Hq, D), z(B, Hkv, ctx, D), z(B, Hkv, D, ctx)
    r = abi.RopeCacheParams()
    r.q, r.k, r.v, r.q_out, r.k_cache, r.v_cache = (t.data_ptr() for t in (q, k, v, qa, ka, va))
    r.table, r.position = table.data_ptr(), position.data_ptr()
    r.batch, r.q_heads, r.kv_heads, r.head_dim, r.ctx = B, Hq, Hkv, D, ctx
    dev._check(dev.lib.sanic_rope_cache_write(dev.h, C.byref(r), dev.stream()), "rope_cache_write")
    # fused epilogue
    qb, kb, vb = z(B, Hq, D), z(B, Hkv, ctx, D), z(B, Hkv, D, ctx)
    p = dev.gemv_params(x, [wq, wk, wv], [], None, abi.EPI_ROPE_CACHE, None, abi.F32)
    p.rope_table, p.rope_position = table.data_ptr(), position.data_ptr()
    p.rope_q_out, p.rope_k_cache, p.rope_v_cache = qb.data_ptr(), kb.data_ptr(), vb.data_ptr()
    p.rope_q_heads, p.rope_kv_heads, p.rope_head_dim, p.rope_ctx = Hq, Hkv, D, ctx
    dev._check(dev.lib.sanic_gemv(dev.h, C.byref(p), dev.stream()), "gemv rope")
    torch.cuda.synchronize()
    assert torch.equal(qa, qb) and torch.equal(ka, kb) and torch.equal(va, vb)
    assert ka[:, :, pos].abs().sum() > 0 and ka[:, :, :pos].abs().sum() == 0    # only the written row is touched
    # and against the oracle's rope of the projected rows
    qo = orc.rope(q.cpu().numpy().astype(np.float64).reshape(B, Hq, D), float(pos), orc.llama3_inv_freq(D // 2))
    assert nerr(qb.float().cpu().numpy(), orc.round_to(orc.DT_BF16, qo)) <= 2.0 ** -7


def test_gemv_rejects_bad_arguments(dev):
    from sanic_b200 import RunError
    x = torch.zeros(17, 256, dtype=torch.bfloat16, device=dev.torch_device)
    w = torch.zeros(16, 256, dtype=torch.bfloat16, device=dev.torch_device)
    with pytest.raises(RunError):
        dev.gemv(x, [w])          # batch > 16
    with pytest.raises(RunError):
        dev.gemv(x[:2, :100].contiguous(), [w[:, :100].contiguous()])   # K not a multiple of 64


# ───────────────────────── extremum index, pointwise, typed stores ─────────────────────────
def test_argmax_first_maximum(dev):
    x = f32t([[2, 5, 5, 1, 5, 2, 0, 5]], dev)
    assert dev.argmax(x).cpu().tolist() == [1]      # reference tests/compile.rs:139-171
    rng = orc.Xorshift(0xA6A5)
    logits = rng.uniform(5, 20); logits[:, 3] = 9.0; logits[:, 11] = 9.0
    assert dev.argmax(f32t(logits, dev)).cpu().tolist() == [3] * 5
    big = orc.round_to(orc.DT_F32, normal(99, 16, 128256))
    big[3, 77777] = big[3, 100000] = 50.0
    exp = orc.argmax(big).astype(np.int64)
    assert exp[3] == 77777
    assert np.array_equal(dev.argmax(f32t(big, dev)).cpu().numpy().astype(np.int64), exp)


def test_round_to_bf16_bit_exact(dev):
    vals = np.array([0.0, -0.0, 1.0, 1.0 + 1.0 / 512.0, 1.0 + 3.0 / 512.0, -1.0 - 1.0 / 512.0, 65504.0, 3.4e38, -3.4e38,
                     np.inf, -np.inf, 1e-40, math.pi, -math.e, 0.1, 123456789.0], dtype=np.float64)  # tests/metal.rs:2177-2250
    rnd = orc.Xorshift(5).normal(100000) * np.exp(orc.Xorshift(6).uniform(100000) * 30.0)
    allv = np.concatenate([vals, rnd]).astype(np.float32)
    got = dev.round_to_bf16_bits(torch.tensor(allv, device=dev.torch_device)).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, orc.to_bf16_bits(allv.astype(np.float64)))
    nan = dev.round_to_bf16_bits(torch.tensor([float("nan")], device=dev.torch_device)).cpu().numpy().view(np.uint16)
    assert (nan[0] & 0x7FC0) == 0x7FC0


def test_u32_store_saturates(dev):
    x = torch.tensor([0.0, 3.0, 128255.0, float("inf"), 5e9, -1.0], device=dev.torch_device)
    got = dev.store_u32_saturating(x).cpu().numpy().view(np.uint32)
    assert got.tolist() == [0, 3, 128255, 0xFFFFFFFF, 0xFFFFFFFF, 0]   # reference src/emit_metal.rs:186-190


def test_rmsnorm_and_rope(dev):
    x = orc.round_to(orc.DT_F32, normal(61, 5, 2048))
    g, gv = bf16t(1.0 + 0.1 * normal(62, 2048), dev)
    exp = orc.round_to(orc.DT_BF16, orc.rms_norm(x, gv))
    got = dev.rmsnorm(f32t(x, dev), g).float().cpu().numpy()
    assert nerr(got, exp) <= 2.0 ** -7      # at most one bf16 ulp on a rounding boundary
    assert np.mean(got == exp) > 0.999
    # rotate-half RoPE on bf16 rows, positions 0..seq-1 (reference src/nn.rs:176-194)
    xr, xrv = bf16t(normal(63, 2, 3, 40, 64), dev)
    inv = orc.rope_inv_freq(500000.0, 32)
    table = dev.rope_table(list(inv), 48)
    exp = orc.round_to(orc.DT_BF16, orc.rope(xrv, np.arange(40.0)[None, None, :], inv))
    got = dev.rope_bf16(xr, table).float().cpu().numpy()
    assert nerr(got, exp) <= 2.0 ** -7
    assert np.mean(got == exp) > 0.995


def test_embed_gather(dev):
    t, tv = bf16t(normal(71, 50, 64), dev)
    tok = torch.tensor([3, 49, 0], dtype=torch.int32, device=dev.torch_device)
    assert np.array_equal(dev.embed_gather(t, tok).cpu().numpy().astype(np.float64), tv[[3, 49, 0]])


# ───────────────────────── deferred-normaliser contraction (tcgen05) ─────────────────────────
def _gemm_case(dev, M, K, N, w_is_nk, out_dtype=torch.bfloat16, seed=81):
    x, xv = bf16t(normal(seed, M, K), dev)
    g, gv = bf16t(1.0 + 0.1 * normal(seed + 1, K), dev)
    wshape = (N, K) if w_is_nk else (K, N)
    w, wv = bf16t(0.02 * normal(seed + 2, *wshape), dev)
    y = dev.gemm_rmsnorm(x, g, w, eps=1e-5, w_is_nk=w_is_nk, out_dtype=out_dtype)
    dev.sync()     # surfaces a bounded wait that ran out as an error instead of a hang
    exp = orc.rmsnorm_gemm(xv, gv, wv, eps=1e-5, w_is_nk=w_is_nk)
    got = y.float().cpu().numpy()
    # bf16 rounding of x*g (2^-9 per term, random sign) then of the output
    assert nerr(got, exp) <= BF16_TOL
    # the carrier form (two Add slots, divide once) is what the kernel computes
    car = orc.rmsnorm_gemm(xv[:4], gv, wv, eps=1e-5, w_is_nk=w_is_nk, blocks=4)
    assert nerr(got[:4], car) <= BF16_TOL
    return got, exp


@pytest.mark.parametrize("w_is_nk", [True, False])
def test_gemm_rmsnorm_one_tile(dev, w_is_nk):
    _gemm_case(dev, 128, 256, 256, w_is_nk)


@pytest.mark.parametrize("w_is_nk", [True, False])
def test_gemm_rmsnorm_multi_tile_and_edges(dev, w_is_nk):
    _gemm_case(dev, 384, 512, 768, w_is_nk, out_dtype=torch.float32)
    _gemm_case(dev, 200, 320, 264, w_is_nk)       # ragged M, K not a multiple of 64, N not a multiple of 256


def test_gemm_rmsnorm_many_tiles_per_cta(dev):
    # more tiles than SMs: exercises the accumulator double buffer and barrier phases
    got, exp = _gemm_case(dev, 2048, 256, 8192, True)
    assert got.shape == (2048, 8192)


@pytest.mark.parametrize("form", ["0", "1", "2"])
def test_gemm_rmsnorm_both_tile_forms(dev, form, monkeypatch):
    # SANIC_GEMM_PAIR forces the one-CTA 128 x 256 tile ("0") or the 256 x 256 tile on a pair of SMs ("1": two CTAs of a
    # cluster, tcgen05 cta_group::2, bulk tensor stores); without it the library picks by problem size
    monkeypatch.setenv("SANIC_GEMM_PAIR", form)
    for nk in (True, False):
        _gemm_case(dev, 128, 256, 256, nk)                                  # one CTA of the pair has no rows at all
        _gemm_case(dev, 384, 512, 768, nk, out_dtype=torch.float32)         # direct f32 stores
        _gemm_case(dev, 200, 320, 264, nk)                                  # ragged M, K, N: the bulk stores clip at the edges
    got, exp = _gemm_case(dev, 2048, 256, 8192, True)                       # several tiles per pair: ring and accumulator phases
    assert got.shape == (2048, 8192)
    _gemm_case(dev, 512, 8192, 256, True)                                   # the longest K: staging does not fit, direct stores


def test_gemm_rmsnorm_pair_profile_counts_clocks_and_computes(dev):
    """The profile entry point runs the pair tile with A through registers with its clock counters on: the result is the
    contraction's, and the counters are those of a run (every k-block issued, clocks in every role)."""
    M, K, N = 512, 512, 512
    x, xv = bf16t(normal(201, M, K), dev)
    g, gv = bf16t(1.0 + 0.1 * normal(202, K), dev)
    w, wv = bf16t(0.02 * normal(203, N, K), dev)
    prof, y = dev.gemm_rmsnorm_pair_profile(x, g, w, w_is_nk=True)
    assert nerr(y.float().cpu().numpy(), orc.rmsnorm_gemm(xv, gv, wv, eps=1e-5, w_is_nk=True)) <= BF16_TOL
    kb = K // 64
    assert prof["k_blocks"] == kb * 1                              # pair 0 owns one of the four 256 x 256 tiles
    assert prof["mma_thread_clocks_per_kb"] > 100 and prof["b_producer_wait_per_kb"] >= 0
    for side in ("leader", "peer"):
        t = prof["transform_warp_" + side]
        assert t["k_blocks"] == kb // 4 and t["arithmetic"] > 0 and t["stores"] > 0


@pytest.mark.parametrize("w_is_nk", [True, False])
def test_gemm_rmsnorm_with_prescaled_weights(dev, w_is_nk):
    # weights bound once: W' = bf16(W * g) along K, then the contraction with gamma = None; the rewrite
    # sum (x*g)*W = sum x*(g*W) rounds g*W instead of x*g, the same one bf16 rounding per term
    for M, K, N in ((128, 256, 256), (200, 320, 264), (1024, 512, 2048)):
        x, xv = bf16t(normal(91, M, K), dev)
        g, gv = bf16t(1.0 + 0.1 * normal(92, K), dev)
        w, wv = bf16t(0.02 * normal(93, *((N, K) if w_is_nk else (K, N))), dev)
        ws = dev.gemm_prescale_weights(g, w, w_is_nk=w_is_nk)
        scaled = orc.round_to(orc.DT_BF16, wv * (gv[None, :] if w_is_nk else gv[:, None]))
        assert np.array_equal(ws.float().cpu().numpy().astype(np.float64), scaled)          # the pre-scale is one exact RNE
        y = dev.gemm_rmsnorm(x, None, ws, eps=1e-5, w_is_nk=w_is_nk)
        dev.sync()
        exp = orc.rmsnorm_gemm(xv, gv, wv, eps=1e-5, w_is_nk=w_is_nk)
        assert nerr(y.float().cpu().numpy(), exp) <= BF16_TOL
        # against the oracle fed the pre-scaled weights (gamma = 1) the only differences are accumulation order and the output rounding
        exp2 = orc.rmsnorm_gemm(xv, np.ones(K), scaled, eps=1e-5, w_is_nk=w_is_nk)
        assert nerr(y.float().cpu().numpy(), exp2) <= 2.0 ** -7


# ───────────────────────── prefill online-softmax fold (tcgen05) ─────────────────────────
def _flash_case(dev, B, Hq, Hkv, Lq, Lk, mode, window=0, seed=91):
    q, qv = bf16t(normal(seed, B, Hq, Lq, 64), dev)
    k, kv = bf16t(normal(seed + 1, B, Hkv, Lk, 64), dev)
    v, vv = bf16t(normal(seed + 2, B, Hkv, Lk, 64), dev)
    if mode == "plain":
        exp = orc.sdpa(qv, kv, vv, enable_gqa=True)
        got = dev.attn_fwd_bf16(q, k, v)
    elif mode == "causal":
        exp = orc.sdpa(qv, kv, vv, is_causal=True, enable_gqa=True)
        got = dev.attn_fwd_bf16(q, k, v, causal=True)
    else:
        exp = orc.sdpa_window(qv, kv, vv, window)
        got = dev.attn_fwd_bf16(q, k, v, causal=True, window=window)
    dev.sync()
    assert nerr(got.float().cpu().numpy(), exp) <= BF16_TOL


@pytest.mark.parametrize("mode", ["plain", "causal"])
@pytest.mark.parametrize("L", [128, 256, 384, 640])
def test_flash_fwd_square(dev, mode, L):
    _flash_case(dev, 1, 4, 2, L, L, mode)


def test_flash_fwd_ragged_and_gqa(dev):
    _flash_case(dev, 2, 8, 2, 200, 300, "plain")      # ragged key tail, query tail, rectangular
    _flash_case(dev, 1, 4, 1, 77, 77, "causal")       # shorter than one tile
    _flash_case(dev, 1, 2, 2, 1000, 1000, "causal")   # ragged on both axes, 4 query blocks


@pytest.mark.parametrize("window", [1, 100, 128, 300])
def test_flash_fwd_sliding_window(dev, window):
    _flash_case(dev, 1, 4, 2, 700, 700, "window", window=window)


@pytest.mark.parametrize("mode", ["plain", "causal", "window"])
def test_flash_fwd_many_items_equals_single_round_calls(dev, mode):
    # The forward kernel is persistent: one block per SM walks a list of (query block, head, batch) items,
    # double-buffering the query tiles and reusing its tensor memory from item to item. A call with several
    # items per block must give, bit for bit, what the same rows give when every (batch, kv head) is its own
    # small call (at most one item per block).
    B, Hq, Hkv, L = 3, 16, 4, 1100
    g = torch.Generator(device=dev.torch_device); g.manual_seed(23)
    q = torch.randn(B, Hq, L, 64, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, L, 64, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, L, 64, generator=g, device=dev.torch_device).to(torch.bfloat16)
    kw = dict(causal=(mode != "plain"), window=(200 if mode == "window" else 0))
    big = dev.attn_fwd_bf16(q, k, v, **kw)       # 5 query blocks x 16 heads x 3 = 240 items on 148 blocks
    dev.sync()
    grp = Hq // Hkv
    for b in range(B):
        for hk in range(Hkv):
            small = dev.attn_fwd_bf16(q[b:b + 1, hk * grp:(hk + 1) * grp].contiguous(), k[b:b + 1, hk:hk + 1].contiguous(),
                                      v[b:b + 1, hk:hk + 1].contiguous(), **kw)
            dev.sync()
            assert torch.equal(small[0], big[b, hk * grp:(hk + 1) * grp]), (b, hk)


@pytest.mark.parametrize("mode", ["plain", "causal", "window"])
def test_flash_fwd_running_maximum_rises_across_key_tiles(dev, mode):
    # Keys grow with their position, so a row's maximum rises by more than 2^8 from one key tile to the next: every later
    # tile moves the row's reference, which is the case in which the half of the exponentials taken against the old
    # reference is redone and O and l are rescaled (with i.i.d. scores only an item's first key tile sets a reference).
    B, Hq, Hkv, L = 1, 4, 2, 640
    q, qv = bf16t(normal(311, B, Hq, L, 64), dev)
    ramp = (1.0 + np.arange(L) / 32.0)[None, None, :, None]
    k, kv = bf16t(normal(312, B, Hkv, L, 64) * ramp, dev)
    v, vv = bf16t(normal(313, B, Hkv, L, 64), dev)
    if mode == "plain":
        exp, got = orc.sdpa(qv, kv, vv, enable_gqa=True), dev.attn_fwd_bf16(q, k, v)
    elif mode == "causal":
        exp, got = orc.sdpa(qv, kv, vv, is_causal=True, enable_gqa=True), dev.attn_fwd_bf16(q, k, v, causal=True)
    else:
        exp, got = orc.sdpa_window(qv, kv, vv, 300), dev.attn_fwd_bf16(q, k, v, causal=True, window=300)
    dev.sync()
    assert nerr(got.float().cpu().numpy(), exp) <= BF16_TOL


def test_flash_fwd_profile_counts_clocks_and_computes(dev):
    """The profile entry point runs the same fold with clock counters on in CTA 0: the output is bit for bit the plain
    call's, and the counters are those of a run (CTA 0's item is the last query block: 5 and 6 key tiles)."""
    B, Hq, Hkv, L = 1, 4, 2, 700
    q, _ = bf16t(normal(301, B, Hq, L, 64), dev)
    k, _ = bf16t(normal(302, B, Hkv, L, 64), dev)
    v, _ = bf16t(normal(303, B, Hkv, L, 64), dev)
    plain = dev.attn_fwd_bf16(q, k, v, causal=True)
    prof, out = dev.attn_fwd_bf16_profile(q, k, v, causal=True)
    dev.sync()
    assert torch.equal(plain, out)
    assert prof["tile0"]["key_tiles"] == 5 and prof["tile1"]["key_tiles"] == 6
    for t in ("tile0", "tile1"):
        per = prof[t]["clocks_per_key_tile"]
        assert per["first_half_exponentials"] > 0 and per["load_scores"] > 0 and per["row_max"] > 0
        assert abs(sum(per.values()) * prof[t]["key_tiles"] - prof[t]["clocks"]) <= 10 * prof[t]["key_tiles"] + 10
    for t, tiles in ((0, 5), (1, 6)):
        assert prof[f"mma_thread{t}"]["qk_issued"] == tiles and prof[f"mma_thread{t}"]["polls"] >= tiles


def test_flash_fwd_rope_pipeline_long(dev):
    # size-independent checks at a longer sequence: causal row 0 equals V row 0, and the output is
    # unchanged when keys beyond the causal edge are replaced (they must never be read into a result)
    B, Hq, Hkv, L = 1, 8, 2, 2048
    g = torch.Generator(device=dev.torch_device); g.manual_seed(17)
    q = torch.randn(B, Hq, L, 64, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, L, 64, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, L, 64, generator=g, device=dev.torch_device).to(torch.bfloat16)
    inv = orc.rope_inv_freq(500000.0, 32)
    table = dev.rope_table(list(inv), L)
    qr, kr = dev.rope_bf16(q, table), dev.rope_bf16(k, table)
    out = dev.attn_fwd_bf16(qr, kr, v, causal=True)
    dev.sync()
    assert torch.equal(out[:, :, 0], v[:, :, 0].repeat_interleave(Hq // Hkv, dim=1))
    half = L // 2
    k2, v2 = kr.clone(), v.clone()
    k2[:, :, half:] = 7.0; v2[:, :, half:] = -3.0
    out2 = dev.attn_fwd_bf16(qr, k2, v2, causal=True)
    dev.sync()
    assert torch.equal(out[:, :, :half], out2[:, :, :half])
    # one head against the oracle
    exp = orc.sdpa(qr[0, :4].float().cpu().numpy().astype(np.float64), kr[0, :1].float().cpu().numpy().astype(np.float64),
                   v[0, :1].float().cpu().numpy().astype(np.float64), is_causal=True, enable_gqa=True)
    assert nerr(out[0, :4].float().cpu().numpy(), exp) <= BF16_TOL


def test_splitkv_peer_exchange_single_rank(dev):
    # world size 1: the peer-memory exchange kernel stores into its own buffer, flags itself and merges one
    # accumulator set; three steps cover both buffer parities. Output equals the NCCL-form call (which at one
    # rank is fold + merge) bit for bit.
    from sanic_b200.splitkv import SplitKVDecoder
    B, Hq, Hkv, D, n = 2, 8, 2, 128, 1000
    g = torch.Generator(device=dev.torch_device); g.manual_seed(31)
    k = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    a = SplitKVDecoder(dev, k, v, n_splits=4, init_nccl=False)
    b = SplitKVDecoder(dev, k, v, n_splits=4, init_nccl=False, exchange="peer")
    for step in range(3):
        q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
        oa = a.step(q).clone(); ob = b.step(q).clone()
        dev.sync()
        assert torch.equal(oa, ob), step
    exp = orc.sdpa(q.float().cpu().numpy().astype(np.float64)[:, :, None, :], k.float().cpu().numpy().astype(np.float64),
                   v.float().cpu().numpy().astype(np.float64), enable_gqa=True)[:, :, 0, :]
    assert nerr(ob.float().cpu().numpy(), exp) <= BF16_TOL
    b.close()


# ───────────────────────── stream-K form of the decode fold, and the fused multi-device step ─────────────────────────
@pytest.mark.parametrize("D,vt", [(64, True), (128, False), (64, False)])
@pytest.mark.parametrize("kv_len,window", [(1, 0), (63, 0), (65, 0), (1000, 0), (5000, 0), (5000, 700), (40000, 0)])
def test_decode_streamk_matches_the_oracle_and_the_chunked_form(dev, D, vt, kv_len, window):
    B, Hq, Hkv, S = 2, 8, 2, 40000 if kv_len > 5000 else 5056
    g = torch.Generator(device=dev.torch_device); g.manual_seed(kv_len + D)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    vdev = v.transpose(2, 3).contiguous() if vt else v
    out, car = dev.attn_decode(q, k, vdev, kv_len, v_transposed=vt, window=window, streamk=True, return_carrier=True,
                               out_dtype=torch.float32)
    ref = dev.attn_decode(q, k, vdev, kv_len, v_transposed=vt, window=window, n_splits=3, out_dtype=torch.float32)
    dev.sync()
    assert nerr(out.cpu().numpy(), ref.cpu().numpy()) <= 2e-3            # another chunking of the same fold
    lo = max(0, kv_len - window) if window else 0
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    exp = orc.sdpa(f64(q[:1]).reshape(1, Hq, 1, D), f64(k[:1, :, lo:kv_len]), f64(v[:1, :, lo:kv_len]), enable_gqa=True).reshape(Hq, D)
    assert nerr(out[0].cpu().numpy(), exp) <= BF16_TOL
    c = car.cpu().numpy().reshape(B, Hq, D + 2)
    assert nerr(c[0, :, 2:] / c[0, :, 1:2], exp) <= BF16_TOL
    # a second launch on the same scratch: the group tickets were reset by the first
    out2 = dev.attn_decode(q, k, vdev, kv_len, v_transposed=vt, window=window, streamk=True, out_dtype=torch.float32)
    dev.sync()
    assert torch.equal(out, out2)


def test_decode_streamk_many_groups_and_device_side_length(dev):
    # more (batch, kv head) groups than resident CTAs can split finely, and a length read from the device
    B, Hq, Hkv, D, S = 16, 32, 8, 64, 1056
    g = torch.Generator(device=dev.torch_device); g.manual_seed(5)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, D, S, generator=g, device=dev.torch_device).to(torch.bfloat16)
    pos = torch.tensor([1029], dtype=torch.int32, device=dev.torch_device)
    out = dev.attn_decode(q, k, v, 1, v_transposed=True, streamk=True, out_dtype=torch.float32, kv_len_dev=pos)
    ref = dev.attn_decode(q, k, v, 1030, v_transposed=True, n_splits=2, out_dtype=torch.float32)
    dev.sync()
    assert nerr(out.cpu().numpy(), ref.cpu().numpy()) <= 2e-3
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    exp = orc.sdpa(f64(q[15:, 28:]).reshape(1, 4, 1, D), f64(k[15:, 7:, :1030]), f64(v[15:, 7:, :, :1030]).transpose(0, 1, 3, 2), enable_gqa=True)
    assert nerr(out[15, 28:].cpu().numpy(), exp.reshape(4, D)) <= BF16_TOL


def test_splitkv_fused_exchange_single_rank(dev):
    # world size 1: the fused step's last arrivers store into the rank's own buffer, flag themselves and merge one
    # accumulator set; three steps cover both buffer parities
    from sanic_b200.splitkv import SplitKVDecoder
    B, Hq, Hkv, D, n = 2, 8, 2, 128, 3000
    g = torch.Generator(device=dev.torch_device); g.manual_seed(32)
    k = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    a = SplitKVDecoder(dev, k, v, n_splits=4, init_nccl=False)
    b = SplitKVDecoder(dev, k, v, init_nccl=False, exchange="fused", force_exchange=True)
    for step in range(3):
        q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
        oa = a.step(q).clone(); ob = b.step(q).clone()
        b.sync()
        assert nerr(ob.float().cpu().numpy(), oa.float().cpu().numpy()) <= 2.0 ** -7, step     # another chunking, one bf16 rounding
    exp = orc.sdpa(q.float().cpu().numpy().astype(np.float64)[:, :, None, :], k.float().cpu().numpy().astype(np.float64),
                   v.float().cpu().numpy().astype(np.float64), enable_gqa=True)[:, :, 0, :]
    assert nerr(ob.float().cpu().numpy(), exp) <= BF16_TOL
    b.close()


def test_measured_specs_and_in_context_tuning_of_the_decode_fold(dev):
    from sanic_b200 import abi, plan
    s = plan.measure_specs(dev)
    assert 4.0e12 < s.hbm_read_bandwidth < 9.0e12          # a read-only sweep of 1 GiB
    assert 8.0 < s.exp_per_clk_per_sm < 16.5               # 16 is the datasheet rate
    assert 0.0 < s.launch_overhead_empty < 2e-5
    B, Hq, Hkv, D, S = 4, 32, 8, 128, 16384
    g = torch.Generator(device=dev.torch_device); g.manual_seed(8)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    out = dev.empty((B, Hq, D), torch.float32)
    slots = max(64, dev.streamk_slots(B, Hkv, D))
    p, _keep = dev.decode_params(q, k, v, S, n_splits=slots, out=out, out_dtype=abi.F32)
    cands = [1, 4, 16, 64, 0]                              # fixed chunks per (batch, kv head); 0 = stream-K
    best, secs = plan.tune_decode(dev, p, cands, repeats=3)
    assert best in cands and len(secs) == len(cands) and all(0.0 < t < 1.0 for t in secs)
    assert secs[cands.index(best)] == min(secs)
    assert secs[cands.index(1)] > min(secs)                # one chunk per (batch, kv head) leaves most SMs idle
    # the buffers hold the last candidate's result, and it is right
    dev.sync()
    f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
    exp = orc.sdpa(f64(q[:1, :4]).reshape(1, 4, 1, D), f64(k[:1, :1]), f64(v[:1, :1]), enable_gqa=True).reshape(4, D)
    assert nerr(out[0, :4].cpu().numpy(), exp) <= BF16_TOL
