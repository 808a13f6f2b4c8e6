"""Parity at the full shapes of the five benchmark configurations, through the C ABI, against the CPU oracle.

The dense f64 oracle cannot evaluate these shapes whole in test time, so it is evaluated on a seeded SAMPLE of
the output (rows, (batch, head, row-block) tiles, one (batch, kv head)) while the device computes the full
problem; size-independent properties cover the rest. Tolerances are the stated ones: f32 storage 1e-5 (plain
relative error with f64 arithmetic, normalised error with f32 arithmetic), bf16 storage 2e-2 normalised,
greedy tokens identical (ties counted and printed).
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from llama_util import lockstep, make_oracle, prefill_on_device

pytestmark = pytest.mark.gpu

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


def f64(t):
    return t.float().cpu().numpy().astype(np.float64)


# ───────────── config 1: f32 attention Q [256x64], K, V [1024x64], scale 1/8 ─────────────
def test_c1_plain_relative_error(dev):
    rng = orc.Xorshift(0xC0F1601)
    q = orc.round_to(orc.DT_F32, rng.normal(256, 64))
    k = orc.round_to(orc.DT_F32, rng.normal(1024, 64))
    v = orc.round_to(orc.DT_F32, rng.normal(1024, 64))
    exp = orc.sdpa(q, k, v, scale=0.125)
    t = lambda a, *s: torch.tensor(np.asarray(a, dtype=np.float32), device=dev.torch_device).view(*s)
    args = (t(q, 1, 1, 256, 64), t(k, 1, 1, 1024, 64), t(v, 1, 1, 1024, 64))
    got64 = dev.attn_fwd_f32(*args, scale=0.125, f64_accumulate=True).cpu().numpy()[0, 0]
    got32 = dev.attn_fwd_f32(*args, scale=0.125).cpu().numpy()[0, 0]
    rel64 = float(np.max(np.abs(got64 - exp) / np.abs(exp)))
    rel32 = float(np.max(np.abs(got32 - exp) / np.abs(exp)))
    print(f"\nC1 max plain relative error: f64 arithmetic {rel64:.3e}, f32 arithmetic {rel32:.3e} "
          f"(smallest |expected| {np.min(np.abs(exp)):.3e}); normalised f32 {nerr(got32, exp):.3e}")
    assert rel64 <= 1e-5          # the stated bound, as plain relative error, zero crossings included
    assert rel64 <= 4 * np.finfo(np.float32).eps      # in fact one f32 rounding
    assert nerr(got32, exp) <= 1e-5


# ───────────── config 2: RMSNorm-fused GEMM 4096 x 2048 x 8192 ─────────────
def test_c2_full_shape_sampled_rows(dev, monkeypatch):
    M, K, N = 4096, 2048, 8192
    rng = np.random.default_rng(0xC2)
    xb = orc.to_bf16_bits(rng.standard_normal((M, K)))
    gb = orc.to_bf16_bits(1.0 + 0.1 * rng.standard_normal(K))
    wb = orc.to_bf16_bits(0.02 * rng.standard_normal((K, N)))          # the configuration's [K, N] layout
    up = lambda bits: torch.tensor(bits.view(np.int16), device=dev.torch_device).view(torch.bfloat16)
    x, g, w_kn = up(xb), up(gb), up(wb)
    w_nk = w_kn.t().contiguous()
    rows = np.sort(rng.choice(M, size=64, replace=False))
    rows[0], rows[-1] = 0, M - 1
    exp = orc.rmsnorm_gemm(orc.from_bf16_bits(xb[rows]), orc.from_bf16_bits(gb), orc.from_bf16_bits(wb), eps=1e-5, w_is_nk=False)
    worst = {}
    for form in ("0", "1", "2"):                # one-CTA 128x256 tile, and the 256x256 tile on SM pairs
        monkeypatch.setenv("SANIC_GEMM_PAIR", form)
        for nk, w in ((False, w_kn), (True, w_nk)):
            y = dev.gemm_rmsnorm(x, g, w, eps=1e-5, w_is_nk=nk)
            dev.sync()
            assert y.shape == (M, N)
            worst[(form, nk)] = nerr(f64(y[torch.as_tensor(rows, device=y.device)]), exp)
            ws = dev.gemm_prescale_weights(g, w, w_is_nk=nk)
            y2 = dev.gemm_rmsnorm(x, None, ws, eps=1e-5, w_is_nk=nk)
            dev.sync()
            worst[(form, nk, "prescaled")] = nerr(f64(y2[torch.as_tensor(rows, device=y.device)]), exp)
            # a property over the WHOLE output: the two weight layouts describe the same contraction (same products,
            # at most a different accumulation order: within one bf16 rounding of each other)
            if nk:
                assert nerr(f64(y), f64(y_prev)) <= 2.0 ** -7, "the [N,K] and [K,N] layouts disagree"
            y_prev = y
    print("\nC2 normalised error on 64 sampled rows:", {k: f"{v:.2e}" for k, v in worst.items()})
    assert max(worst.values()) <= BF16_TOL


# ───────────── config 3: causal flash with RoPE, B8 Hq32 Hkv8 D64 S4096 (+ window 1024) ─────────────
def _c3_inputs(dev):
    B, Hq, Hkv, S, D = 8, 32, 8, 4096, 64
    g = torch.Generator(device=dev.torch_device); g.manual_seed(0xC3)
    q = torch.randn(B, Hq, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    inv = orc.rope_inv_freq(500000.0, D // 2)
    table = dev.rope_table(list(inv), S)
    return q, k, v, inv, dev.rope_bf16(q, table), dev.rope_bf16(k, table)


@pytest.mark.parametrize("window", [0, 1024])
def test_c3_full_shape_sampled_blocks(dev, window):
    B, Hq, Hkv, S, D = 8, 32, 8, 4096, 64
    q, k, v, inv, qr, kr = _c3_inputs(dev)
    out = dev.attn_fwd_bf16(qr, kr, v, causal=True, window=window)
    dev.sync()
    assert out.shape == (B, Hq, S, D)
    # property over the whole output: causal row 0 sees key 0 only
    assert torch.equal(out[:, :, 0], v[:, :, 0].repeat_interleave(Hq // Hkv, dim=1))
    worst, worst_rope = 0.0, 0.0
    # (batch, query head, first row of a 128-row block): first, middle and last blocks, first and last heads
    for b, h, r0 in ((0, 0, 0), (3, 13, 1920), (7, 31, S - 128), (5, 6, 1024), (1, 27, 2944)):
        hk = h // (Hq // Hkv)
        hi = r0 + 128
        pos_q = np.arange(r0, hi, dtype=np.float64)
        pos_k = np.arange(0, hi, dtype=np.float64)
        # the oracle applies RoPE itself to the raw inputs, then rounds to the declared bf16 storage
        q_o = orc.round_to(orc.DT_BF16, orc.rope(f64(q[b, h, r0:hi]), pos_q, inv))
        k_o = orc.round_to(orc.DT_BF16, orc.rope(f64(k[b, hk, :hi]), pos_k, inv))
        worst_rope = max(worst_rope, nerr(f64(qr[b, h, r0:hi]), q_o), nerr(f64(kr[b, hk, :hi]), k_o))
        rows = np.arange(r0, hi)[:, None]
        cols = np.arange(hi)[None, :]
        vis = cols <= rows
        if window:
            vis &= cols > rows - window
        mask = np.where(vis, 0.0, -1e30)      # computed masks are -1e30 (src/ir.rs:1522)
        exp = orc.sdpa(q_o.reshape(1, 1, 128, D), k_o.reshape(1, 1, hi, D), f64(v[b, hk, :hi]).reshape(1, 1, hi, D), mask=mask)
        worst = max(worst, nerr(f64(out[b, h, r0:hi]), exp[0, 0]))
    print(f"\nC3 window {window}: attention normalised error {worst:.2e}, RoPE {worst_rope:.2e} on 5 sampled 128-row blocks")
    assert worst_rope <= 2.0 ** -7      # one bf16 rounding of values computed in f32 instead of f64
    assert worst <= BF16_TOL


# ───────────── config 4: Llama-3.2-1B architecture, ctx 1024, 32 greedy steps ─────────────
# Token identity is asserted step by step inside `lockstep`: a token that differs from the oracle's is an error unless the
# oracle's own top-2 gap on that row lies inside the bf16 bound (then both indices are maxima to within the storage
# precision). Such near-ties are counted and printed. Random-init logits are nearly flat, and the trajectory is chaotic in
# the last bits of the prefilled cache (which the device writes), so which steps meet a near-tie is not stable under any
# change of summation order: over seeds 1-3 the bf16 batch-1 case has met 0 to 2 of them in its 32 steps, with gaps of
# 2.6e-4 to 7.8e-3.
C4_SEED = 1


@pytest.mark.parametrize("batch", [1, 16])
@pytest.mark.parametrize("w4", [False, True])
def test_c4_full_architecture_32_greedy_steps(dev, batch, w4):
    from sanic_b200 import llama
    cfg, prefill, steps = llama.LLAMA_3_2_1B, 1024, 32
    ctx = prefill + steps
    w = llama.random_weights(cfg, C4_SEED, dev.torch_device, w4=w4)
    # The forms the benchmark times: the launch list with the deferred normaliser (stored(x * gamma): the oracle moves its
    # rounding point with it) and, at batch 1, the single-kernel step (which rounds at stored(rms_norm(x)): an oracle of its
    # own). The single-kernel step at batch 16 is covered on the small model (tests/test_gpu_llama.py).
    groups = [dict(list=llama.LlamaMachine(dev, cfg, w, ctx=ctx, batch=batch, w4=w4))]
    if batch == 1:
        groups.append(dict(persistent=llama.LlamaMachine(dev, cfg, w, ctx=ctx, batch=batch, w4=w4, persistent=True)))
    for forms in groups:
        deferred = next(iter(forms.values())).deferred_norm
        o = make_oracle(cfg, w, ctx, batch, w4, norm_store=2 if deferred else 0)
        rng = np.random.default_rng(C4_SEED)
        prefill_on_device(list(forms.values()), o, cfg, prefill, rng)
        stats = lockstep(list(forms.values()), o, cfg, prefill, steps, rng, label=f"w4={w4} batch={batch}")
        for name, st in zip(forms, stats):
            print(f"\nC4 {'int4' if w4 else 'bf16'} batch {batch} {name}: {st['ties']} near-ties in {steps * batch} token steps "
                  f"(worst tie gap {st['worst_gap']:.3e}; smallest oracle top-2 gap seen {st['min_gap']:.3e}); "
                  f"max normalised logit error {st['err']:.3e}, relative rms {st['rms']:.3e}")
            assert st["ties"] <= max(2, steps * batch // 16)


# ───────────── config 5: split-KV decode, 1,048,576 keys per sequence ─────────────
def test_c5_full_length_one_kv_head_against_the_oracle(dev):
    Hq, D, S = 4, 128, 1 << 20           # the GQA group of one kv head
    g = torch.Generator(device=dev.torch_device); g.manual_seed(0xC5)
    q = torch.randn(1, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(1, 1, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(1, 1, S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    out, car = dev.attn_decode(q, k, v, S, n_splits=148, return_carrier=True, out_dtype=torch.float32)
    dev.sync()
    # the oracle folds the axis in 16 chunks of 65,536 keys (run_carrier_split, src/interp.rs:597-640) and merges
    qv = f64(q).reshape(1, Hq, 1, D)
    parts = []
    step = S // 16
    for c in range(16):
        _, pc = orc.sdpa_carrier_split(qv, f64(k[:, :, c * step:(c + 1) * step]), f64(v[:, :, c * step:(c + 1) * step]), 1,
                                       enable_gqa=True, return_carriers=True)
        parts.append(pc.reshape(Hq, D + 2))
    exp = orc.carrier_merge_mlo(np.stack(parts))
    err = nerr(out.cpu().numpy()[0], exp)
    print(f"\nC5 2^20 keys, one kv head: normalised error {err:.2e}")
    assert err <= BF16_TOL


def test_c5_full_shape_properties(dev):
    # B4 Hq32 Hkv8 D128, 2^20 keys: 17 GB of K and V. Any chunking gives the same answer, two device-level halves
    # merged with the derived combine equal the whole, and one (batch, kv head) of the whole equals the oracle sample.
    B, Hq, Hkv, D, S = 4, 32, 8, 128, 1 << 20
    g = torch.Generator(device=dev.torch_device); g.manual_seed(0xC5)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.empty(B, Hkv, S, D, dtype=torch.bfloat16, device=dev.torch_device)
    v = torch.empty(B, Hkv, S, D, dtype=torch.bfloat16, device=dev.torch_device)
    for b in range(B):
        for h in range(Hkv):
            k[b, h] = torch.randn(S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
            v[b, h] = torch.randn(S, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    a = dev.attn_decode(q, k, v, S, n_splits=37, out_dtype=torch.float32)
    b_ = dev.attn_decode(q, k, v, S, n_splits=64, out_dtype=torch.float32)
    dev.sync()
    assert nerr(a.cpu().numpy(), b_.cpu().numpy()) <= 2e-3
    half = S // 2
    _, c0 = dev.attn_decode(q, k[:, :, :half], v[:, :, :half], half, n_splits=19, return_carrier=True)
    _, c1 = dev.attn_decode(q, k[:, :, half:], v[:, :, half:], half, n_splits=19, return_carrier=True)
    merged = dev.carrier_merge(torch.stack([c0, c1])).cpu().numpy().reshape(B, Hq, D)
    assert nerr(merged, a.cpu().numpy()) <= 2e-3
    # the last (batch, kv head) against the oracle on a 131,072-key prefix folded with the same kernel
    n = 1 << 17
    sub = dev.attn_decode(q[3:, 28:].contiguous(), k[3:, 7:, :n], v[3:, 7:, :n], n, n_splits=8, out_dtype=torch.float32)
    exp = orc.sdpa(f64(q[3:, 28:]).reshape(1, 4, 1, D), f64(k[3:, 7:, :n]), f64(v[3:, 7:, :n]), enable_gqa=True).reshape(1, 4, D)
    assert nerr(sub.cpu().numpy(), exp) <= BF16_TOL
    del k, v
    torch.cuda.empty_cache()
