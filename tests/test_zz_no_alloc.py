"""The allocation-free decode entry point against the ordinary one.

`sanic_attn_decode_splitkv_static` exists for hosts that must not allocate device memory where
they decode: a serving loop where an allocation would stall the device,
a plugin that is given a fixed arena, a process whose memory is budgeted up front. Its split-KV
scratch is a static array inside the library instead of a caller buffer. This file calls it
through the C ABI twice in a row (the second call meets whatever the first left in the shared
array) and requires the same output as `sanic_attn_decode_splitkv` within the bf16 bound the
other GPU tests use; the kernel is deterministic, so in practice the bits are identical. It is
named to be collected last: if it fails under `-x`, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2


def _nerr(a, b):
    a = a.float().cpu().numpy().astype(np.float64)
    b = b.float().cpu().numpy().astype(np.float64)
    assert np.all(np.isfinite(a)) and np.all(np.isfinite(b))
    return float(np.max(np.abs(a - b) / (1.0 + np.abs(b))))


def test_static_scratch_decode_matches_caller_scratch_twice():
    from sanic_b200 import CudaDevice, abi
    dev = CudaDevice(0)
    td = dev.torch_device
    g = torch.Generator(device=td)
    g.manual_seed(2024)
    B, Hq, Hkv, D, S = 2, 16, 4, 128, 4096
    k = torch.randn(B, Hkv, S, D, generator=g, device=td).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D, generator=g, device=td).to(torch.bfloat16)
    for call, (kv_len, n_splits) in enumerate(((4096, 6), (1000, 3))):
        q = torch.randn(B, Hq, D, generator=g, device=td).to(torch.bfloat16)
        ref = dev.empty((B, Hq, D), torch.float32)
        ref_car = dev.empty((B * Hq, D + 2), torch.float32)
        p, _keep = dev.decode_params(q, k, v, kv_len, n_splits=n_splits, out=ref, carrier_out=ref_car, out_dtype=abi.F32)
        dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
        got = dev.empty((B, Hq, D), torch.float32)
        got_car = dev.empty((B * Hq, D + 2), torch.float32)
        ps, _keep2 = dev.decode_params(q, k, v, kv_len, n_splits=n_splits, out=got, carrier_out=got_car, out_dtype=abi.F32)
        ps.partials = None                       # the static entry point brings its own scratch
        rc = dev.lib.sanic_attn_decode_splitkv_static(dev.h, C.byref(ps), dev.stream())
        dev._check(rc, "decode_static")
        torch.cuda.synchronize()
        assert _nerr(got, ref) <= BF16_TOL, f"call {call}"
        assert _nerr(got_car[:, 1:], ref_car[:, 1:]) <= BF16_TOL, f"call {call}"
        assert torch.equal(got, ref), f"call {call}: the two entry points run the same deterministic kernel"
        # and both agree with the CPU oracle on one (batch, kv head)
        from oracle import oracle as orc
        f64 = lambda t: t.float().cpu().numpy().astype(np.float64)
        exp = orc.sdpa(f64(q[1:, 12:]).reshape(1, 4, 1, D), f64(k[1:, 3:, :kv_len]), f64(v[1:, 3:, :kv_len]), enable_gqa=True)
        assert np.max(np.abs(f64(got[1, 12:]) - exp.reshape(4, D)) / (1.0 + np.abs(exp.reshape(4, D)))) <= BF16_TOL


def test_static_scratch_rejects_oversized_requests():
    from sanic_b200 import CudaDevice, abi
    dev = CudaDevice(0)
    td = dev.torch_device
    cap = dev.lib.sanic_attn_decode_static_scratch_capacity()
    assert cap == 4 << 20
    B, Hq, Hkv, D, S = 4, 32, 8, 128, 256
    q = torch.zeros(B, Hq, D, dtype=torch.bfloat16, device=td)
    k = torch.zeros(B, Hkv, S, D, dtype=torch.bfloat16, device=td)
    out = dev.empty((B, Hq, D), torch.float32)
    n_splits = cap // 4 // (B * Hq * (D + 2)) + 1          # one chunk too many for the built-in array
    p, _keep = dev.decode_params(q, k, k, S, n_splits=n_splits, out=out, out_dtype=abi.F32,
                                 partials=torch.zeros(1, device=td))
    rc = dev.lib.sanic_attn_decode_splitkv_static(dev.h, C.byref(p), dev.stream())
    assert rc == abi.ERR_INVALID
    assert b"exceeds the built-in scratch" in dev.lib.sanic_last_error(dev.h)
    # the other limit, one ticket counter per (batch, kv head), has its own message
    B2, H2 = 4100, 1
    q2 = torch.zeros(B2, H2, 64, dtype=torch.bfloat16, device=td)
    k2 = torch.zeros(B2, H2, 8, 64, dtype=torch.bfloat16, device=td)
    p2, _keep = dev.decode_params(q2, k2, k2, 8, n_splits=1, out=dev.empty((B2, H2, 64), torch.float32), out_dtype=abi.F32,
                                  partials=torch.zeros(1, device=td))
    assert dev.lib.sanic_attn_decode_splitkv_static(dev.h, C.byref(p2), dev.stream()) == abi.ERR_INVALID
    assert b"ticket counters" in dev.lib.sanic_last_error(dev.h)
