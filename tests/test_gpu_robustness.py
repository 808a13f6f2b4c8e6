"""Error paths that must return, not hang or read out of range. Every failure here is made on the host or by a
wait that simply runs out: no test faults, traps or hangs the device (the reference surfaces device failures as
`Err(String)` from `run_graph_timed`, src/metal.rs:686-705, and typed `RunError`s, src/compile.rs:41-76).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2
SMALL = dict(vocab=1024, layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=512)


@pytest.fixture(scope="module")
def dev():
    from sanic_b200 import CudaDevice
    return CudaDevice(0)


def nerr(got, exp):
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64)
    assert np.all(np.isfinite(got)), "non-finite values in the GPU result"
    return float(np.max(np.abs(got - exp) / (1.0 + np.abs(exp))))


def bf16t(a, dev):
    bits = orc.to_bf16_bits(a)
    return torch.tensor(bits.view(np.int16), device=dev.torch_device).view(torch.bfloat16), orc.from_bf16_bits(bits)


@pytest.mark.parametrize("vt", [False, True])
def test_device_length_past_the_cache_is_clamped_and_reported(dev, vt):
    from sanic_b200 import RunError, abi
    B, Hq, Hkv, D, S = 1, 8, 2, 64, 200
    rng = orc.Xorshift(0xCA9)
    q, qv = bf16t(rng.normal(B, Hq, D), dev)
    k, kv = bf16t(rng.normal(B, Hkv, S, D), dev)
    v, vv = bf16t(rng.normal(B, Hkv, S, D), dev)
    vdev = v.transpose(2, 3).contiguous() if vt else v
    # the buffers end right after the cache: a read past kv_cap would leave the allocation's slice
    pos = torch.tensor([S + 500], dtype=torch.int32, device=dev.torch_device)
    out = dev.empty((B, Hq, D), torch.float32)
    p, _keep = dev.decode_params(q, k, vdev, 1, v_transposed=vt, n_splits=3, kv_len_dev=pos, out=out, out_dtype=abi.F32,
                                 kv_cap=S)
    dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
    with pytest.raises(RunError, match="code 52"):
        dev.sync()
    # the clamped call folded exactly the cache, nothing beyond it
    exp = orc.sdpa(qv.reshape(B, Hq, 1, D), kv, vv, enable_gqa=True).reshape(B, Hq, D)
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL
    # the context is usable afterwards and an in-range position reports nothing
    pos.fill_(S - 1)
    dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
    dev.sync()
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL
    # a negative position is clamped to one key
    pos.fill_(-7)
    dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
    with pytest.raises(RunError, match="code 52"):
        dev.sync()


def test_decode_params_need_a_capacity_that_fits_the_strides(dev):
    from sanic_b200 import RunError, abi
    B, Hq, Hkv, D, S = 2, 4, 2, 64, 64
    q = torch.zeros(B, Hq, D, dtype=torch.bfloat16, device=dev.torch_device)
    k = torch.zeros(B, Hkv, S, D, dtype=torch.bfloat16, device=dev.torch_device)
    pos = torch.zeros(1, dtype=torch.int32, device=dev.torch_device)
    out = dev.empty((B, Hq, D), torch.float32)
    for cap, kv_len_dev, kv_len in ((0, pos, 1), (S + 1, pos, 1), (S + 8, None, S + 8), (32, None, 33)):
        p, _keep = dev.decode_params(q, k, k, kv_len, n_splits=1, kv_len_dev=kv_len_dev, out=out, out_dtype=abi.F32, kv_cap=cap)
        with pytest.raises(RunError):
            dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")
    vt = torch.zeros(B, Hkv, D, S, dtype=torch.bfloat16, device=dev.torch_device)
    p, _keep = dev.decode_params(q, k, vt, 1, v_transposed=True, n_splits=1, kv_len_dev=pos, out=out, out_dtype=abi.F32,
                                 kv_cap=S + 8)
    with pytest.raises(RunError):
        dev._check(dev.lib.sanic_attn_decode_splitkv(dev.h, C.byref(p), dev.stream()), "decode")


@pytest.mark.parametrize("kv_len", [1, 13, 67, 250])
def test_transposed_v_tail_beyond_the_visible_keys_is_never_read(dev, kv_len):
    # a recycled cache may hold NaN bit patterns beyond the visible prefix: 0 * NaN must not reach the output
    B, Hq, Hkv, D, S = 1, 8, 2, 64, 256
    rng = orc.Xorshift(0x7A11 + kv_len)
    q, qv = bf16t(rng.normal(B, Hq, D), dev)
    k, kv = bf16t(rng.normal(B, Hkv, S, D), dev)
    v, vv = bf16t(rng.normal(B, Hkv, S, D), dev)
    vt = v.transpose(2, 3).contiguous()
    vt[..., kv_len:] = float("nan")
    k2 = k.clone(); k2[:, :, kv_len:] = float("nan")
    out = dev.attn_decode(q, k2, vt, kv_len, v_transposed=True, n_splits=2, out_dtype=torch.float32)
    exp = orc.sdpa(qv.reshape(B, Hq, 1, D), kv[:, :, :kv_len], vv[:, :, :kv_len], enable_gqa=True).reshape(B, Hq, D)
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL


def test_injected_status_makes_the_machine_raise(dev):
    """A step whose bounded wait ran out leaves a code in the status word; `generate`, `read_tokens` and
    `set_state` must raise instead of returning its tokens. The code is written from the host."""
    from sanic_b200 import RunError, llama
    w = llama.random_weights(SMALL, 3, dev.torch_device)
    m = llama.LlamaMachine(dev, SMALL, w, ctx=64, batch=2)
    m.set_state([1, 2], 0)
    m.step()
    m.sync()                                            # clean
    for code, text in ((31, "bounded device-side wait"), (52, "cache extent"), (51, "gather index")):
        m.step()
        m.stream.synchronize()
        assert dev.lib.sanic_status_inject(dev.h, code) == 0
        with pytest.raises(RunError, match=text):
            m.read_tokens()
        m.read_tokens()                                 # the word was cleared by the failed sync
    assert dev.lib.sanic_status_inject(dev.h, 33) == 0
    with pytest.raises(RunError):
        m.generate(np.array([[1, 2], [3, 4]], dtype=np.int32), 2)


def test_machine_refuses_to_step_past_the_cache(dev):
    from sanic_b200 import RunError, llama
    w = llama.random_weights(SMALL, 4, dev.torch_device)
    for persistent in (False, True):
        m = llama.LlamaMachine(dev, SMALL, w, ctx=16, batch=1, persistent=persistent)
        m.set_state([5], 13)
        m.step(); m.step(); m.step()                    # positions 13, 14, 15: the last row of the cache
        with pytest.raises(RunError, match="outside the cache extent"):
            m.step()
        with pytest.raises(RunError, match="outside the cache extent"):
            m.step_stage_times()
        m.sync()                                        # nothing ran out of range, so nothing is reported
        assert int(m.position.item()) == 16


def test_splitkv_decoder_sync_raises_on_status(dev):
    from sanic_b200 import RunError
    from sanic_b200.splitkv import SplitKVDecoder
    k = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16, device=dev.torch_device)
    d = SplitKVDecoder(dev, k, k, n_splits=2, init_nccl=False)
    q = torch.zeros(1, 8, 128, dtype=torch.bfloat16, device=dev.torch_device)
    d.step(q)
    d.sync()
    d.step(q)
    assert dev.lib.sanic_status_inject(dev.h, 42) == 0
    with pytest.raises(RunError, match="code 42"):
        d.sync()


def test_peer_flag_that_never_arrives_times_out_and_returns(dev):
    """Two 'ranks' on one device, the second never runs: rank 0 stores its accumulators into both exchange
    buffers, publishes its flags, and waits for a flag nobody writes. With a short poll limit the wait gives up,
    the kernel returns, sanic_sync reports SANIC_ERR_TIMEOUT (code 41 + rank 1), and the next call works."""
    import time
    from sanic_b200 import RunError, abi
    lib = dev.lib
    B, Hq, Hkv, D, n = 1, 8, 2, 128, 512
    g = torch.Generator(device=dev.torch_device); g.manual_seed(77)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    rows = B * Hq
    nbytes = int(lib.sanic_peer_exchange_bytes(rows, D, 2))
    bufs = [torch.zeros(nbytes // 4 + 4, dtype=torch.float32, device=dev.torch_device) for _ in range(2)]
    carrier = dev.empty((rows, D + 2), torch.float32)
    out = torch.full((B, Hq, D), 7.0, dtype=torch.float32, device=dev.torch_device)
    p, _keep = dev.decode_params(q, k, v, n, n_splits=2, carrier_out=carrier, out=None)
    x = abi.PeerExchange()
    x.rank, x.nranks, x.epoch, x.spin_limit = 0, 2, 1, 1 << 12
    x.buffers[0], x.buffers[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
    t0 = time.time()
    dev._check(lib.sanic_splitkv_decode_step_peer(dev.h, C.byref(p), C.byref(x), C.c_void_p(out.data_ptr()), abi.F32, dev.stream()),
               "peer step")
    with pytest.raises(RunError, match="code 42"):
        dev.sync()
    assert time.time() - t0 < 5.0
    assert torch.all(out == 7.0)                        # the merge never ran: the output is untouched
    # rank 0's accumulators and flag did reach the other buffer
    flags = bufs[1][:32].view(torch.int32).cpu().numpy()
    assert flags[16] == 1 and flags[17] == 0   # parity 1 (epoch 1): slot of rank 0 set, slot of rank 1 never
    # the context still works: one rank alone completes
    x1 = abi.PeerExchange()
    x1.rank, x1.nranks, x1.epoch = 0, 1, 1
    buf1 = torch.zeros(int(lib.sanic_peer_exchange_bytes(rows, D, 1)) // 4 + 4, dtype=torch.float32, device=dev.torch_device)
    x1.buffers[0] = buf1.data_ptr()
    dev._check(lib.sanic_splitkv_decode_step_peer(dev.h, C.byref(p), C.byref(x1), C.c_void_p(out.data_ptr()), abi.F32, dev.stream()),
               "peer step")
    dev.sync()
    exp = orc.sdpa(q.float().cpu().numpy().astype(np.float64)[:, :, None, :], k.float().cpu().numpy().astype(np.float64),
                   v.float().cpu().numpy().astype(np.float64), enable_gqa=True)[:, :, 0, :]
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL


def test_fused_step_times_out_when_a_device_never_publishes(dev):
    """The one-launch multi-device step with two 'ranks' of which only rank 0 runs: its last arrivers store and flag
    every group into both buffers, then wait for rank 1's group flags, which nobody writes. The bounded wait gives up,
    the kernel returns, sanic_sync reports code 41 + 1, the output is untouched and the context keeps working."""
    import time
    from sanic_b200 import RunError, abi
    lib = dev.lib
    B, Hq, Hkv, D, n = 1, 8, 2, 128, 2048
    g = torch.Generator(device=dev.torch_device); g.manual_seed(78)
    q = torch.randn(B, Hq, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    k = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    v = torch.randn(B, Hkv, n, D, generator=g, device=dev.torch_device).to(torch.bfloat16)
    rows, groups = B * Hq, B * Hkv
    nbytes = int(lib.sanic_peer_exchange_bytes_fused(rows, D, 2, groups))
    bufs = [torch.zeros(nbytes // 4 + 4, dtype=torch.float32, device=dev.torch_device) for _ in range(2)]
    out = torch.full((B, Hq, D), 7.0, dtype=torch.float32, device=dev.torch_device)
    p, _keep = dev.decode_params(q, k, v, n, n_splits=dev.streamk_slots(B, Hkv, D), out=None)
    x = abi.PeerExchange()
    x.rank, x.nranks, x.epoch, x.spin_limit = 0, 2, 1, 1 << 12
    x.buffers[0], x.buffers[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
    t0 = time.time()
    dev._check(lib.sanic_splitkv_decode_step_fused(dev.h, C.byref(p), C.byref(x), C.c_void_p(out.data_ptr()), abi.F32, dev.stream()),
               "fused step")
    with pytest.raises(RunError, match="code 42"):
        dev.sync()
    assert time.time() - t0 < 5.0
    assert torch.all(out == 7.0)
    flags = bufs[1][:64].view(torch.int32).cpu().numpy()       # [2 parities][8 ranks][4 (groups padded)]
    assert list(flags[32:34]) == [1, 1] and list(flags[36:38]) == [0, 0]      # parity 1: rank 0's two groups set, rank 1's never
    x1 = abi.PeerExchange()
    x1.rank, x1.nranks, x1.epoch = 0, 1, 1
    buf1 = torch.zeros(int(lib.sanic_peer_exchange_bytes_fused(rows, D, 1, groups)) // 4 + 4, dtype=torch.float32, device=dev.torch_device)
    x1.buffers[0] = buf1.data_ptr()
    dev._check(lib.sanic_splitkv_decode_step_fused(dev.h, C.byref(p), C.byref(x1), C.c_void_p(out.data_ptr()), abi.F32, dev.stream()),
               "fused step")
    dev.sync()
    exp = orc.sdpa(q.float().cpu().numpy().astype(np.float64)[:, :, None, :], k.float().cpu().numpy().astype(np.float64),
                   v.float().cpu().numpy().astype(np.float64), enable_gqa=True)[:, :, 0, :]
    assert nerr(out.cpu().numpy(), exp) <= BF16_TOL
