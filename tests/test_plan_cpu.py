"""Planning facts and the device-level split, on the host: fitted specs, the split's legality rule, the chunking, and the
pricing that decides how many devices a fold's streamed axis is cut over (reference src/cost.rs:33-119,
src/plan.rs:434-488, src/interp.rs:597-606)."""
import pytest

from sanic_b200 import _abi as abi
from sanic_b200 import backend, plan


def test_fitted_specs_are_a_b200():
    s = plan.fitted_specs()
    assert s.sm_count == 148 and s.compute_dtype == abi.F32 and s.boundary_dtype == abi.BF16
    assert 6.0e12 < s.hbm_bandwidth < 8.0e12 and s.hbm_read_bandwidth >= s.hbm_bandwidth
    assert 1.0e15 < s.peak_flops < 2.5e15
    assert 1e-6 < s.launch_overhead < 1e-5 and 1e-6 < s.mem_latency_s < 1e-5
    # Little's law: the bytes that must be in flight to saturate HBM are what 296 CTAs with two 32 KB tiles each hold
    assert s.hbm_read_bandwidth * s.mem_latency_s == pytest.approx(s.min_blocks * 2 * 32768, rel=0.1)


def test_every_known_slot_kind_splits_out_of_order():
    assert plan.mergeable_out_of_order(backend.carrier_online_softmax())
    assert plan.mergeable_out_of_order(backend.carrier_deferred_norm())
    assert plan.mergeable_out_of_order(backend.carrier_contraction(abi.I4))
    assert plan.mergeable_out_of_order(backend.carrier_extremum_index())
    assert not plan.mergeable_out_of_order(backend.make_carrier([abi.SLOT_PLAIN_ADD, 99]))      # an unknown kind never splits


def test_shard_range_is_the_split_law_chunking():
    for n, parts in ((10, 3), (1 << 20, 8), (7, 7), (1000, 1)):
        ranges = [plan.shard_range(n, r, parts) for r in range(parts)]
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        assert all(hi > lo for lo, hi in ranges)                  # blocks <= extent keeps every part non-empty
        assert ranges == [(r * n // parts, (r + 1) * n // parts) for r in range(parts)]
    with pytest.raises(ValueError):
        plan.shard_range(3, 0, 4)                                  # more parts than elements (src/interp.rs:570-574)
    with pytest.raises(ValueError):
        plan.shard_range(8, 8, 8)


def test_long_context_decode_is_cut_over_the_devices_and_short_context_is_not():
    c = backend.carrier_online_softmax()
    # config 5: 4 x 32 query heads, 8 kv heads, head_dim 128, 2^20 keys: 32 streams, 2 * 128 * 2 bytes per key per stream
    B, Hq, Hkv, D, L = 4, 32, 8, 128, 1 << 20
    args = dict(points=B * Hq, streams=B * Hkv, stream_extent=L, bytes_per_step=B * Hkv * 2 * D * 2,
                flops_per_step=B * Hq * 4 * D, carrier_floats_per_point=D + 2)
    one = plan.plan_fold(c, max_devices=1, **args)
    assert one.devices == 1 and one.seconds == pytest.approx(2.45e-3, rel=0.1)          # measured: 2.43-2.55 ms
    eight = plan.plan_fold(c, max_devices=8, **args)
    assert eight.devices == 8 and eight.exchange_seconds > 3e-5
    assert eight.seconds == pytest.approx(0.36e-3, rel=0.15)                             # measured: 0.360 ms
    assert one.seconds / eight.seconds > 6.0
    # the decode step's attention at a 1024-key cache: 2 MB per layer; an exchange costs more than the whole fold
    small = plan.plan_fold(c, points=32, streams=8, stream_extent=1024, bytes_per_step=8 * 2 * 64 * 2, flops_per_step=32 * 4 * 64,
                           carrier_floats_per_point=66, max_devices=8)
    assert small.devices == 1
    # a carrier that does not merge out of order is never split across devices
    opaque = backend.make_carrier([99])
    assert plan.plan_fold(opaque, max_devices=8, **args).devices == 1
    with pytest.raises(ValueError):
        plan.plan_fold(c, max_devices=0, **args)
