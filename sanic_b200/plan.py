"""Planning facts and the device-level split over the C ABI: the fitted `DeviceSpecs::b200()`, `mergeable_out_of_order`,
the device-level factor of `FoldSched` priced with the roofline plus an exchange latency, and measured tuning of the
decode fold's schedule candidates (reference src/cost.rs:33-119, src/plan.rs:434-488, src/compile.rs:1348-1630)."""
from __future__ import annotations

import ctypes as C

from . import _abi as abi


def fitted_specs() -> abi.FittedSpecs:
    s = abi.FittedSpecs()
    assert abi.load().sanic_specs_b200(C.byref(s)) == abi.OK
    return s


def measure_specs(dev) -> abi.FittedSpecs:
    s = abi.FittedSpecs()
    dev._check(dev.lib.sanic_specs_measure(dev.h, dev.stream(), C.byref(s)), "specs_measure")
    return s


def mergeable_out_of_order(carrier) -> bool:
    return bool(abi.load().sanic_mergeable_out_of_order(C.byref(carrier)))


def shard_range(extent: int, part: int, parts: int):
    lo, hi = C.c_int64(0), C.c_int64(0)
    if abi.load().sanic_shard_range(extent, part, parts, C.byref(lo), C.byref(hi)) != abi.OK:
        raise ValueError(f"parts must be in [1, extent = {extent}] and part in [0, parts)")
    return lo.value, hi.value


def plan_fold(carrier, points, streams, stream_extent, bytes_per_step, flops_per_step, carrier_floats_per_point, max_devices,
              specs=None) -> abi.FoldPlan:
    specs = specs or fitted_specs()
    out = abi.FoldPlan()
    rc = abi.load().sanic_plan_fold(C.byref(specs), C.byref(carrier), points, streams, stream_extent, float(bytes_per_step),
                                    float(flops_per_step), carrier_floats_per_point, max_devices, C.byref(out))
    if rc != abi.OK:
        raise ValueError("plan_fold: bad arguments")
    return out


def tune_decode(dev, params, candidates, repeats=3):
    """Times the decode fold's candidates on the caller's buffers; returns (best candidate, [seconds per candidate])."""
    arr = (C.c_int32 * len(candidates))(*candidates)
    best = C.c_int32(-1)
    secs = (C.c_double * len(candidates))()
    dev._check(dev.lib.sanic_tune_decode(dev.h, C.byref(params), arr, len(candidates), repeats, dev.stream(), C.byref(best), secs),
               "tune_decode")
    return candidates[best.value], list(secs)
