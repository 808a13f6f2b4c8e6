"""The multi-rank split-KV host logic on CPU: two gloo ranks shard the key axis exactly as
run_carrier_split chunks it (reference src/interp.rs:603), fold their slices to raw (m, l, o)
accumulators (the oracle stands in for the device fold), exchange them with the package's
all-gather helper and merge in rank order with the derived combine. The result must equal the
unsharded evaluation. Also covers a rank whose slice is entirely masked (identity partial)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc
from sanic_b200.splitkv import exchange_and_merge, shard_range


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, masked_tail, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv, D, L = 2, 4, 2, 8, 37
        rng = orc.Xorshift(0x5EED)
        q, k, v = rng.normal(B, Hq, 1, D), rng.normal(B, Hkv, L, D), rng.normal(B, Hkv, L, D)
        mask = np.zeros((1, L))
        if masked_tail:                      # everything the last rank owns is hidden
            lo_last, _ = shard_range(L, world - 1, world)
            mask[:, lo_last:] = -np.inf
        lo, hi = shard_range(L, rank, world)
        _, car = orc.sdpa_carrier_split(q, k[:, :, lo:hi], v[:, :, lo:hi], 1, mask=mask[:, lo:hi], enable_gqa=True,
                                        return_carriers=True)
        local = torch.tensor(car.reshape(B * Hq, D + 2))
        out = exchange_and_merge(local, lambda parts: torch.tensor(orc.carrier_merge_mlo(parts.numpy())))
        full = orc.sdpa(q, k, v, mask=mask, enable_gqa=True).reshape(B * Hq, D)
        err = float(np.max(np.abs(out.numpy() - full)))
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("masked_tail", [False, True])
def test_two_rank_shard_exchange_merge(masked_tail):
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, masked_tail, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert len(ret) == world and all(e < 1e-12 for e in ret.values()), dict(ret)


def _withheld_worker(rank, world, port, ret):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from sanic_b200.backend import RunError
    if rank == 1:
        ret[rank] = "left"          # this rank leaves between steps without joining the exchange
        return
    local = torch.zeros(4, 10, dtype=torch.float64)
    try:
        exchange_and_merge(local, lambda parts: parts.sum(0))
        ret[rank] = "completed"
    except RunError as e:
        ret[rank] = "RunError" if "did not take part" in str(e) else f"other: {e}"


def test_exchange_with_a_rank_that_never_joins_raises_instead_of_hanging():
    # failure made on the host: rank 1 never takes part; rank 0's collective ends with the process group's timeout and
    # the helper turns that into a RunError (the step has no output)
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_withheld_worker, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        if p.is_alive():
            p.kill()
    assert ret.get(1) == "left" and ret.get(0) == "RunError", dict(ret)


def test_shard_range_is_the_reference_chunking():
    n = 1048576
    for world in (1, 2, 4, 8, 3, 7):
        edges = [shard_range(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert all(hi > lo for lo, hi in edges)
        assert edges == [(r * n // world, (r + 1) * n // world) for r in range(world)]
    with pytest.raises(ValueError):
        shard_range(3, 0, 4)      # blocks may not exceed the extent (src/interp.rs:570-574)
