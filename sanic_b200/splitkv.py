"""Sequence-sharded split-KV decode across ranks.

The key axis is cut into `world` contiguous slices exactly as run_carrier_split chunks it
(reference src/interp.rs:603: chunk b = [b*n/B, (b+1)*n/B)). Each rank folds its slice to one raw
(m, l, o) accumulator per (batch, query head); the accumulators are all-gathered and merged left
to right in rank order with the derived combine, then projected. The exchange is
(2 + D) * 4 bytes per (batch, head) per rank: latency-bound, not bandwidth-bound.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _abi as abi


def shard_range(n: int, rank: int, world: int):
    """[lo, hi) of rank's slice; every slice is non-empty when world <= n (src/interp.rs:570-574)."""
    if not (1 <= world <= n):
        raise ValueError(f"world must be in [1, extent = {n}]")
    return rank * n // world, (rank + 1) * n // world


def exchange_and_merge(local_carrier, merge_fn, group=None):
    """All-gather [rows, 2+D] accumulators over `group` and merge them in rank order.

    `merge_fn(parts[world, rows, 2+D])` applies the derived combine and projects. Works on any
    backend torch.distributed offers; the GPU path below uses NCCL from inside the C library.
    """
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_carrier) for _ in range(world)]
    dist.all_gather(parts, local_carrier, group=group)
    return merge_fn(torch.stack(parts))


class SplitKVDecoder:
    """One rank of a sequence-sharded decode. `k`, `v` are this rank's slices [B, Hkv, n_local, D] bf16."""

    def __init__(self, dev, k, v, n_splits=None, init_nccl=True):
        self.dev, self.k, self.v = dev, k, v
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        B, Hkv, n_local, D = k.shape
        self.n_local = n_local
        self.n_splits = n_splits or dev.suggest_splits(B, Hkv, D, n_local)
        if self.world > 1 and init_nccl:
            ident = torch.zeros(128, dtype=torch.uint8)
            if self.rank == 0:
                buf = (C.c_uint8 * 128)()
                rc = dev.lib.sanic_nccl_unique_id(buf)
                if rc != abi.OK:
                    raise RuntimeError("sanic_nccl_unique_id failed: libnccl.so.2 is not loaded in this process")
                ident = torch.tensor(list(buf), dtype=torch.uint8)
            ident = ident.to(dev.torch_device)
            dist.broadcast(ident, src=0)
            arr = (C.c_uint8 * 128)(*ident.cpu().tolist())
            dev._check(dev.lib.sanic_nccl_init(dev.h, self.rank, self.world, arr), "nccl_init")
        self._bufs = None

    def _buffers(self, B, Hq, D):
        if self._bufs is None:
            td = self.dev.torch_device
            self._bufs = dict(carrier=torch.empty((B * Hq, D + 2), dtype=torch.float32, device=td),
                              gathered=torch.empty((self.world, B * Hq, D + 2), dtype=torch.float32, device=td),
                              out=torch.empty((B, Hq, D), dtype=torch.bfloat16, device=td))
        return self._bufs

    def step(self, q, scale=None):
        """q [B, Hq, D] bf16 (replicated on every rank) -> attention output [B, Hq, D] bf16 on every rank."""
        B, Hq, D = q.shape
        b = self._buffers(B, Hq, D)
        p, _keep = self.dev.decode_params(q, self.k, self.v, self.n_local, n_splits=self.n_splits, scale=scale,
                                          carrier_out=b["carrier"], out=None)
        rc = self.dev.lib.sanic_splitkv_decode_step(self.dev.h, C.byref(p), C.c_void_p(b["gathered"].data_ptr()),
                                                    C.c_void_p(b["out"].data_ptr()), abi.BF16, self.dev.stream())
        self.dev._check(rc, "splitkv_decode_step")
        return b["out"]
