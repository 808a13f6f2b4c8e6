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
    """[lo, hi) of rank's slice; every slice is non-empty when world <= n (src/interp.rs:570-574). The device-level
    chunking is the library's (sanic_shard_range), the same one every other level of the split uses."""
    from .plan import shard_range as _lib_range
    if not (1 <= world <= n):
        raise ValueError(f"world must be in [1, extent = {n}]")
    return _lib_range(n, rank, world)


def exchange_and_merge(local_carrier, merge_fn, group=None):
    """All-gather [rows, 2+D] accumulators over `group` and merge them in rank order.

    `merge_fn(parts[world, rows, 2+D])` applies the derived combine and projects. Works on any
    backend torch.distributed offers; the GPU path below uses NCCL from inside the C library.
    """
    from .backend import RunError
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local_carrier) for _ in range(world)]
    try:
        dist.all_gather(parts, local_carrier, group=group)
    except (RuntimeError, dist.DistBackendError) as e:
        # a rank that never joined (it raised, exited, or was never started) ends the collective with the process
        # group's timeout: the step's output does not exist, and the caller must not continue on it
        raise RunError(f"carrier exchange failed: a rank did not take part within the process group's timeout ({e})") from e
    return merge_fn(torch.stack(parts))


class SplitKVDecoder:
    """One rank of a sequence-sharded decode. `k`, `v` are this rank's slices [B, Hkv, n_local, D] bf16."""

    def __init__(self, dev, k, v, n_splits=None, init_nccl=True, exchange="nccl", force_exchange=False):
        """`exchange`: "nccl" (all-gather, then a merge kernel), "peer" (a second kernel stores the accumulators into
        every peer's buffer over NVLink, waits for the others' flags and merges) or "fused" (the whole step is one
        launch: the stream-K fold whose last arrivers store, flag, wait and merge per (batch, kv head) group)."""
        self.dev, self.k, self.v = dev, k, v
        self.exchange = exchange
        self.force_exchange = force_exchange      # run the exchange path even with one rank (tests)
        self.epoch = 0
        self._peer = None
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        B, Hkv, n_local, D = k.shape
        self.n_local = n_local
        self.n_splits = n_splits or dev.suggest_splits(B, Hkv, D, n_local)
        if exchange == "fused":
            self.n_splits = dev.streamk_slots(B, Hkv, D)
        if self.world > 1 and init_nccl and exchange == "nccl":
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

    def _peer_setup(self, rows, D, groups=0):
        """Allocate this rank's exchange buffer, trade IPC handles over torch.distributed, map the peers' buffers.

        Every rank takes the same collective calls whether or not its own part succeeded; the ranks then agree
        on the outcome, so a rank that cannot export or map raises on all of them instead of leaving the others
        waiting."""
        lib, dev = self.dev.lib, self.dev
        ok, why = 1, ""
        local = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        try:
            nbytes = int(lib.sanic_peer_exchange_bytes_fused(rows, D, self.world, groups) if groups
                         else lib.sanic_peer_exchange_bytes(rows, D, self.world))
            dev._check(lib.sanic_alloc(dev.h, nbytes, C.byref(local)), "alloc")
            dev._check(lib.sanic_memset(dev.h, local, 0, nbytes, dev.stream()), "memset")
            dev.sync()
            dev._check(lib.sanic_ipc_export(dev.h, local, handle), "ipc_export")
        except Exception as e:      # noqa: BLE001 - reported below, on every rank
            ok, why = 0, str(e)
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev.torch_device)
        theirs = [torch.empty_like(mine) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(theirs, mine)
        x = abi.PeerExchange()
        x.rank, x.nranks = self.rank, self.world
        opened = []
        if ok:
            try:
                for r in range(self.world):
                    if r == self.rank:
                        x.buffers[r] = local.value
                        continue
                    h = (C.c_uint8 * 64)(*theirs[r].cpu().tolist())
                    ptr = C.c_void_p()
                    dev._check(lib.sanic_ipc_open(dev.h, h, C.byref(ptr)), "ipc_open")
                    x.buffers[r] = ptr.value
                    opened.append(ptr)
            except Exception as e:  # noqa: BLE001
                ok, why = 0, str(e)
        if self.world > 1:
            agreed = torch.tensor([ok], dtype=torch.int32, device=dev.torch_device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)      # also the barrier: every buffer is zero-filled and mapped
            all_ok = int(agreed.item())
        else:
            all_ok = ok
        if not all_ok:
            for ptr in opened:
                lib.sanic_ipc_close(dev.h, ptr)
            if local.value:
                lib.sanic_free(dev.h, local)
            raise RuntimeError("peer exchange set-up failed" + (f": {why}" if why else " on another rank"))
        self._peer = dict(x=x, local=local, opened=opened)

    def close(self):
        if self._peer is not None:
            self.dev.sync()
            if self.world > 1:
                dist.barrier()      # nobody is still storing into a buffer that is about to go away
            for ptr in self._peer["opened"]:
                self.dev.lib.sanic_ipc_close(self.dev.h, ptr)
            self.dev.lib.sanic_free(self.dev.h, self._peer["local"])
            self._peer = None

    def sync(self, timeout_s: float = 0.0):
        """Wait for the steps in flight on the current stream and raise RunError if a peer's flag never arrived
        (status codes 41 + rank) or any other bounded wait ran out. The tensor `step` returned is valid only after
        this returns. With the NCCL exchange and `timeout_s` > 0 the wait is bounded on the host as well: the
        communicator's asynchronous error state is polled, and when the deadline passes with the collective still in
        flight (a rank that never joined) the communicator is aborted and RunError raised."""
        if timeout_s > 0.0 and self.exchange == "nccl" and self.world > 1:
            rc = self.dev.lib.sanic_nccl_wait(self.dev.h, self.dev.stream(), int(timeout_s * 1000))
            self.dev._check(rc, "nccl_wait")
            return
        self.dev.sync()

    def step(self, q, scale=None):
        """q [B, Hq, D] bf16 (replicated on every rank) -> attention output [B, Hq, D] bf16 on every rank.
        Asynchronous: call sync() before reading the result."""
        B, Hq, D = q.shape
        b = self._buffers(B, Hq, D)
        p, _keep = self.dev.decode_params(q, self.k, self.v, self.n_local, n_splits=self.n_splits, scale=scale,
                                          carrier_out=b["carrier"], out=None)
        if self.exchange == "fused" and self.world == 1 and not self.force_exchange:
            # one device: nothing to exchange, the stream-K fold projects straight into the output
            p.out, p.out_dtype, p.carrier_out = b["out"].data_ptr(), abi.BF16, None
            self.dev._check(self.dev.lib.sanic_attn_decode_streamk(self.dev.h, C.byref(p), self.dev.stream()), "attn_decode_streamk")
            return b["out"]
        if self.exchange == "fused":
            if self._peer is None:
                self._peer_setup(B * Hq, D, groups=B * self.k.shape[1])
            self.epoch += 1
            x = self._peer["x"]
            x.epoch = self.epoch
            p.carrier_out = None
            rc = self.dev.lib.sanic_splitkv_decode_step_fused(self.dev.h, C.byref(p), C.byref(x), C.c_void_p(b["out"].data_ptr()),
                                                          abi.BF16, self.dev.stream())
            self.dev._check(rc, "splitkv_decode_step_fused")
            return b["out"]
        if self.exchange == "peer":
            if self._peer is None:
                self._peer_setup(B * Hq, D)
            self.epoch += 1
            x = self._peer["x"]
            x.epoch = self.epoch
            rc = self.dev.lib.sanic_splitkv_decode_step_peer(self.dev.h, C.byref(p), C.byref(x), C.c_void_p(b["out"].data_ptr()),
                                                         abi.BF16, self.dev.stream())
            self.dev._check(rc, "splitkv_decode_step_peer")
            return b["out"]
        rc = self.dev.lib.sanic_splitkv_decode_step(self.dev.h, C.byref(p), C.c_void_p(b["gathered"].data_ptr()),
                                                    C.c_void_p(b["out"].data_ptr()), abi.BF16, self.dev.stream())
        self.dev._check(rc, "splitkv_decode_step")
        return b["out"]
