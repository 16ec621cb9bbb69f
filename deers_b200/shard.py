"""(batch x head) sharding of the attention path over the GPUs of one box.

The (b, h) slices of ``[B, H, T, D]`` are independent in forward and backward
(src/models/gpt.rs:139-144 is batched over the two leading axes), so rank ``r`` of
``W`` owns a contiguous range of the flattened slice index and no data-path
collective is needed for the gradients.  The one exchange step is optional: an
all-gather of O for callers that need the full output on every rank; it runs on
a side stream so that it overlaps the backward of the same step.

One process per GPU; ``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the
CPU tests) is the plumbing.  The reference has no multi-device code at all
(``Device::Cuda`` carries no ordinal, src/device.rs:15-22).

``PeerGather`` is the product path of the all-gather: the C ABI's copy-engine pushes
(``deers_b200_allgather_o``), with ``torch.distributed`` used only to exchange the
buffer handles once.  ``gather_output`` / ``OverlappedGather`` (a library all-gather) stay
as the fallback for boxes where peer mappings cannot be opened.  ``StepRendezvous`` is the
host-side failure detection: ranks meet in the store before every step, so a rank that
left or died turns into an exception on the others instead of a hung collective.
"""
from __future__ import annotations

import ctypes
import datetime
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def partition(n_slices: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) range of flattened (b*H + h) slices owned by `rank`.

    The first ``n_slices % world`` ranks take one extra slice, so any count shards."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_slices, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_shape(B: int, H: int, world: int, rank: int) -> Tuple[int, int]:
    """Shape (B', H') of this rank's shard viewed as a [B', H', T, D] tensor."""
    begin, end = partition(B * H, world, rank)
    n = end - begin
    if n % H == 0 and begin % H == 0:
        return n // H, H            # whole batches: keep the head axis
    return n, 1


def gather_output(o_shard: torch.Tensor, n_slices: int, group=None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gathers the per-rank O shards ([n_r, T, D], slices flattened) into [n_slices, T, D].

    Equal shards use one all_gather_into_tensor (NCCL all-gather, in place in `out`);
    ragged shards fall back to all_gather over padded buffers."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T, D = o_shard.shape[-2:]
    o_shard = o_shard.reshape(-1, T, D)
    if out is None:
        out = torch.empty((n_slices, T, D), dtype=o_shard.dtype, device=o_shard.device)
    if n_slices % world == 0:
        dist.all_gather_into_tensor(out, o_shard.contiguous(), group=group)
        return out
    width = -(-n_slices // world)
    padded = torch.zeros((width, T, D), dtype=o_shard.dtype, device=o_shard.device)
    padded[: o_shard.shape[0]] = o_shard
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    for r in range(world):
        b, e = partition(n_slices, world, r)
        out[b:e] = parts[r][: e - b]
    return out


class OverlappedGather:
    """Issues the O all-gather on a side CUDA stream so that it overlaps the backward.

    ``start(o_shard)`` is called right after the forward was enqueued; ``finish()``
    makes the compute stream wait for the gather (call it after the backward)."""

    def __init__(self, n_slices: int, T: int, D: int, dtype, device, group=None):
        self.n_slices, self.group = n_slices, group
        self.out = torch.empty((n_slices, T, D), dtype=dtype, device=device)
        self.stream = torch.cuda.Stream(device=device)
        self.done = torch.cuda.Event()

    def start(self, o_shard: torch.Tensor) -> None:
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            gather_output(o_shard, self.n_slices, self.group, out=self.out)
            self.done.record(self.stream)

    def finish(self) -> torch.Tensor:
        torch.cuda.current_stream().wait_event(self.done)
        return self.out


class PeerGather:
    """All-gather of O by device-to-device pushes into every peer's buffer (``deers_b200_allgather_o``).

    Every rank allocates the full ``[n_slices, T, D]`` buffer ``out``; the forward writes this rank's slices
    straight into ``local()`` (no staging copy), ``start()`` pushes them to the peers on the copy engines while
    the backward runs, ``join()`` orders the compute stream after the pushes.  The gathered tensor is complete
    on a rank once every peer has finished its pushes: ``flush()`` + a barrier (``wait_all``)."""

    def __init__(self, n_slices: int, T: int, D: int, dtype, device, ctx, group=None):
        from . import _lib
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.ctx = ctx
        self.out = torch.empty((n_slices, T, D), dtype=dtype, device=device)
        self.begin, self.end = partition(n_slices, self.world, self.rank)
        self.slice_bytes = T * D * self.out.element_size()
        L = _lib.lib()
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        _lib.check(L.deers_b200_comm_export(ctx.handle, self.out.data_ptr(), handle), ctx.handle)
        everyone = [None] * self.world                       # any backend: the handles are 72 opaque bytes each
        dist.all_gather_object(everyone, bytes(handle.raw), group=group)
        blob = b"".join(everyone)
        self.handle = ctypes.c_void_p()
        _lib.check(L.deers_b200_comm_init_ipc(ctx.handle, self.rank, self.world, self.out.data_ptr(),
                                              self.out.numel() * self.out.element_size(), blob,
                                              ctypes.byref(self.handle)), ctx.handle)

    def local(self) -> torch.Tensor:
        """This rank's slices of the gather buffer: hand it to the forward as its output."""
        return self.out[self.begin:self.end]

    def start(self, first: int = 0, count: Optional[int] = None) -> None:
        """Pushes `count` of this rank's slices starting at its `first`-th to every peer (default: all)."""
        from . import _lib
        n = self.end - self.begin
        count = n - first if count is None else count
        _lib.check(_lib.lib().deers_b200_allgather_o(self.handle, (self.begin + first) * self.slice_bytes,
                                                     count * self.slice_bytes), self.ctx.handle)

    def set_lanes(self, lanes: int) -> None:
        """How many of the world - 1 pushes of a `start()` are in flight at once (default: one)."""
        from . import _lib
        _lib.check(_lib.lib().deers_b200_comm_set_lanes(self.handle, int(lanes)), self.ctx.handle)

    def join(self) -> None:
        from . import _lib
        _lib.check(_lib.lib().deers_b200_allgather_join(self.handle), self.ctx.handle)

    def flush(self) -> None:
        from . import _lib
        _lib.check(_lib.lib().deers_b200_allgather_flush(self.handle), self.ctx.handle)

    def wait_all(self) -> torch.Tensor:
        """Blocks until every rank's pushes have landed everywhere; returns the gathered O."""
        self.flush()
        dist.barrier(group=self.group)
        return self.out

    def close(self) -> None:
        from . import _lib
        if self.handle:
            _lib.lib().deers_b200_comm_destroy(self.handle)
            self.handle = None


class RankLeft(RuntimeError):
    """A rank did not show up for a step (it left, crashed, or is stuck)."""

    def __init__(self, step: int, missing: List[int], why: str):
        super().__init__(f"step {step}: rank(s) {missing} {why}")
        self.step, self.missing = step, missing


class StepRendezvous:
    """Host-side failure detection between steps.  Before launching step k every rank calls ``arrive(k)``: it
    posts a key in the store and waits, with a time limit, for the keys of all the others.  A rank that leaves
    calls ``leave()`` (between steps, with none of its kernels or copies in flight); the others then get
    ``RankLeft`` at their next ``arrive`` at once, and after `timeout_s` if the rank vanished without a word.
    Nothing here touches a GPU: a missing peer becomes an exception before any copy towards it is enqueued."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "deers_b200/step"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, step: int, rank: int) -> str:
        return f"{self.prefix}/{step}/{rank}"

    def leave(self) -> None:
        self.store.set(f"{self.prefix}/left/{self.rank}", "1")

    def arrive(self, step: int) -> None:
        self.store.set(self._key(step, self.rank), "1")
        others = [r for r in range(self.world) if r != self.rank]
        deadline = datetime.datetime.now() + datetime.timedelta(seconds=self.timeout_s)
        pending = list(others)
        while pending:
            gone = [r for r in pending if self.store.check([f"{self.prefix}/left/{r}"])]
            if gone:
                raise RankLeft(step, gone, "announced that they left")
            pending = [r for r in pending if not self.store.check([self._key(step, r)])]
            if not pending:
                break
            if datetime.datetime.now() > deadline:
                raise RankLeft(step, pending, f"did not arrive within {self.timeout_s:g} s")
            try:
                self.store.wait([self._key(step, pending[0])], datetime.timedelta(milliseconds=50))
            except Exception:                                # timeout of the short wait: look at the flags again
                pass
