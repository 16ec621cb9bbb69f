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
"""
from __future__ import annotations

from typing import Optional, Tuple

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
