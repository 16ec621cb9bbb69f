"""Multi-GPU tests of the C ABI's sharding entry points: need two GPUs in one box (skipped otherwise).
The all-gather of O is device-to-device copies only; no kernel reads a peer's memory."""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _two_gpus():
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_single_process_comm_init_all_gathers_byte_ranges():
    """deers_b200_comm_init_all: one process, one context per GPU; every rank pushes its byte range."""
    from deers_b200 import _lib
    L = _lib.lib()
    n, nbytes = min(torch.cuda.device_count(), 4), 1 << 20
    ctxs, bufs = [], []
    for g in range(n):
        h = ctypes.c_void_p()
        _lib.check(L.deers_b200_init(g, None, ctypes.byref(h)))
        ctxs.append(h)
        with torch.cuda.device(g):
            bufs.append(torch.zeros(nbytes, dtype=torch.uint8, device=f"cuda:{g}"))
    for g in range(n):
        torch.cuda.synchronize(g)
    comms = (ctypes.c_void_p * n)()
    _lib.check(L.deers_b200_comm_init_all(n, (ctypes.c_void_p * n)(*[c.value for c in ctxs]),
                                          (ctypes.c_void_p * n)(*[b.data_ptr() for b in bufs]), nbytes, comms), ctxs[0])
    half = nbytes // n
    for g in range(n):
        bufs[g][g * half:(g + 1) * half] = g + 1            # each rank fills only its own range
        torch.cuda.synchronize(g)
    for g in range(n):
        if g % 2:
            _lib.check(L.deers_b200_comm_set_lanes(comms[g], n), ctxs[g])      # clamped to n - 1: all pushes at once
        _lib.check(L.deers_b200_allgather_o(comms[g], g * half, half), ctxs[g])
    for g in range(n):
        _lib.check(L.deers_b200_allgather_flush(comms[g]), ctxs[g])
    want = torch.cat([torch.full((half,), g + 1, dtype=torch.uint8) for g in range(n)])
    for g in range(n):
        assert torch.equal(bufs[g].cpu(), want), f"rank {g}"
    assert L.deers_b200_allgather_o(comms[0], nbytes, 16) != 0, "a range beyond the buffer is refused"
    for g in range(n):
        L.deers_b200_comm_destroy(comms[g])
        L.deers_b200_destroy(ctxs[g])


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from deers_b200 import ops, shard
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)      # plumbing only: handles and barriers
    try:
        B, H, T, D = 2, 3, 384, 128
        g = torch.Generator(device="cpu").manual_seed(5)                # every rank draws the same full problem
        q, k, v = (torch.randn(B * H, 1, T, D, generator=g).to(dev, torch.float16) for _ in range(3))
        scale = ops.default_scale(D)
        full_o, _ = ops.attention_fwd(q, k, v, scale, True)              # unsharded, on this rank's GPU
        ctx = ops.Context.current(dev)
        gather = shard.PeerGather(B * H, T, D, torch.float16, dev, ctx)
        b, e = shard.partition(B * H, world, rank)
        ops.attention_fwd(q[b:e], k[b:e], v[b:e], scale, True, out=gather.local().view(e - b, 1, T, D))
        gather.start()
        gather.join()
        got = gather.wait_all()
        torch.cuda.synchronize()
        assert torch.equal(got, full_o.view(B * H, T, D)), "gathered O must equal the unsharded O bit for bit"
        # a second round with other values: the buffers and mappings are reused; this time with every push in
        # flight at once instead of one after the other
        gather.set_lanes(world - 1)
        gather.local().fill_(float(rank + 1))
        gather.start()
        got = gather.wait_all()
        torch.cuda.synchronize()
        for r in range(world):
            rb, re_ = shard.partition(B * H, world, r)
            assert (got[rb:re_] == float(r + 1)).all()
        dist.barrier()
        gather.close()
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_two_process_peer_gather_equals_unsharded_forward(tmp_path):
    """One process per GPU: handles exchanged over the process group, O pushed by the copy engines."""
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)                # more than two ranks exercise the push rotation
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
