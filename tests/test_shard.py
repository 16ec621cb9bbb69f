"""CPU tests of the (batch x head) sharding: partition arithmetic and a world_size-2
gloo run where each rank computes its shard (with the oracle standing in for the
kernels) and the gathered O equals the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deers_b200 import shard


def test_partition_covers_everything_once():
    for n in (1, 7, 8, 24, 2048):
        for w in (1, 2, 3, 4, 8):
            spans = [shard.partition(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and b0 <= e0
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_partition_cfg5_counts():
    # B=64, H=32 -> 2048 slices: 1024 / 512 / 256 per GPU at 2 / 4 / 8 GPUs.
    for w, per in ((2, 1024), (4, 512), (8, 256)):
        assert all(shard.partition(2048, w, r) == (r * per, (r + 1) * per) for r in range(w))
        assert shard.shard_shape(64, 32, w, 0) == (64 // w, 32)


def test_shard_shape_falls_back_to_flat():
    assert shard.shard_shape(3, 4, 8, 0) == (2, 1)
    with pytest.raises(ValueError):
        shard.partition(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_bh, result_dir):
    from oracle import ref
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, D = 20, 8
        rng = np.random.default_rng(0)                      # every rank draws the same full problem
        q, k, v = (rng.standard_normal((n_bh, 1, T, D)).astype(np.float32) for _ in range(3))
        full_o, _ = ref.attn_fwd(q, k, v)
        b, e = shard.partition(n_bh, world, rank)
        o_shard, _ = ref.attn_fwd(q[b:e], k[b:e], v[b:e])
        got = shard.gather_output(torch.from_numpy(o_shard), n_bh)
        assert got.shape == (n_bh, T, D)
        np.testing.assert_array_equal(got.numpy(), full_o[:, 0])
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_bh", [6, 5])      # equal shards and ragged shards
def test_two_rank_gloo_gather_matches_unsharded(tmp_path, n_bh):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), n_bh, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_partition_matches_the_c_abi():
    """deers_b200_shard_range (what a Rust host calls) and shard.partition agree."""
    import ctypes
    from deers_b200 import _lib
    L = _lib.lib()
    b, e = ctypes.c_int64(), ctypes.c_int64()
    for n in (0, 1, 5, 24, 2048, 2049):
        for w in (1, 2, 3, 8):
            for r in range(w):
                L.deers_b200_shard_range(n, w, r, ctypes.byref(b), ctypes.byref(e))
                assert (b.value, e.value) == shard.partition(n, w, r)
    L.deers_b200_shard_range(8, 2, 2, ctypes.byref(b), ctypes.byref(e))      # bad rank: empty range, no crash
    assert (b.value, e.value) == (0, 0)


def _leaver(rank, world, port, result_dir, announce):
    """Rank 1 runs one step and leaves between steps; rank 0 must get RankLeft at its next step, not hang."""
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    rv = shard.StepRendezvous(store, rank, world, timeout_s=3.0)
    rv.arrive(0)                                            # step 0: everyone is here
    if rank == 1:
        if announce:
            rv.leave()
        open(os.path.join(result_dir, "left1"), "w").close()
        os._exit(0)                                          # gone between steps, nothing in flight
    t0 = time.monotonic()
    try:
        rv.arrive(1)
    except shard.RankLeft as err:
        took = time.monotonic() - t0
        assert err.missing == [1] and err.step == 1
        assert took < (1.5 if announce else 10.0), took
        open(os.path.join(result_dir, "ok0"), "w").close()
    os._exit(0)                                              # no collective teardown with a dead peer


@pytest.mark.parametrize("announce", [True, False])
def test_rank_leaving_between_steps_raises_on_the_others(tmp_path, announce):
    world = 2
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, world, port, str(tmp_path), announce)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
        assert not p.is_alive(), "a rank hung"
    assert (tmp_path / "left1").exists() and (tmp_path / "ok0").exists()
