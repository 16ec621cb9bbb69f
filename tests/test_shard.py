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
