"""Host-side logic of the multi-GPU path on CPU: the sequence partitioner, and the head all-gather under a
world_size-2 gloo group (the attention itself needs a GPU; here each rank fills its slot with known values)."""
import os
import socket

import numpy as np
import pytest

from tract_b200 import sharding


def test_partition_is_a_balanced_partition():
    g = np.random.default_rng(3)
    lens = [int(x) for x in g.integers(512, 16385, size=256)]  # config 3's length distribution
    for world in (1, 2, 4, 8):
        bins, imbalance = sharding.partition_sequences(lens, world)
        assert sorted(i for b in bins for i in b) == list(range(256))
        assert 1.0 <= imbalance < 1.01
    bins, imbalance = sharding.partition_sequences([10, 1], 4)  # fewer sequences than ranks
    assert [len(b) for b in bins] == [1, 1, 0, 0] and imbalance == pytest.approx(10 / (11 / 4))
    with pytest.raises(ValueError):
        sharding.head_slice(8, 3, 0)
    assert sharding.head_slice(8, 4, 3) == (6, 8)


def _worker(rank, world, port, ok):
    import torch
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, S, D = 3, 8, 2, 16
        full = torch.arange(B * Hq * S * D, dtype=torch.float32).reshape(B, Hq, S, D)
        lo, hi = sharding.head_slice(Hq, world, rank)
        buf = sharding.gather_buffer(torch, world, B, hi - lo, S, D, torch.float32, "cpu")
        buf.fill_(float("nan"))
        buf[rank].copy_(full[:, lo:hi])  # what this rank's attention kernel would have written
        out = sharding.all_gather_heads(buf, rank)
        ok[rank] = int(torch.equal(out, full))
        # by-sequence partition needs no collective at all: every rank derives the same bins locally
        bins, _ = sharding.partition_sequences([5, 9, 2, 7, 7, 1], world)
        mine = torch.tensor([sum(bins[rank])], dtype=torch.int64)
        dist.all_reduce(mine)
        ok[rank] &= int(mine.item() == sum(range(6)))
    finally:
        dist.destroy_process_group()


def test_head_all_gather_two_ranks_gloo():
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ok = mp.get_context("spawn").Array("i", [0, 0])
    mp.spawn(_worker, args=(2, port, ok), nprocs=2, join=True)
    assert list(ok) == [1, 1]
