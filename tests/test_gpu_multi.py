"""Two GPUs: KV-head sharding with a single NCCL all-gather of the attention outputs against the single-GPU
result, and sequences partitioned across ranks with no collective.  Skipped on a one-GPU box."""
import os
import socket

import numpy as np
import pytest

from util import TOL, normal, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _worker(rank, world, port, ok):
    import torch.distributed as dist

    import tract_b200 as kv
    from tract_b200 import sharding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        Hq, Hkv, D, lens = 32, 8, 128, [700, 65, 1300]
        layer = sharding.HeadShardedAttention("q8_1", Hq, Hkv, D, max_seqs=len(lens), max_seq_tokens=2048)
        full = kv.KvCache("q8_1", Hkv, D, max_seqs=len(lens), max_seq_tokens=2048)  # every rank also holds all heads
        s_sh, s_full = [layer.new_seq() for _ in lens], [full.new_seq() for _ in lens]
        for b, n in enumerate(lens):  # the same seeded K/V on every rank (replicated input)
            k = torch.from_numpy(normal(100 + b, (1, Hkv, n, D)).astype(np.float16)).cuda()
            v = torch.from_numpy(normal(200 + b, (1, Hkv, n, D)).astype(np.float16)).cuda()
            layer.append([s_sh[b]], k, v)
            full.append([s_full[b]], k, v)
        q = torch.from_numpy(normal(7, (len(lens), Hq, 1, D)).astype(np.float16)).cuda()
        out = layer.attend(s_sh, q, causal=True)
        want = full.attend(s_full, q, causal=True)
        good = rel_err(out.float().cpu().numpy(), want.float().cpu().numpy()) <= 1e-3
        # by sequence: each rank attends only over its own bin; together they cover the batch exactly once
        bins, _ = sharding.partition_sequences(lens, world)
        mine = bins[rank]
        if mine:
            part = full.attend([s_full[i] for i in mine], q[mine].contiguous(), causal=True)
            good &= rel_err(part.float().cpu().numpy(), want[mine].float().cpu().numpy()) <= 1e-3
        layer.cache.check(), full.check()
        ok[rank] = int(good)
    finally:
        dist.destroy_process_group()


def test_head_sharding_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ok = mp.get_context("spawn").Array("i", [0, 0])
    mp.spawn(_worker, args=(2, port, ok), nprocs=2, join=True)
    assert list(ok) == [1, 1]
