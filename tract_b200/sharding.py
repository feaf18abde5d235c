"""Multi-GPU use of the path: one process per GPU, sequences as the unit of partition.

tract itself has no multi-GPU support (its CUDA context is pinned to device 0, cuda/src/context.rs:65); every
(sequence, layer) KV cache is an independent state, so the natural partition is by sequence, with no traffic
between GPUs.  The second, optional axis is the KV head: rank r keeps kv heads [r * Hkv / N, (r + 1) * Hkv / N) and
the query heads that read them; append and attention stay local and the attention outputs are put together with
ONE all-gather along the head axis.  The attention kernel writes its output straight into this rank's slot of the
gather buffer, so the collective runs in place over NVLink with no staging copy.
"""
from __future__ import annotations


def partition_sequences(lens, world):
    """Longest-processing-time-first split of sequences (by cached length) into `world` bins.

    Returns (bins, imbalance): bins[r] = sorted indices of the sequences rank r owns; imbalance = max bin load /
    mean bin load.  Decode attention time is proportional to the cached tokens a rank streams."""
    if world <= 0:
        raise ValueError("world must be positive")
    bins = [[] for _ in range(world)]
    load = [0] * world
    for i in sorted(range(len(lens)), key=lambda i: (-lens[i], i)):
        r = min(range(world), key=lambda r: (load[r], r))
        bins[r].append(i)
        load[r] += lens[i]
    mean = sum(load) / world if world else 0
    return [sorted(b) for b in bins], (max(load) / mean if mean else 1.0)


def head_slice(n_heads, world, rank):
    """Heads [lo, hi) owned by `rank` when `n_heads` are split evenly."""
    if n_heads % world:
        raise ValueError(f"{n_heads} heads cannot be split evenly over {world} ranks")
    per = n_heads // world
    return rank * per, (rank + 1) * per


def gather_buffer(torch, world, batch, local_q_heads, n_new, head_dim, dtype, device):
    """[world, B, Hq/world, S, D]: slot r is what rank r's attention writes."""
    return torch.empty((world, batch, local_q_heads, n_new, head_dim), dtype=dtype, device=device)


def all_gather_heads(buffer, rank, group=None):
    """One all-gather over the slots of `buffer` (slot `rank` must already hold this rank's output); returns the
    full [B, Hq, S, D] tensor as a view of the buffer (head index = slot * Hq/world + local head)."""
    import torch.distributed as dist

    world = buffer.shape[0]
    if world > 1:
        mine = buffer[rank]
        if dist.get_backend(group) != "nccl":
            mine = mine.clone()  # only NCCL takes an input that aliases its slot of the output
        dist.all_gather_into_tensor(buffer.view(-1), mine.reshape(-1), group=group)
    w, b, h, s, d = buffer.shape
    return buffer.permute(1, 0, 2, 3, 4).reshape(b, w * h, s, d)


class HeadShardedAttention:
    """A layer's cache + attention with the kv heads split over the ranks of a process group."""

    def __init__(self, fmt, n_q_heads, n_kv_heads, head_dim, max_seqs, max_seq_tokens, group=None):
        import torch
        import torch.distributed as dist

        from . import KvCache

        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.kv_lo, self.kv_hi = head_slice(n_kv_heads, self.world, self.rank)
        self.q_lo, self.q_hi = head_slice(n_q_heads, self.world, self.rank)
        self.head_dim = head_dim
        self.cache = KvCache(fmt, self.kv_hi - self.kv_lo, head_dim, max_seqs, max_seq_tokens)
        self._torch = torch

    def new_seq(self):
        return self.cache.new_seq()

    def append(self, seqs, k_new, v_new):
        """k_new / v_new: the FULL [B, Hkv, S, D] tensors (replicated input); the local head slice is a strided view."""
        self.cache.append(seqs, k_new[:, self.kv_lo:self.kv_hi], v_new[:, self.kv_lo:self.kv_hi])

    def attend(self, seqs, q, causal=True, scale=None, buffer=None):
        """q: the FULL [B, Hq, S, D]; returns the full output on every rank.  `buffer`: a gather_buffer() to reuse from
        step to step (none is allocated then)."""
        b, _, s, d = q.shape
        buf = buffer if buffer is not None else gather_buffer(self._torch, self.world, b, self.q_hi - self.q_lo, s, d, q.dtype, q.device)
        self.cache.attend(seqs, q[:, self.q_lo:self.q_hi], scale=scale, causal=causal, out=buf[self.rank])
        return all_gather_heads(buf, self.rank, self.group)
