"""Token-balanced sharding of a jagged batch across GPUs.

Sequences are independent in both passes, so a batch splits by sequence with no exchange step:
each rank takes a contiguous range of sequences chosen on the prefix sum of token counts, slices
its rows out of Q / K / V, rebases its offsets to zero and runs the single-GPU operator unchanged.
The same planner cuts a batch that does not fit one GPU into shards that run one after another.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def plan_token_balanced_shards(q_lens: Sequence[int], kv_lens: Sequence[int], n_shards: int,
                               balance: str = "tokens") -> List[Tuple[int, int]]:
    """Contiguous sequence ranges ``[(start, end), ...]``, one per shard.

    ``balance="tokens"`` equalises ``sum(Lq + Lkv)`` per shard; ``balance="pairs"`` equalises
    ``sum(Lq * Lkv)`` (the contraction work).  Every sequence lands in exactly one shard; shards may
    be empty when there are fewer sequences than shards.
    """
    if n_shards <= 0:
        raise ValueError("n_shards must be positive")
    q = np.asarray(q_lens, dtype=np.int64)
    k = np.asarray(kv_lens, dtype=np.int64)
    if q.shape != k.shape or q.ndim != 1:
        raise ValueError("q_lens and kv_lens must be 1-D and of equal length")
    if (q < 0).any() or (k < 0).any():
        raise ValueError("negative sequence length")
    if balance == "tokens":
        cost = q + k
    elif balance == "pairs":
        cost = q * k
    else:
        raise ValueError(f"unknown balance mode {balance!r}")
    n = q.size
    csum = np.concatenate([[0], np.cumsum(cost)])
    total = int(csum[-1])
    bounds = [0]
    for r in range(1, n_shards):
        target = total * r / n_shards
        # first boundary whose prefix cost reaches the target, never moving backwards
        b = int(np.searchsorted(csum, target, side="left"))
        if b > 0 and abs(csum[b - 1] - target) <= abs(csum[min(b, n)] - target):
            b -= 1
        bounds.append(min(max(b, bounds[-1]), n))
    bounds.append(n)
    return [(bounds[i], bounds[i + 1]) for i in range(n_shards)]


def shard_jagged(offsets, start: int, end: int):
    """(row_start, row_end, rebased_offsets) of sequences ``[start, end)`` of a prefix-sum array
    (numpy array or torch tensor; the result has the same type)."""
    row_start = int(offsets[start])
    row_end = int(offsets[end])
    return row_start, row_end, offsets[start:end + 1] - row_start


def shard_inputs(q, k, v, q_offsets, kv_offsets, rank: int, world: int, balance: str = "tokens"):
    """Slice a jagged batch for one rank: returns ``(q_r, k_r, v_r, q_off_r, kv_off_r, (seq_start,
    seq_end), (q_row_start, q_row_end))`` with offsets rebased to zero.  Works on torch tensors on any
    device; the offsets are read on the host once (planning is host logic)."""
    qo = q_offsets.detach().cpu().numpy().astype(np.int64)
    ko = kv_offsets.detach().cpu().numpy().astype(np.int64)
    shards = plan_token_balanced_shards(np.diff(qo), np.diff(ko), world, balance)
    s, e = shards[rank]
    q0, q1 = int(qo[s]), int(qo[e])
    k0, k1 = int(ko[s]), int(ko[e])
    return (q[q0:q1], k[k0:k1], v[k0:k1], q_offsets[s:e + 1] - q0, kv_offsets[s:e + 1] - k0, (s, e), (q0, q1))


def gather_rows(local, group=None):
    """All-gather row-sharded tensors of different lengths (validation only; the hot path has no
    collective).  Returns the concatenation in rank order on every rank."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    n = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    counts = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(counts, n, group=group)
    counts = [int(c.item()) for c in counts]
    mx = max(counts) if counts else 0
    pad = torch.zeros((mx,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad, group=group)
    return torch.cat([b[:c] for b, c in zip(bufs, counts)], dim=0)


def max_over_ranks(value: float, device, group=None) -> float:
    """Maximum of a per-rank scalar (device-timed step duration) over the ranks."""
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
