"""Work partitioning across the GPUs of one node.

The hot path has no exchange step: every (sequence, KV head) is independent in quantize-on-append and in
attention, and the query heads of a GQA group travel with their KV head.  So a job is sharded by KV head
(few long sequences) or by sequence (large ragged batches, balanced by cached tokens), each rank keeps its own
cache shard, and the only optional collective is an all-gather of the output slices.
"""
from __future__ import annotations

from typing import List, Sequence


def shard_kv_heads(num_kv_heads: int, world: int, rank: int) -> range:
    """Contiguous KV heads of ``rank``; needs num_kv_heads % world == 0 so that every rank does equal work."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads do not split evenly over {world} ranks")
    per = num_kv_heads // world
    return range(rank * per, (rank + 1) * per)


def query_heads_of(kv_heads: range, group: int) -> range:
    """Query heads that read the given KV heads (head h reads KV head h // group)."""
    return range(kv_heads.start * group, kv_heads.stop * group)


def shard_batch_by_tokens(seq_lens: Sequence[int], world: int) -> List[List[int]]:
    """Sequence indices per rank, balanced by total cached tokens (longest first onto the lightest rank);
    deterministic, ties go to the lower rank, indices within a rank ascending."""
    if world < 1:
        raise ValueError("world must be >= 1")
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(seq_lens)), key=lambda j: (-int(seq_lens[j]), j)):
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(seq_lens[i])
    return [sorted(x) for x in out]


def all_gather_heads(out_local, group=None):
    """All-gather of per-rank output slices (batch, heads_local, d) along the head axis (head sharding).
    Works on any torch.distributed backend (NCCL over NVLink on GPUs, gloo on CPU)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    parts = [torch.empty_like(out_local) for _ in range(world)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def all_gather_batch(out_local, counts: Sequence[int], index_lists: Sequence[Sequence[int]], group=None):
    """All-gather of per-rank (n_r, heads, d) outputs of a batch-sharded job back into batch order.
    ``counts[r]`` = sequences on rank r, ``index_lists[r]`` = their positions in the full batch."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    width = max(counts)
    pad = torch.zeros((width,) + tuple(out_local.shape[1:]), dtype=out_local.dtype, device=out_local.device)
    pad[: out_local.shape[0]] = out_local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    full = torch.zeros((sum(counts),) + tuple(out_local.shape[1:]), dtype=out_local.dtype, device=out_local.device)
    for r in range(world):
        if counts[r]:
            full[torch.as_tensor(list(index_lists[r]), device=full.device)] = parts[r][: counts[r]]
    return full
