"""Sharding of the attention work across GPUs of one node.

A (batch b, KV head hkv) group needs only K,V[b,hkv] and Q,O,dO,LSE[b, hkv*G .. hkv*G+G-1] and produces
dK,dV[b,hkv] and dQ (or O, LSE) of its G query heads (head map ``hkv = hq // G``,
src/attention/GQA_bwd_baseline.cu:415; precision/baseline_gqa.py:51).  Groups are therefore independent:
rank r owns the contiguous group range ``group_range(r, world, B*Hkv)`` and runs the unmodified
single-GPU operators on it; there is no data-path collective.  With the ``[B, H, S, D]`` layout a group
range is one contiguous slab of every tensor, so a shard is a zero-copy view that is itself a valid
GQA problem with ``B' = groups, Hkv' = 1, Hq' = G``.

``gather_groups`` (torch.distributed all_gather) reassembles outputs for verification only.
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch


def group_range(rank: int, world: int, n_groups: int) -> Tuple[int, int]:
    """Contiguous range [begin, end) of groups owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(n_groups, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def as_groups(t: torch.Tensor, Hkv: int) -> torch.Tensor:
    """View ``[B, H, ...]`` as ``[B*Hkv, H/Hkv, ...]`` (no copy); H is Hq or Hkv."""
    B, H = t.shape[:2]
    if H % Hkv:
        raise ValueError(f"{H} heads do not divide into {Hkv} KV heads")
    return t.reshape(B * Hkv, H // Hkv, *t.shape[2:])


def shard(t: torch.Tensor, Hkv: int, rank: int, world: int) -> torch.Tensor:
    """This rank's slab of `t` as a ``[groups, H/Hkv, ...]`` view."""
    g = as_groups(t, Hkv)
    begin, end = group_range(rank, world, g.shape[0])
    return g[begin:end]


def run_sharded(fn: Callable[..., Sequence[torch.Tensor]], tensors: Sequence[torch.Tensor], Hkv: int,
                rank: int, world: int) -> Sequence[torch.Tensor]:
    """Apply `fn` (forward or backward over a GQA problem) to this rank's shard of `tensors`.

    An empty shard (more ranks than groups) returns empty outputs without calling `fn`."""
    parts = [shard(t, Hkv, rank, world) for t in tensors]
    if parts[0].shape[0] == 0:
        return None
    return fn(*parts)


def gather_groups(local: torch.Tensor, n_groups: int, rank: int, world: int, group=None) -> torch.Tensor:
    """All-gather per-rank ``[groups_r, ...]`` outputs into ``[n_groups, ...]`` (verification only).

    Ranks may own different numbers of groups: shards are padded to the largest one for the collective."""
    import torch.distributed as dist

    sizes = [group_range(r, world, n_groups) for r in range(world)]
    most = max(e - b for b, e in sizes)
    tail = local.shape[1:] if local is not None else None
    if tail is None:
        raise ValueError("gather_groups needs the local tensor (possibly with zero groups)")
    padded = local.new_zeros((most, *tail))
    padded[: local.shape[0]] = local
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded, group=group)
    return torch.cat([o[: e - b] for o, (b, e) in zip(out, sizes)], dim=0)
