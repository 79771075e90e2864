"""Work partitioning over the GPUs of one box, and the one collective of the end-to-end step.

Both kernels shard without any exchange on the data path: the replay by sequence (a GPU owns
every layer and head of its sequences, states never move), the verify attention by
(sequence, KV head) pair.  The only collective is an all-gather of the per-sequence acceptance
results (and, for the caller that wants them, logits slices) after the step.
The reference is single-device; there is nothing to cite.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Tuple

from . import _lib


def plan(units: int, n_gpus: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) ranges, sizes differing by at most one (dflash_partition_plan)."""
    arr = (C.c_int32 * (2 * n_gpus))()
    _lib.check(_lib.lib().dflash_partition_plan(units, n_gpus, arr))
    return [(arr[2 * i], arr[2 * i + 1]) for i in range(n_gpus)]


def sequences_for_rank(n_sequences: int, rank: int, world: int) -> Tuple[int, int]:
    return plan(n_sequences, world)[rank]


def kv_pairs_for_rank(n_sequences: int, n_kv_heads: int, rank: int, world: int) -> List[Tuple[int, int]]:
    """The (sequence, KV head) pairs owned by `rank`: pair p = sequence * n_kv_heads + kv head."""
    lo, hi = plan(n_sequences * n_kv_heads, world)[rank]
    return [(p // n_kv_heads, p % n_kv_heads) for p in range(lo, hi)]


def all_gather_acceptance(accept_local, next_local, n_sequences: int, group=None):
    """All-gather of the acceptance results of a sequence-sharded step.  accept_local and
    next_local are int32 tensors holding this rank's contiguous range of plan(n_sequences, world);
    returns (accept [n_sequences], next_token [n_sequences]) on every rank.  Ranges may differ in
    length by one, so shards are padded to the longest range for the collective."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    ranges = plan(n_sequences, world)
    longest = max(e - b for b, e in ranges)
    send = torch.zeros(2, longest, dtype=torch.int32, device=accept_local.device)
    n = accept_local.numel()
    send[0, :n] = accept_local
    send[1, :n] = next_local
    recv = torch.empty(world, 2, longest, dtype=torch.int32, device=accept_local.device)
    dist.all_gather_into_tensor(recv.view(-1), send.view(-1), group=group)
    acc = torch.cat([recv[r, 0, :e - b] for r, (b, e) in enumerate(ranges)])
    nxt = torch.cat([recv[r, 1, :e - b] for r, (b, e) in enumerate(ranges)])
    return acc, nxt
