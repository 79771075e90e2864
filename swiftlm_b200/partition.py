"""Work partitioning over the GPUs of one box, and the one collective of the end-to-end step.

Both kernels shard without any exchange on the data path: the replay by sequence (a GPU owns
every layer and head of its sequences, states never move), the verify attention by
(sequence, KV head) pair.  The only collectives are all-gathers after the step: the per-sequence
acceptance results and one logits row per sequence (the row at the accepted position).
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


def all_gather_acceptance(accept_local, next_local, n_sequences: int, group=None, logits_rows_local=None):
    """All-gather of the results of a sequence-sharded step.  accept_local and next_local are int32 tensors holding
    this rank's contiguous range of plan(n_sequences, world); returns (accept [n_sequences], next_token
    [n_sequences]) on every rank.  With logits_rows_local [n_local, V] (the verify-logits row at each sequence's
    accepted position, kernels.gather_logits_rows) a second all-gather returns those rows as [n_sequences, V] too:
    the posterior row is what a consumer on another rank needs beyond the token itself (sampling with a temperature,
    log-probabilities), at V values per sequence instead of the block's T x V.  Ranges may differ in length by one,
    so shards are padded to the longest range for the collectives (one all_gather_into_tensor each)."""
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
    if logits_rows_local is None:
        return acc, nxt
    V = logits_rows_local.shape[1]
    if n == longest:
        lsend = logits_rows_local.contiguous()
    else:
        lsend = torch.zeros(longest, V, dtype=logits_rows_local.dtype, device=logits_rows_local.device)
        lsend[:n] = logits_rows_local
    lrecv = torch.empty(world, longest, V, dtype=lsend.dtype, device=lsend.device)
    dist.all_gather_into_tensor(lrecv.view(-1), lsend.view(-1), group=group)
    if all(e - b == longest for b, e in ranges):
        rows = lrecv.view(world * longest, V)
    else:
        rows = torch.cat([lrecv[r, :e - b] for r, (b, e) in enumerate(ranges)])
    return acc, nxt, rows
