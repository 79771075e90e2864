"""CPU tests of the host-side mirror: rollback-cache indexing contract (integer, exact),
partition plans, and the N > 1 path over gloo with two CPU ranks."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dflash_oracle as O
from swiftlm_b200 import partition
from swiftlm_b200.rollback_cache import RecurrentRollbackCache, restore_after_acceptance


def test_arm_record_clear_and_full_accept_shortcut():
    c = RecurrentRollbackCache()
    assert not c.is_armed
    c.state = [torch.zeros(1, 3, 4), torch.ones(1, 2, 8, 8)]
    c.arm_rollback(prefix_len=7)
    assert c.is_armed and c._snapshot[1] is c.state[1]          # snapshot by reference, no copy
    c.state[1] = torch.full((1, 2, 8, 8), 5.0)                  # the verify pass moved the state on
    c.record_tape(torch.zeros(1, 16, 2, 8), torch.zeros(1, 16, 1, 8), torch.zeros(1, 16, 2), torch.zeros(1, 16, 4))
    restore_after_acceptance([c], target_len=10, acceptance_length=15, drafted_tokens=15)
    assert not c.is_armed and c._tape is None and float(c.state[1][0, 0, 0, 0]) == 5.0   # kept the verify state
    c.offset = 20
    assert c.trim(6) == 6 and c.offset == 14 and c.trim(100) == 14 and c.offset == 0
    # rollback without a snapshot only clears
    c.rollback(3)
    assert not c.is_armed


def test_partition_helpers():
    assert partition.plan(64, 8) == [(8 * i, 8 * i + 8) for i in range(8)]
    assert partition.sequences_for_rank(10, 3, 4) == (8, 10)
    pairs = [partition.kv_pairs_for_rank(8, 2, r, 8) for r in range(8)]
    assert pairs[0] == [(0, 0), (0, 1)] and pairs[7] == [(7, 0), (7, 1)]
    assert sorted(sum(pairs, [])) == [(s, h) for s in range(8) for h in range(2)]
    odd = [partition.kv_pairs_for_rank(5, 2, r, 4) for r in range(4)]
    assert [len(x) for x in odd] == [3, 3, 2, 2] and len(set(sum(odd, []))) == 10


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, n_seq, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = partition.sequences_for_rank(n_seq, rank, world)
    # each rank "verifies" its own sequences: acceptance from the CPU oracle on seeded tokens
    rng = np.random.default_rng(99)
    post = rng.integers(0, 50, (n_seq, 16)).astype(np.int32)
    ids = np.concatenate([rng.integers(0, 50, (n_seq, 1)), post[:, :-1]], axis=1).astype(np.int32)
    for b in range(n_seq):
        cut = rng.integers(0, 16)
        if cut < 15:
            ids[b, cut + 1] = (ids[b, cut + 1] + 1) % 50
    acc_local, nxt_local = [], []
    for b in range(lo, hi):
        a, _, staged = O.accept_block(ids[b], post[b])
        acc_local.append(a)
        nxt_local.append(staged)
    acc, nxt = partition.all_gather_acceptance(torch.tensor(acc_local, dtype=torch.int32),
                                               torch.tensor(nxt_local, dtype=torch.int32), n_seq)
    want = [O.accept_block(ids[b], post[b]) for b in range(n_seq)]
    assert acc.tolist() == [w[0] for w in want] and nxt.tolist() == [w[2] for w in want]
    # with the logits rows: every rank ends up with each sequence's logits row at its accepted position
    V = 50
    logits = np.random.default_rng(7).standard_normal((n_seq, 16, V)).astype(np.float32)
    rows_local = torch.from_numpy(np.stack([logits[b, acc_local[b - lo]] for b in range(lo, hi)]).reshape(hi - lo, V))
    acc2, nxt2, rows = partition.all_gather_acceptance(torch.tensor(acc_local, dtype=torch.int32),
                                                       torch.tensor(nxt_local, dtype=torch.int32), n_seq,
                                                       logits_rows_local=rows_local)
    assert torch.equal(acc2, acc) and torch.equal(nxt2, nxt) and rows.shape == (n_seq, V)
    np.testing.assert_array_equal(rows.numpy(), np.stack([logits[b, want[b][0]] for b in range(n_seq)]))
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()


@pytest.mark.parametrize("n_seq", [64, 7])
def test_sequence_sharded_step_with_gloo_all_gather(tmp_path, n_seq):
    world = 2
    port = _free_port()
    mp.spawn(_gloo_worker, args=(world, port, n_seq, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))


def test_paged_kv_cache_page_bookkeeping_on_the_host():
    """Page hand-out, table rows and return of unreachable pages (no kernel runs: CPU tensors)."""
    from swiftlm_b200.kv_cache import KVCacheFull, PagedKVCache
    c = PagedKVCache(2, 1, 8, 16, num_pages=5, max_pages=3, device="cpu")
    c.reserve(0, 17)
    c.reserve(1, 48)
    assert c.pages_of(0) == [0, 1] and c.pages_of(1) == [2, 3, 4] and c.free_pages == 0
    with pytest.raises(KVCacheFull):
        c.reserve(0, 49)                       # a fourth page does not fit the table
    with pytest.raises(KVCacheFull):
        c.reserve(0, 33)                       # a third page would, but the pool is empty
    c._shrink(1, 16)
    assert c.pages_of(1) == [2] and c.free_pages == 2
    assert c._table_host.tolist() == [[0, 1, -1], [2, -1, -1]]
    c.reserve(0, 48)
    assert len(c.pages_of(0)) == 3 and c.free_pages == 1
    assert len({*c.pages_of(0), *c.pages_of(1)}) == 4


def test_oracle_trimmable_cache_follows_the_restore_rule():
    from oracle import dflash_oracle as O
    ref = O.TrimmableKVCache(2, 1, 4)
    blk = np.arange(2 * 1 * 16 * 4, dtype=np.float32).reshape(2, 1, 16, 4)
    ref.update(blk, -blk)
    ref.restore([0, 0], [5, 16])               # targetLen = start + accepted inputs
    assert ref.offset(0) == 5 and ref.offset(1) == 16
    ref.update(blk, -blk)
    ref.restore([5, 16], [1, 9])
    assert ref.offset(0) == 6 and ref.offset(1) == 25
    np.testing.assert_array_equal(ref.k[0][0, 5], blk[0, 0, 0])       # the new block starts right behind the kept prefix
    np.testing.assert_array_equal(ref.v[1][0, 24], -blk[1, 0, 8])


def test_chunk_schedule_covers_the_batch():
    from swiftlm_b200.host_api import _chunk_schedule
    for B, chunk in ((2304, 144), (100, 144), (576, 144), (7, 3), (1, 1), (33, 8)):
        r = _chunk_schedule(B, chunk)
        assert r[0][0] == 0 and r[-1][1] == B and all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(0 < hi - lo <= chunk for lo, hi in r)
