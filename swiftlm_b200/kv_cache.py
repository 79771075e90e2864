"""Paged KV cache of one attention layer for the DFlash verify cycle.

The reference keeps one growing array per layer, appends the verify block's 16 rows during the
target forward and trims back to the accepted prefix afterwards
(Sources/DFlash/DFlashRuntime.swift:188-223).  Here the rows live in a page pool
[num_pages, Hkv, page_tokens, D] (the layout the verify attention reads), the committed length of
every sequence is a device array, and one cycle is

    lens = cache.append_block(k_new, v_new)      # rows land behind the committed tokens
    out  = cache.attend(q, scale)                # block-verify attention over committed + block
    cache.commit(replay_len)                     # keep accepted + 1 rows; the rest is overwritten next time

with no host read of the accepted count.  Pages are handed out on the host from an upper bound
of every sequence's length (committed length known at the last sync() plus the rows appended
since); sync() reads the true lengths once, tightens the bounds and returns pages that are no
longer reachable.  The verify attention reads whole 128-key tiles from one page, so attend() needs
page_tokens to be a multiple of 128 (256 in the benchmark configuration).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from . import kernels


class KVCacheFull(RuntimeError):
    """The pool has no free page left, or a sequence needs more pages than its table holds."""


class PagedKVCache:
    def __init__(self, batch: int, kv_heads: int, head_dim: int, page_tokens: int, num_pages: int, max_pages: int,
                 dtype: torch.dtype = torch.bfloat16, device="cuda", block: int = 16):
        self.B, self.Hkv, self.D = batch, kv_heads, head_dim
        self.page_tokens, self.num_pages, self.max_pages, self.block = page_tokens, num_pages, max_pages, block
        self.k_pool = torch.zeros(num_pages, kv_heads, page_tokens, head_dim, dtype=dtype, device=device)
        self.v_pool = torch.zeros_like(self.k_pool)
        # pageable on purpose: a copy from pageable memory snapshots the table when it is issued, so the host may go on
        # editing it while earlier work is still running on the stream
        self._table_host = torch.full((batch, max_pages), -1, dtype=torch.int32)
        self.page_table = self._table_host.to(device)
        self.kv_len = torch.zeros(batch, dtype=torch.int32, device=device)        # committed tokens per sequence
        self.kv_len_block = torch.zeros(batch, dtype=torch.int32, device=device)  # committed + the block just appended
        self._free: List[int] = list(range(num_pages - 1, -1, -1))                # pop() hands out page 0 first
        self._pages: List[List[int]] = [[] for _ in range(batch)]
        self._upper = [0] * batch            # host upper bound of kv_len
        self._dirty = False
        self._appended = 0

    # ---- host-side page bookkeeping ----
    @property
    def free_pages(self) -> int:
        return len(self._free)

    def pages_of(self, b: int) -> List[int]:
        return list(self._pages[b])

    def reserve(self, b: int, tokens: int) -> None:
        """Makes positions [0, tokens) of sequence b addressable."""
        need = -(-tokens // self.page_tokens)
        if need > self.max_pages:
            raise KVCacheFull(f"sequence {b} needs {need} pages, its table holds {self.max_pages}")
        while len(self._pages[b]) < need:
            if not self._free:
                raise KVCacheFull("page pool exhausted")
            page = self._free.pop()
            self._table_host[b, len(self._pages[b])] = page
            self._pages[b].append(page)
            self._dirty = True

    def _shrink(self, b: int, tokens: int) -> None:
        keep = -(-tokens // self.page_tokens)
        while len(self._pages[b]) > keep:
            page = self._pages[b].pop()
            self._table_host[b, len(self._pages[b])] = -1
            self._free.append(page)
            self._dirty = True

    def _flush_table(self) -> None:
        if self._dirty:
            self.page_table.copy_(self._table_host)
            self._dirty = False

    # ---- the verify cycle ----
    def append_block(self, k_new: torch.Tensor, v_new: torch.Tensor) -> torch.Tensor:
        """k_new, v_new [B,Hkv,T,D]: rows t = 0..T-1 of sequence b go to positions kv_len[b] + t.
        Returns the device array of lengths including the block (what attend() uses)."""
        T = k_new.shape[2]
        for b in range(self.B):
            self.reserve(b, self._upper[b] + T)
        self._flush_table()
        kernels.kv_append(k_new.contiguous(), v_new.contiguous(), self.k_pool, self.v_pool, kv_len=self.kv_len,
                          page_table=self.page_table, kv_len_out=self.kv_len_block)
        self._appended = T
        return self.kv_len_block

    def attend(self, queries: torch.Tensor, scale: float, mask: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Block-verify attention of queries [B,Hq,16,D] over the committed tokens and the block just appended."""
        n_max = min(max(self._upper) + self._appended, self.max_pages * self.page_tokens)
        return kernels.batched_sdpa_2pass(queries, self.k_pool, self.v_pool, scale, mask=mask, kv_len=self.kv_len_block,
                                          page_table=self.page_table, n_max=n_max)

    def commit(self, commit_count: torch.Tensor) -> None:
        """commit_count int32[B] on the device (replay_len of accept_lengths = accepted drafts + 1): the committed
        length grows by that many rows, at most by the block."""
        kernels.kv_commit(self.kv_len, commit_count, self._appended)
        for b in range(self.B):
            self._upper[b] += self._appended
        self._appended = 0

    def extend(self, k: torch.Tensor, v: torch.Tensor, lens) -> None:
        """Prefill: appends k, v [B,Hkv,T,D] and commits lens[b] <= T rows of sequence b."""
        lens_dev = torch.as_tensor(lens, dtype=torch.int32).to(self.kv_len.device)
        self.append_block(k, v)
        self.commit(lens_dev)

    def sync(self) -> np.ndarray:
        """Reads the committed lengths (one device-to-host copy), tightens the host bounds and returns the pages
        beyond every sequence's committed length to the pool."""
        lens = self.kv_len.cpu().numpy()
        for b in range(self.B):
            self._upper[b] = int(lens[b])
            self._shrink(b, self._upper[b])
        self._flush_table()
        return lens

    def release(self, b: int) -> None:
        """Forgets sequence b: its pages return to the pool, its length becomes 0."""
        self._shrink(b, 0)
        self._upper[b] = 0
        self.kv_len[b] = 0
        self._flush_table()

    # ---- inspection (tests) ----
    def gather(self, b: int, length: Optional[int] = None):
        """The first `length` rows of sequence b as dense [Hkv, length, D] tensors (k, v)."""
        n = int(self.kv_len[b].item()) if length is None else length
        idx = torch.arange(n, device=self.k_pool.device)
        pages = self.page_table[b, (idx // self.page_tokens).long()].long()
        slot = (idx % self.page_tokens).long()
        return self.k_pool[pages, :, slot].transpose(0, 1), self.v_pool[pages, :, slot].transpose(0, 1)
