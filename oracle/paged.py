"""Paged-cache oracle in numpy: slot arithmetic, append, gather and the block manager's bookkeeping.

No reference counterpart exists (the reference has no KV cache: README.md:316, :412, :424 name it as future
work), so this restates the contract of include/llaisys/paged_kv.h instead:
    pool[page][K|V][kvh][slot][d];  token pos of a sequence -> page table[pos // page_size], slot pos % page_size.
All movement is bit-exact: rows are copied as 16-bit / 32-bit words, never converted.
"""
from __future__ import annotations

import numpy as np


class PagedCacheModel:
    """One layer of a page pool plus the free-list block manager, in plain numpy / Python lists."""

    def __init__(self, num_pages: int, page_size: int, nkvh: int, d: int, word_dtype=np.uint16, max_seqs: int = 256,
                 max_pages_per_seq: int | None = None):
        self.num_pages, self.page_size, self.nkvh, self.d = num_pages, page_size, nkvh, d
        self.max_seqs = max_seqs
        self.max_pages_per_seq = max_pages_per_seq if max_pages_per_seq is not None else num_pages
        self.pool = np.zeros((num_pages, 2, nkvh, page_size, d), dtype=word_dtype)
        # Free pages as a stack whose top is handed out next; page 0 first, and pages a sequence frees come back
        # in reverse table order so that re-reserving pops them in their original order.
        self.free = list(range(num_pages - 1, -1, -1))
        self.free_ids = list(range(max_seqs - 1, -1, -1))
        self.tables: dict[int, list[int]] = {}

    # ---- block manager ----
    def add_seq(self) -> int:
        if not self.free_ids:
            raise KeyError("NO_SEQ")
        seq = self.free_ids.pop()
        self.tables[seq] = []
        return seq

    def reserve(self, seq: int, n_tokens: int) -> None:
        table = self.tables[seq]
        want = -(-n_tokens // self.page_size)
        extra = want - len(table)
        if extra <= 0:
            return
        if want > self.max_pages_per_seq:
            raise ValueError("INVALID")
        if extra > len(self.free):
            raise MemoryError("NO_PAGES")
        for _ in range(extra):
            table.append(self.free.pop())

    def assign_pages(self, seq: int, pages) -> None:
        table = self.tables[seq]
        pages = [int(p) for p in pages]
        if len(table) + len(pages) > self.max_pages_per_seq:
            raise ValueError("INVALID")
        free = set(self.free)
        if len(set(pages)) != len(pages) or any(p not in free for p in pages):
            if any(p < 0 or p >= self.num_pages for p in pages):
                raise ValueError("INVALID")
            raise MemoryError("NO_PAGES")
        taken = set(pages)
        self.free = [p for p in self.free if p not in taken]
        table.extend(pages)

    def free_seq(self, seq: int) -> None:
        table = self.tables.pop(seq)
        self.free.extend(reversed(table))
        self.free_ids.append(seq)

    # ---- data movement ----
    def slot(self, seq: int, pos: int) -> tuple[int, int]:
        return self.tables[seq][pos // self.page_size], pos % self.page_size

    def append(self, k_rows: np.ndarray, v_rows: np.ndarray, seq_ids, positions) -> None:
        """k_rows, v_rows: [n_rows, nkvh, d] words."""
        for i, (seq, pos) in enumerate(zip(seq_ids, positions)):
            page, slot = self.slot(int(seq), int(pos))
            self.pool[page, 0, :, slot, :] = k_rows[i]
            self.pool[page, 1, :, slot, :] = v_rows[i]

    def gather(self, seq: int, n_tokens: int) -> tuple[np.ndarray, np.ndarray]:
        k = np.empty((n_tokens, self.nkvh, self.d), dtype=self.pool.dtype)
        v = np.empty_like(k)
        for pos in range(n_tokens):
            page, slot = self.slot(seq, pos)
            k[pos] = self.pool[page, 0, :, slot, :]
            v[pos] = self.pool[page, 1, :, slot, :]
        return k, v
