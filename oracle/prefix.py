"""Oracle for the prefix-sharing block manager: the bookkeeping of include/llaisys/paged_kv.h's publish / match /
fork calls in plain Python, with prefixes kept as token tuples instead of hash chains.

No reference counterpart exists (the reference asks for "a KV-Cache pool with prefix matching", README.md:412 and :424,
and has none), so this restates the header's contract: pages are reference-counted; full pages are published under the
tokens they hold; a released published page stays findable until the pool needs it; the page released longest ago is
evicted first; plain free pages are used before cached ones. Page numbers are part of the contract being checked, so the
allocation order mirrors the library's: a stack of free pages (page 0 first; a freed sequence's pages come back in
reverse table order). TEST INFRASTRUCTURE ONLY (see oracle/__init__.py)."""
from __future__ import annotations

from collections import OrderedDict


class PrefixPoolModel:
    def __init__(self, num_pages: int, page_size: int, max_seqs: int, max_pages_per_seq: int):
        self.num_pages, self.page_size = num_pages, page_size
        self.max_pages_per_seq = max_pages_per_seq
        self.free = list(range(num_pages - 1, -1, -1))
        self.free_ids = list(range(max_seqs - 1, -1, -1))
        self.ref = [0] * num_pages
        self.key_of: dict[int, tuple] = {}       # published page -> the whole token prefix it ends
        self.page_of: dict[tuple, int] = {}      # token prefix -> page
        self.cached: OrderedDict[int, None] = OrderedDict()  # ref 0 and published, oldest first
        self.tables: dict[int, list[int]] = {}

    def num_free(self) -> int:
        return len(self.free) + len(self.cached)

    def _unpublish(self, page: int) -> None:
        key = self.key_of.pop(page, None)
        if key is not None:
            del self.page_of[key]
        if page in self.cached:
            del self.cached[page]
            if self.ref[page] == 0:
                self.free.append(page)

    def _take(self) -> int:
        if self.free:
            return self.free.pop()
        if not self.cached:
            raise MemoryError("NO_PAGES")
        page = next(iter(self.cached))
        self._unpublish(page)
        return self.free.pop()

    def _release(self, page: int) -> None:
        self.ref[page] -= 1
        if self.ref[page] > 0:
            return
        if page in self.key_of:
            self.cached[page] = None
        else:
            self.free.append(page)

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
        if extra > self.num_free():
            raise MemoryError("NO_PAGES")
        for _ in range(extra):
            page = self._take()
            self.ref[page] = 1
            table.append(page)

    def free_seq(self, seq: int) -> None:
        for page in reversed(self.tables.pop(seq)):
            self._release(page)
        self.free_ids.append(seq)

    def publish(self, seq: int, tokens) -> None:
        table = self.tables[seq]
        if len(tokens) > len(table) * self.page_size:
            raise ValueError("INVALID")
        for i in range(len(tokens) // self.page_size):
            key = tuple(tokens[: (i + 1) * self.page_size])
            page = table[i]
            if page not in self.key_of and key not in self.page_of:
                self.key_of[page] = key
                self.page_of[key] = page

    def match(self, seq: int, tokens) -> int:
        table = self.tables[seq]
        if table:
            raise ValueError("INVALID")
        full = min(len(tokens) // self.page_size, self.max_pages_per_seq)
        for i in range(full):
            page = self.page_of.get(tuple(tokens[: (i + 1) * self.page_size]))
            if page is None:
                break
            if self.ref[page] == 0:
                del self.cached[page]
            self.ref[page] += 1
            table.append(page)
        return len(table) * self.page_size

    def fork(self, parent: int, n_tokens: int):
        """-> (child, (src_page, dst_page) of the copied partial page or None)"""
        ptable = self.tables[parent]
        if n_tokens > len(ptable) * self.page_size:
            raise ValueError("INVALID")
        full, rest = divmod(n_tokens, self.page_size)
        if rest and self.num_free() < 1:
            raise MemoryError("NO_PAGES")
        child = self.add_seq()
        table = self.tables[child]
        for page in ptable[:full]:
            self.ref[page] += 1
            table.append(page)
        copied = None
        if rest:
            dst = self._take()
            self.ref[dst] = 1
            table.append(dst)
            copied = (ptable[full], dst)
        return child, copied
