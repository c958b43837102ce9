"""A pool of cache pages with reference counts, a free list and prefix hashes.

Policy as in the reference's block manager (jllm/engine/paged.py:58-148): the free list
is doubly linked; `alloc` takes its head (the page freed longest ago); `release` puts
pages whose count falls to zero at the tail, a request's pages in reverse order, so the
last pages of a sequence are used again before its first ones and shared prefixes live
longest.  A free page keeps its content and its hash until it is given out again, so a
later request with the same prefix can take it back (`touch`).  Unlike the reference no
page is set aside as a sink: kernels never read or write beyond a request's length.
"""

from __future__ import annotations

import hashlib
import struct
from typing import Iterable, Optional


class OutOfPages(MemoryError):
    pass


def chain_hash(parent: bytes, token_ids: Iterable[int]) -> bytes:
    """Hash of a full page: sha256(parent hash | tokens as little-endian uint32); the first
    page's parent is b"" (jllm/engine/paged.py:41-46)."""
    h = hashlib.sha256()
    h.update(parent)
    h.update(struct.pack(f"<{len(token_ids)}I", *[int(t) for t in token_ids]))
    return h.digest()


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self.ref = [0] * num_pages
        self.hash_of: list[Optional[bytes]] = [None] * num_pages
        self.page_of_hash: dict[bytes, int] = {}
        # free list over all pages, ascending
        self.prev = [i - 1 for i in range(num_pages)]
        self.next = [i + 1 if i + 1 < num_pages else -1 for i in range(num_pages)]
        self.head, self.tail = 0, num_pages - 1
        self.in_free = [True] * num_pages
        self.num_free = num_pages

    # ------------------------------------------------------------------ free list
    def _unlink(self, p: int) -> None:
        a, b = self.prev[p], self.next[p]
        if a >= 0: self.next[a] = b
        else: self.head = b
        if b >= 0: self.prev[b] = a
        else: self.tail = a
        self.prev[p] = self.next[p] = -1
        self.in_free[p] = False
        self.num_free -= 1

    def _append(self, p: int) -> None:
        self.prev[p], self.next[p] = self.tail, -1
        if self.tail >= 0: self.next[self.tail] = p
        else: self.head = p
        self.tail = p
        self.in_free[p] = True
        self.num_free += 1

    # ------------------------------------------------------------------------ use
    def alloc(self) -> int:
        """A page for new content: the head of the free list; its old hash is dropped."""
        p = self.head
        if p < 0:
            raise OutOfPages("no free pages")
        self._unlink(p)
        h = self.hash_of[p]
        if h is not None:
            if self.page_of_hash.get(h) == p:
                del self.page_of_hash[h]
            self.hash_of[p] = None
        self.ref[p] = 1
        return p

    def touch(self, p: int) -> None:
        """One more holder of page p (taking it off the free list if it had none)."""
        if self.ref[p] == 0:
            if not self.in_free[p]:
                raise RuntimeError(f"page {p} has no holder and is not free")
            self._unlink(p)
        self.ref[p] += 1

    def release(self, pages: Iterable[int]) -> None:
        """One holder fewer for each page, last page first."""
        for p in reversed(list(pages)):
            if p < 0:
                continue
            if self.ref[p] <= 0:
                raise RuntimeError(f"page {p} released more often than held")
            self.ref[p] -= 1
            if self.ref[p] == 0:
                self._append(p)

    # --------------------------------------------------------------------- hashes
    def register(self, p: int, h: bytes) -> None:
        """Records that page p holds the content hashed h; the first page to claim a hash
        keeps it, and a page keeps its first hash (jllm/engine/paged.py:137-144)."""
        if self.hash_of[p] is not None or h in self.page_of_hash:
            return
        self.page_of_hash[h] = p
        self.hash_of[p] = h

    def lookup(self, h: bytes) -> Optional[int]:
        return self.page_of_hash.get(h)

    # --------------------------------------------------------------------- checks
    def free_pages(self) -> list[int]:
        out, p = [], self.head
        while p >= 0:
            out.append(p)
            p = self.next[p]
        return out

    def check(self) -> None:
        """Internal consistency: every page is either held or on the free list, never both."""
        free = self.free_pages()
        assert len(free) == len(set(free)) == self.num_free, "free list is inconsistent"
        for p in range(self.num_pages):
            assert (self.ref[p] == 0) == (p in set(free)) == self.in_free[p], f"page {p}: ref/free mismatch"
            assert self.ref[p] >= 0
        for h, p in self.page_of_hash.items():
            assert self.hash_of[p] == h
