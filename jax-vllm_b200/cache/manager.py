"""The cache manager: which pages and which state slot each live request holds.

Layers are put into groups by what they need: all layers with the same `PagedKVNeed`
(kv heads, head size, window) share one group, with one pool of pages and one block
table per request; a page id of a group addresses the same page in every layer of the
group.  Layers with a `FixedStateNeed` get a row per state slot instead.  Pages are given
back when a request ends, when it is preempted, and - in a group with a window - as soon
as every position of a page lies before the window of the next query.

Prefix reuse (jllm/engine/cache.py:20-57): full pages are hashed in a chain over the
tokens; a new request takes the longest run of pages whose hashes are known, in every
group, but always leaves at least its last token to compute.  A group with a window needs
only the pages that the window of the next query still reaches: the hit is the longest
prefix whose pages are known from the start in every group without a window and over the
last `window` positions in every group with one; the pages before that are entered as
given back, as they would be had the request computed the prefix itself.  Reuse is
switched off for models with fixed-size state, which a page hit does not restore.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..parts.base import FixedStateNeed, PagedKVNeed, PagedLayerCache, StateLayerCache
from .page_pool import OutOfPages, PagePool, chain_hash
from .state_slots import StateSlots


@dataclass
class CacheGroup:
    need: PagedKVNeed
    layers: list
    pool: PagePool
    k: Optional[torch.Tensor] = None     # [layers, num_pages, page_size, kv_heads, head_dim]
    v: Optional[torch.Tensor] = None

    def bytes_per_page(self, page_size: int, itemsize: int) -> int:
        return 2 * len(self.layers) * page_size * self.need.num_kv_heads * self.need.head_dim * itemsize


class PageTable:
    """Page ids of one request in one group by logical page index (-1: given back): a list of ints
    kept as a growing int32 array, so that a batch copies a row of a block table without
    converting it number by number (a request of 32k tokens has 2k pages, in every step)."""

    __slots__ = ("_a", "_n")

    def __init__(self):
        self._a = np.empty(16, dtype=np.int32)
        self._n = 0

    def append(self, page: int) -> None:
        if self._n == self._a.size:
            grown = np.empty(2 * self._a.size, dtype=np.int32)
            grown[:self._n] = self._a[:self._n]
            self._a = grown
        self._a[self._n] = page
        self._n += 1

    def array(self, n=None) -> np.ndarray:
        """The first `n` entries (all by default) as a view of the array; not to be kept over an append."""
        return self._a[:self._n if n is None else n]

    def __len__(self):
        return self._n

    def __getitem__(self, i):
        if isinstance(i, slice):
            return self._a[:self._n][i].tolist()
        if not -self._n <= i < self._n:
            raise IndexError(i)
        return int(self._a[i % self._n])

    def __setitem__(self, i, page):
        if not 0 <= i < self._n:
            raise IndexError(i)
        self._a[i] = page

    def __iter__(self):
        return iter(self._a[:self._n].tolist())

    def __eq__(self, other):
        return list(self) == list(other)

    def __repr__(self):
        return f"PageTable({list(self)})"


@dataclass
class RequestCache:
    """What one live request holds."""
    request_id: object
    slot: int
    tables: list                          # per group: a PageTable
    num_tokens: int = 0                   # tokens whose keys and values are in the cache
    hashes: list = field(default_factory=list)   # hash chain of the full pages so far
    freed_upto: list = field(default_factory=list)  # per group: logical pages below this were given back
    tokens: list = field(default_factory=list)   # token ids in the cache (kept only with prefix reuse)


class CacheManager:
    def __init__(self, needs: list, page_size: int, num_pages: int, max_live: int, prefix_cache: bool = True):
        self.page_size, self.num_pages, self.max_live = page_size, num_pages, max_live
        self.groups: list[CacheGroup] = []
        self.layer_group: dict[int, int] = {}
        self.state_layers: dict[int, FixedStateNeed] = {}
        for layer, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, FixedStateNeed):
                self.state_layers[layer] = need
            elif isinstance(need, PagedKVNeed):
                for g, grp in enumerate(self.groups):
                    if grp.need == need:
                        grp.layers.append(layer)
                        self.layer_group[layer] = g
                        break
                else:
                    self.layer_group[layer] = len(self.groups)
                    self.groups.append(CacheGroup(need, [layer], PagePool(num_pages)))
            else:
                raise TypeError(f"layer {layer}: unknown cache need {need!r}")
        self.slots = StateSlots(max_live)
        self.prefix_cache = bool(prefix_cache) and not self.state_layers
        self.live: dict[object, RequestCache] = {}
        self.stats = {"prefix_hit_pages": 0, "prefix_hit_tokens": 0, "pages_allocated": 0, "pages_released": 0}

    # ------------------------------------------------------------------- storage
    def allocate_storage(self, dtype: torch.dtype, device) -> dict:
        """Allocates pages and state rows on `device`; returns the cache view of every layer
        that has a need (layer index -> PagedLayerCache | StateLayerCache)."""
        views = {}
        for g, grp in enumerate(self.groups):
            shape = (len(grp.layers), self.num_pages, self.page_size, grp.need.num_kv_heads, grp.need.head_dim)
            grp.k = torch.zeros(shape, dtype=dtype, device=device)
            grp.v = torch.zeros(shape, dtype=dtype, device=device)
            for i, layer in enumerate(grp.layers):
                views[layer] = PagedLayerCache(group=g, k=grp.k[i], v=grp.v[i])
        for layer, need in self.state_layers.items():
            views[layer] = StateLayerCache(self.slots.add_layer(layer, need.shape, need.dtype, device))
        return views

    def bytes_per_page(self, itemsize: int) -> int:
        return sum(g.bytes_per_page(self.page_size, itemsize) for g in self.groups)

    # ------------------------------------------------------------------ requests
    def can_admit(self) -> bool:
        return self.slots.num_free > 0

    def admit(self, request_id, prompt=None) -> RequestCache:
        """Gives the request a state slot and, with prefix reuse, the pages of the longest
        known prefix of `prompt`; `num_tokens` tells how many tokens those pages cover."""
        if request_id in self.live:
            raise KeyError(f"request {request_id!r} is already live")
        rc = RequestCache(request_id, self.slots.take(), [PageTable() for _ in self.groups],
                          freed_upto=[0 for _ in self.groups])
        self.live[request_id] = rc
        if self.prefix_cache and prompt is not None and self.groups:
            P = self.page_size
            parent, hashes, found = b"", [], []
            for i in range((len(prompt) - 1) // P):       # always leaves >= 1 token to compute
                h = chain_hash(parent, prompt[i * P:(i + 1) * P])
                pages = [grp.pool.lookup(h) for grp in self.groups]
                if any(p is None and grp.need.window is None for p, grp in zip(pages, self.groups)):
                    break
                hashes.append(h)
                found.append(pages)
                parent = h
            n = len(hashes)                               # pages known from the start where there is no window
            windowed = [g for g, grp in enumerate(self.groups) if grp.need.window is not None]
            while n > 0 and not all(found[i][g] is not None for g in windowed
                                    for i in range(self._first_page_needed(g, n * P), n)):
                n -= 1
            for g, grp in enumerate(self.groups):
                first = self._first_page_needed(g, n * P)
                for i in range(n):
                    if i >= first:
                        grp.pool.touch(found[i][g])
                    rc.tables[g].append(found[i][g] if i >= first else -1)
                rc.freed_upto[g] = first
            rc.hashes = hashes[:n]
            rc.num_tokens = n * P
            rc.tokens = list(prompt[:rc.num_tokens])
            self.stats["prefix_hit_pages"] += n
            self.stats["prefix_hit_tokens"] += rc.num_tokens
        return rc

    def _first_page_needed(self, g: int, num_tokens: int) -> int:
        """The first logical page of group g that a query at position >= num_tokens can still see: it sees keys at
        positions > num_tokens - window, and all keys in a group without a window."""
        w = self.groups[g].need.window
        return 0 if w is None else max(0, num_tokens - w + 1) // self.page_size

    def pages_needed(self, rc: RequestCache, new_len: int) -> list:
        """Pages each group must still allocate so that positions < new_len have a page."""
        want = -(-new_len // self.page_size)
        return [max(0, want - len(t)) for t in rc.tables]

    def can_grow(self, rc: RequestCache, new_len: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(rc, new_len), self.groups))

    def max_len_allocatable(self, rc: RequestCache) -> int:
        """The longest length this request could grow to with the pages that are free now."""
        if not self.groups:
            return 1 << 60
        return min((len(t) + g.pool.num_free) * self.page_size for t, g in zip(rc.tables, self.groups))

    def grow(self, rc: RequestCache, new_len: int) -> None:
        """Allocates pages so that positions < new_len have one; all or nothing."""
        need = self.pages_needed(rc, new_len)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"need {n} pages, {g.pool.num_free} are free")
        for n, g, t in zip(need, self.groups, rc.tables):
            for _ in range(n):
                t.append(g.pool.alloc())
            self.stats["pages_allocated"] += n

    def commit(self, rc: RequestCache, new_tokens) -> None:
        """Records that the step which writes `new_tokens` at positions num_tokens.. has been
        issued: hashes pages that became full, gives back pages that a window has passed."""
        P = self.page_size
        rc.num_tokens += len(new_tokens)
        if self.prefix_cache:
            rc.tokens.extend(int(t) for t in new_tokens)
            while (len(rc.hashes) + 1) * P <= rc.num_tokens:
                i = len(rc.hashes)
                parent = rc.hashes[-1] if rc.hashes else b""
                h = chain_hash(parent, rc.tokens[i * P:(i + 1) * P])
                for g, grp in enumerate(self.groups):
                    grp.pool.register(rc.tables[g][i], h)
                rc.hashes.append(h)
        for g, grp in enumerate(self.groups):
            if grp.need.window is None:
                continue
            upto = self._first_page_needed(g, rc.num_tokens)
            for i in range(rc.freed_upto[g], min(upto, len(rc.tables[g]))):
                if rc.tables[g][i] >= 0:
                    grp.pool.release([rc.tables[g][i]])
                    rc.tables[g][i] = -1
                    self.stats["pages_released"] += 1
            rc.freed_upto[g] = max(rc.freed_upto[g], min(upto, len(rc.tables[g])))

    def release(self, request_id) -> None:
        """The request is over (finished or preempted): everything it holds is given back."""
        rc = self.live.pop(request_id)
        for g, grp in enumerate(self.groups):
            held = [p for p in rc.tables[g] if p >= 0]
            grp.pool.release(held)
            self.stats["pages_released"] += len(held)
        self.slots.give_back(rc.slot)

    # -------------------------------------------------------------------- checks
    def check(self) -> None:
        """No page lost, none held twice without being counted twice, none both held and free."""
        for g, grp in enumerate(self.groups):
            grp.pool.check()
            holders = [0] * grp.pool.num_pages
            for rc in self.live.values():
                for p in rc.tables[g]:
                    if p >= 0:
                        holders[p] += 1
            assert holders == grp.pool.ref, f"group {g}: reference counts {grp.pool.ref} != holders {holders}"
        assert len(self.slots.held) == len(self.live) == len({rc.slot for rc in self.live.values()})
        assert len(self.slots.held) + self.slots.num_free == self.max_live
