"""Builds the device-side description of one batch (`StepContext`).

An entry is (what the request holds in the cache, its next tokens, the places among them
whose logits are wanted).  All integer arrays of the batch are laid out in one pinned
host buffer and reach the device in one copy; the parts get views into the device
buffer.  A reused page needs no clearing: positions at or beyond a request's length are
never read.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..parts.base import StepContext


@dataclass
class StepEntry:
    cache: object                 # cache.RequestCache of the request
    tokens: list                  # its next tokens (written at positions cache.num_tokens ..)
    want: tuple = ()              # indices into `tokens` whose logits are wanted


class BatchLayout:
    """Offsets (in int32 elements) of the arrays of a batch inside one buffer."""

    def __init__(self, n_tokens, n_entries, n_rows, table_widths, tile_counts: dict, n_decode):
        off = 0
        self.sections = {}

        def add(name, n):
            nonlocal off
            self.sections[name] = (off, n)
            off += (n + 3) // 4 * 4            # keep every array 16-byte aligned

        add("token_ids", n_tokens); add("positions", n_tokens); add("token_entry", n_tokens)
        add("cu_seqlens", n_entries + 1); add("start_pos", n_entries); add("state_slots", n_entries)
        add("logit_rows", n_rows)
        for g, w in enumerate(table_widths):
            add(f"table{g}", n_entries * w)
        for cls, n in tile_counts.items():
            add(f"tiles{cls}", 2 * n)
        add("decode", 2 * n_decode)
        self.total = max(off, 4)
        self.table_widths = list(table_widths)
        self.tile_counts = dict(tile_counts)

    def view(self, buf, name):
        off, n = self.sections[name]
        return buf[off:off + n]


class BatchBuilder:
    def __init__(self, n_groups: int, page_size: int, tile_classes, device):
        """`tile_classes`: the work lists that mixers want for entries of more than one token, each a
        triple (tokens per tile, least number of new tokens, one more than the most): an entry of q new
        tokens with least <= q < most is cut into tiles of that many tokens in that list."""
        self.n_groups, self.page_size = n_groups, page_size
        self.tile_token_sizes = [tuple(c) for c in tile_classes]
        self.device = torch.device(device)
        self._pinned = None
        self._copied = None           # event: the last copy out of the pinned buffer has finished

    def _staging(self, n: int) -> torch.Tensor:
        if self._copied is not None:
            self._copied.synchronize()
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=self.device.type == "cuda")
        return self._pinned

    def fill(self, entries, host: np.ndarray, layout: BatchLayout) -> None:
        """Writes the arrays of `entries` into `host` according to `layout`."""
        P = self.page_size
        v = lambda name: layout.view(host, name)
        tok, pos, ent = v("token_ids"), v("positions"), v("token_entry")
        cu, start, slots, rows = v("cu_seqlens"), v("start_pos"), v("state_slots"), v("logit_rows")
        n = r = 0
        cu[0] = 0
        tiles = {cls: [] for cls in layout.tile_counts}
        decode = []
        for e, entry in enumerate(entries):
            q = len(entry.tokens)
            s = entry.cache.num_tokens
            tok[n:n + q] = entry.tokens
            pos[n:n + q] = np.arange(s, s + q, dtype=np.int32)
            ent[n:n + q] = e
            for w in entry.want:
                if not 0 <= w < q:
                    raise IndexError(f"wanted place {w} outside the entry's {q} tokens")
                rows[r] = n + w
                r += 1
            start[e], slots[e] = s, entry.cache.slot
            n += q
            cu[e + 1] = n
            if q == 1:
                decode.append((e, 0))
            else:
                for cls in tiles:
                    tpt, lo, hi = cls
                    if lo <= q < hi:
                        tiles[cls].extend((e, t) for t in range(0, q, tpt))
            for g in range(self.n_groups):
                w = layout.table_widths[g]
                row = layout.view(host, f"table{g}")[e * w:(e + 1) * w]
                t = entry.cache.tables[g]
                need = -(-(s + q) // P)
                if len(t) < need:
                    raise RuntimeError(f"request {entry.cache.request_id!r} has {len(t)} pages, "
                                       f"{s + q} tokens need {need}")
                if need > w:
                    raise RuntimeError(f"block table of width {w} is too narrow for {need} pages")
                row[:need] = t.array(need)
                row[need:] = -1
        for cls, lst in tiles.items():
            if lst:
                layout.view(host, f"tiles{cls}")[:] = np.asarray(lst, dtype=np.int32).reshape(-1)
        if decode:
            v("decode")[:] = np.asarray(decode, dtype=np.int32).reshape(-1)

    def layout_for(self, entries, table_width=None) -> BatchLayout:
        P = self.page_size
        n_tokens = sum(len(e.tokens) for e in entries)
        n_rows = sum(len(e.want) for e in entries)
        widest = max([1] + [-(-(e.cache.num_tokens + len(e.tokens)) // P) for e in entries])
        w = table_width or widest
        tile_counts = {cls: sum(-(-len(e.tokens) // cls[0]) for e in entries if len(e.tokens) > 1 and cls[1] <= len(e.tokens) < cls[2])
                       for cls in self.tile_token_sizes}
        n_decode = sum(1 for e in entries if len(e.tokens) == 1)
        return BatchLayout(n_tokens, len(entries), n_rows, [w] * self.n_groups, tile_counts, n_decode)

    def context(self, entries, layout: BatchLayout, dev: torch.Tensor, max_seq_len=None) -> StepContext:
        v = lambda name: layout.view(dev, name)
        n_tokens = sum(len(e.tokens) for e in entries)
        n_rows = sum(len(e.want) for e in entries)
        R = len(entries)
        tables = [v(f"table{g}").view(R, layout.table_widths[g]) for g in range(self.n_groups)]
        tile_work = {cls: (v(f"tiles{cls}").view(-1, 2), n) for cls, n in layout.tile_counts.items()}
        n_dec = layout.sections["decode"][1] // 2
        seq = max([1] + [e.cache.num_tokens + len(e.tokens) for e in entries])
        return StepContext(
            n_tokens=n_tokens, n_entries=R, token_ids=v("token_ids"), positions=v("positions"),
            token_entry=v("token_entry"), cu_seqlens=v("cu_seqlens"), start_pos=v("start_pos"),
            state_slots=v("state_slots"), logit_rows=v("logit_rows"), n_logit_rows=n_rows, block_tables=tables,
            tile_work=tile_work, decode_work=(v("decode").view(-1, 2), n_dec),
            max_seq_len=max_seq_len or seq,
            host_q_lens=[len(e.tokens) for e in entries], host_start_pos=[e.cache.num_tokens for e in entries],
            host_slots=[e.cache.slot for e in entries])

    def build(self, entries) -> StepContext:
        """Lays the batch out, copies it to the device (one copy) and returns the context."""
        layout = self.layout_for(entries)
        pinned = self._staging(layout.total)
        host = pinned.numpy()[:layout.total]
        self.fill(entries, host, layout)
        dev = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        dev.copy_(pinned[:layout.total], non_blocking=True)
        if self.device.type == "cuda":
            self._copied = torch.cuda.Event()
            self._copied.record()
        return self.context(entries, layout, dev)
