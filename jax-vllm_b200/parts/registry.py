"""Registries of part kinds.  A spec's `kind` picks the class; the class is built as
`cls(spec, prefix, ctx)`.  Tests register toy parts here without touching the package."""

from __future__ import annotations

MIXERS: dict = {}
FEED_FORWARDS: dict = {}
NORMS: dict = {}
POSITIONS: dict = {}
BLOCKS: dict = {}


def _register(table, kind, cls):
    table[kind] = cls
    return cls


def register_mixer(kind, cls): return _register(MIXERS, kind, cls)
def register_feed_forward(kind, cls): return _register(FEED_FORWARDS, kind, cls)
def register_norm(kind, cls): return _register(NORMS, kind, cls)
def register_position(kind, cls): return _register(POSITIONS, kind, cls)
def register_block(kind, cls): return _register(BLOCKS, kind, cls)


def build(table: dict, what: str, spec, prefix: str, ctx):
    kind = getattr(spec, "kind", None)
    try:
        cls = table[kind]
    except KeyError:
        raise ValueError(f"unknown {what} kind {kind!r}; registered: {sorted(table)}") from None
    return cls(spec, prefix, ctx)
