"""Interfaces that parts of a model keep to.

A part is built from its spec and a weight-name prefix, says which tensors it wants
(`tensor_specs`), receives them (`bind`) and is then called in the step.  No part knows
which model it sits in.

    Norm            norm(h, delta=None) -> x            h: float32 stream, updated with delta
                    gather(h, delta, rows) -> x[rows]
    Position        table(device) -> tensor handed to the mixer's kernels (e.g. inverse
                    frequencies); rot_dim
    Mixer           forward(x, step, cache) -> y        x, y: [tokens, hidden] compute dtype
                    cache_need() -> PagedKVNeed | FixedStateNeed | None
                    tile_classes() -> work lists it wants for entries of several tokens: triples
                                      (tokens per tile, least new tokens, one more than the most)
    FeedForward     forward(x, step) -> y
    Block           forward(h, delta, step, cache) -> (h, delta)   delta: not yet added to h
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects from the model folder."""
    shape: tuple
    kind: str = "matrix"        # "matrix", "vector" (norm weights and the like) or "table" (integers)
    init: str = "normal"        # random mode: "normal" = N(0, 0.02); "ones_normal" = 1 + N(0, 0.1)


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every earlier token (or of the last `window`), in pages."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedStateNeed:
    """State of a fixed size per request, whatever its length."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class BuildContext:
    dtype: torch.dtype            # compute dtype: activations, 16-bit weights, cache
    device: torch.device
    decode_split_size: int = 256


class Part:
    kernels: tuple = ()           # csrc sources whose launchers the part calls
    # Whether the part's work in a step depends on the step's device tensors only.  A step of single tokens is
    # captured into a CUDA graph once and replayed with new contents in the same device buffers; a part that
    # reads `StepContext.host_*` (or anything else on the host that changes from step to step) would replay the
    # captured step's values, so it says `capturable = False` and its model is stepped eagerly.
    capturable: bool = True

    def tensor_specs(self) -> dict:
        return {}

    def bind(self, tensors: dict) -> None:
        pass

    def compute_weight(self, t: torch.Tensor, ctx: BuildContext) -> torch.Tensor:
        """Matrix weights as the products read them: the compute dtype in 32-bit mode;
        in 16-bit mode a tensor stored in 32-bit stays so (and takes the 32-bit product)."""
        if ctx.dtype == torch.float32 and t.dtype != torch.float32:
            return t.to(torch.float32)
        return t


@dataclass
class PagedLayerCache:
    group: int                    # index into StepContext.block_tables
    k: torch.Tensor               # [num_pages, page_size, kv_heads, head_dim]
    v: torch.Tensor
    writes: bool = True           # False for a layer that reads another layer's cache


@dataclass
class StateLayerCache:
    state: torch.Tensor           # [max_live, *shape], row = state slot of the request


@dataclass
class StepContext:
    """One batch, as the parts see it: N tokens of R entries (an entry = the next tokens
    of one request), all device tensors int32."""
    n_tokens: int
    n_entries: int
    token_ids: torch.Tensor       # [N]
    positions: torch.Tensor       # [N] absolute position of each token in its request
    token_entry: torch.Tensor     # [N] entry of each token
    cu_seqlens: torch.Tensor      # [R+1] token offsets of the entries
    start_pos: torch.Tensor       # [R] tokens of the request already in the cache
    state_slots: torch.Tensor     # [R] fixed-state slot of the request
    logit_rows: torch.Tensor      # [M] token rows whose logits are wanted
    n_logit_rows: int
    block_tables: list            # per cache group: [R, width] page ids (-1 = none)
    tile_work: dict               # tile class (tokens per tile, least, most+1 new tokens) -> (work [n, 2] (entry, first token), n)
    decode_work: tuple            # (work [n, 2], n) for entries of exactly one token
    max_seq_len: int              # longest start_pos + new tokens in the batch (or the engine's bound, in a graph)
    # the same lengths, positions and slots as host lists, for parts that loop over entries on the host; a part
    # that reads them must say `capturable = False`
    host_q_lens: list = field(default_factory=list)
    host_start_pos: list = field(default_factory=list)
    host_slots: list = field(default_factory=list)
