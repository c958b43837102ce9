"""What a model is made of, as data.

A `ModelSpec` lists layers; a layer names its block arrangement, its mixer, its
feed-forward and its norms; each of those is a small frozen record with a `kind` (the
key under which the part is registered in `parts.registry`) and the sizes and constants
the part needs.  `schedule` is the order in which layers run: a list of layer indices
that may name a layer twice.  A layer whose `cache_from` names another layer reads that
layer's cache and keeps none of its own.  Nothing in this file knows an architecture;
`models/` turns a config.json into these records.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    name: str                      # tensor name of the weight, relative to the owner's prefix
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class RopeSpec:
    dim: int                       # number of rotated elements of a head (<= head size, even)
    theta: float
    kind: str = "rope"


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float                   # multiplies q.k before the softmax
    position: Optional[Any] = None  # a position-encoding spec, or None
    qk_norm_eps: Optional[float] = None  # per-head RMSNorm of queries and keys, or None
    window: Optional[int] = None   # keys visible to a query: the last `window`, or all
    prefix: str = "self_attn"
    kind: str = "attention"


@dataclass(frozen=True)
class GatedMLPSpec:
    hidden_size: int
    intermediate_size: int
    activation: str = "silu"
    prefix: str = "mlp"
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class LayerSpec:
    prefix: str                    # e.g. "model.layers.3"
    mixer: Any
    feed_forward: Any
    mixer_norm: NormSpec
    ffn_norm: NormSpec
    cache_from: Optional[int] = None
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple
    final_norm: NormSpec
    embedding_name: str = "model.embed_tokens.weight"
    lm_head_name: Optional[str] = "lm_head.weight"   # None: the embedding table is the output matrix
    schedule: tuple = field(default=())
    max_position: int = 0

    def run_order(self) -> tuple:
        return self.schedule if self.schedule else tuple(range(len(self.layers)))

    def validate(self) -> None:
        n = len(self.layers)
        for i in self.run_order():
            if not 0 <= i < n:
                raise ValueError(f"schedule names layer {i}, the model has {n}")
        for i, layer in enumerate(self.layers):
            j = layer.cache_from
            if j is not None:
                if not 0 <= j < n or j == i or self.layers[j].cache_from is not None:
                    raise ValueError(f"layer {i}: cache_from={j} must name another layer that owns a cache")
                order = list(self.run_order())
                if j not in order or (i in order and order.index(j) > order.index(i)):
                    raise ValueError(f"layer {i} reads the cache of layer {j}, which must run before it")
