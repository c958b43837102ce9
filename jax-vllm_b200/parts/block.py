"""Arrangement of a layer: pre-norm with two residual sums
(jllm/model/common.py:140-147),

    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h)).

The stream `h` is float32 in every mode.  A block hands back its last branch output as
`delta`, not yet added, so that the next norm (of the next block, or the final one) adds
and normalises in one pass over the stream.  A branch output is a tensor [n, hidden] or an
`ops.PartialSum` (the parts of a product whose k was cut); the norms take either.
"""

from __future__ import annotations

from ..ops import trace_range
from .base import Part
from .registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, build, register_block


class PreNormBlock(Part):
    def __init__(self, spec, prefix, ctx):
        p = spec.prefix
        self.spec = spec
        self.mixer_norm = build(NORMS, "norm", spec.mixer_norm, p, ctx)
        self.mixer = build(MIXERS, "mixer", spec.mixer, p, ctx)
        self.ffn_norm = build(NORMS, "norm", spec.ffn_norm, p, ctx)
        self.feed_forward = build(FEED_FORWARDS, "feed-forward", spec.feed_forward, p, ctx)
        if spec.cache_from is not None:
            if not hasattr(self.mixer, "writes_cache"):
                raise ValueError(f"{p}: this mixer cannot read another layer's cache")
            self.mixer.writes_cache = False

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def tensor_specs(self):
        out = {}
        for part in self.parts():
            out.update(part.tensor_specs())
        return out

    def bind(self, tensors):
        for part in self.parts():
            part.bind(tensors)

    def forward(self, h, delta, step, cache):
        with trace_range("mixer_norm"):
            x = self.mixer_norm.norm(h, delta)
        with trace_range("mixer"):
            a = self.mixer.forward(x, step, cache)
        with trace_range("ffn_norm"):
            x = self.ffn_norm.norm(h, a)
        with trace_range("feed_forward"):
            return h, self.feed_forward.forward(x, step)


register_block("pre_norm", PreNormBlock)


def build_block(spec, ctx):
    return build(BLOCKS, "block", spec, spec.prefix, ctx)
