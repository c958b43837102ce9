"""Rotary position encoding: inv_freq[j] = 1 / theta^(2j/dim), j < dim/2, in 32-bit
(jllm/model/common.py:51-55).  The part only owns the table; the rotation itself is
applied to queries and keys inside the mixer's preparation kernel (csrc/rope_kv.cu), which
forms the angle position * inv_freq[j] and its cos and sin in 32-bit."""

from __future__ import annotations

import torch

from .base import Part
from .registry import register_position


class Rope(Part):
    def __init__(self, spec, prefix, ctx):
        if spec.dim % 2 or spec.dim < 2:
            raise ValueError(f"rotary dim must be even and positive, got {spec.dim}")
        self.dim, self.theta = int(spec.dim), float(spec.theta)
        exponents = torch.arange(0, self.dim, 2, dtype=torch.float32) / self.dim
        self.inv_freq = (1.0 / (self.theta ** exponents)).to(torch.float32).to(ctx.device)

    def table(self):
        return self.inv_freq


register_position("rope", Rope)
