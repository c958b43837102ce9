"""Gated feed-forward: down(act(gate(x)) * up(x)), act = SiLU, no bias
(jllm/model/common.py:75-76).  Gate and up matrices are stored packed, gate rows first,
so that one product reads the input once."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec
from .registry import register_feed_forward


class GatedMLP(Part):
    kernels = ("activation", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward: activation {spec.activation!r} is not built (silu is)")
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        p, s = self.prefix, self.spec
        return {f"{p}.gate_proj.weight": TensorSpec((s.intermediate_size, s.hidden_size)),
                f"{p}.up_proj.weight": TensorSpec((s.intermediate_size, s.hidden_size)),
                f"{p}.down_proj.weight": TensorSpec((s.hidden_size, s.intermediate_size))}

    def bind(self, tensors):
        p = self.prefix
        g = self.compute_weight(tensors[f"{p}.gate_proj.weight"], self.ctx)
        u = self.compute_weight(tensors[f"{p}.up_proj.weight"], self.ctx)
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = self.compute_weight(tensors[f"{p}.down_proj.weight"], self.ctx).contiguous()

    def forward(self, x, step):
        dt = self.ctx.dtype
        act = ops.swiglu(ops.linear(x, self.w_gate_up, dt))
        return ops.linear(act, self.w_down, dt)


register_feed_forward("gated_mlp", GatedMLP)
