"""RMSNorm over the hidden axis: y = h * rsqrt(mean(h^2) + eps) * weight, in 32-bit
(jllm/model/common.py:44-48), fused with the residual sum before it."""

from __future__ import annotations

from .. import ops
from .base import Part, TensorSpec
from .registry import register_norm


class RMSNorm(Part):
    kernels = ("norm",)

    def __init__(self, spec, prefix, ctx):
        self.size, self.eps = spec.size, float(spec.eps)
        self.name = f"{prefix}.{spec.name}" if prefix else spec.name
        self.ctx = ctx
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.size,), kind="vector", init="ones_normal")}

    def bind(self, tensors):
        self.weight = tensors[self.name].contiguous()

    def norm(self, h, delta=None):
        """x = norm(h + delta); h is updated in place with the sum."""
        return ops.rmsnorm(h, self.weight, self.eps, self.ctx.dtype, delta=delta)

    def gather(self, h, delta, rows):
        """x[i] = norm(h[rows[i]] + delta[rows[i]]); h is left as it is."""
        return ops.rmsnorm(h, self.weight, self.eps, self.ctx.dtype, delta=delta, rows=rows)


register_norm("rmsnorm", RMSNorm)
