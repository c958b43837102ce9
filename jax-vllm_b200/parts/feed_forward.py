"""Gated feed-forward: down(act(gate(x)) * up(x)), act = SiLU, no bias
(jllm/model/common.py:75-76).  Gate and up matrices are stored packed so that one product reads
the input once: in bfloat16 with an intermediate size that is a multiple of 128, as blocks of 128
gate rows followed by the 128 up rows of the same indices, which lets the tcgen05 product of prompt
steps apply the gate in its epilogue (the [tokens, 2*intermediate] product never reaches memory);
otherwise all gate rows, then all up rows."""

from __future__ import annotations

import torch

from .. import ops
from .base import Part, TensorSpec
from .registry import register_feed_forward


class GatedMLP(Part):
    kernels = ("activation", "gemm_simt")
    BLOCK = 128          # gate/up interleaving of the fused product (a tile of it is 256 columns wide)

    def __init__(self, spec, prefix, ctx):
        if spec.activation != "silu":
            raise ValueError(f"gated feed-forward: activation {spec.activation!r} is not built (silu is)")
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.w_gate_up = self.w_down = self.block = None

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
        inter, hidden = g.shape
        self.block = None
        if self.ctx.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and inter % self.BLOCK == 0 and hidden % 8 == 0:
            self.block = self.BLOCK
            self.kernels = ("activation", "gemm_simt", "gemm_tcgen05", "linear_skinny")
            self.w_gate_up = torch.stack([g.reshape(-1, self.BLOCK, hidden), u.reshape(-1, self.BLOCK, hidden)],
                                         dim=1).reshape(2 * inter, hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = self.compute_weight(tensors[f"{p}.down_proj.weight"], self.ctx).contiguous()

    # The gate is applied in the epilogue of the tcgen05 product once its 128 x 256 tiles are at least this many per
    # multiprocessor; with fewer, too many multiprocessors idle in the last round and the library product followed by
    # the gate kernel is faster.  Measured on 148 multiprocessors, this product against the library's plus the gate
    # kernel, microseconds: 24,576 x 4,096 at 1,024 rows (5.2 tiles each) 165 / 159, at 2,048 rows (10.4) 291 / 307;
    # 34,816 x 5,120 at 1,024 rows (7.4) 275 / 268, at 2,048 rows (14.7) 501 / 507; 51,200 x 5,120 at 1,024 rows (10.8)
    # 388 / 390, at 2,048 rows (21.6) 731 / 728.  FUSED_GATE_ROWS, if set, is a plain row count instead (tests).
    FUSED_GATE_TILES_PER_SM = 9.0
    FUSED_GATE_ROWS = None

    def _fuse_gate(self, rows: int) -> bool:
        if self.block is None:
            return False
        if self.FUSED_GATE_ROWS is not None:
            return rows >= self.FUSED_GATE_ROWS
        tiles = -(-rows // 128) * -(-self.w_gate_up.shape[0] // 256)
        return tiles >= self.FUSED_GATE_TILES_PER_SM * ops.multiprocessors(self.w_gate_up.device)

    def forward(self, x, step):
        dt = self.ctx.dtype
        if self._fuse_gate(x.shape[0]):
            act = ops.gemm_tcgen05(x, self.w_gate_up, "swiglu")
        else:
            act = ops.swiglu(ops.linear(x, self.w_gate_up, dt, parts_ok=True), self.block, out_dtype=dt)
        # a few rows: the product may come as the parts of a sum, which the next norm adds as it reads them
        return ops.linear(act, self.w_down, dt, parts_ok=True)


register_feed_forward("gated_mlp", GatedMLP)
