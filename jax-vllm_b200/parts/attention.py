"""Grouped-query causal attention over the paged cache.

    qkv = x @ [Wq; Wk; Wv]^T                     one product over the packed matrix
    q, k = per-head RMSNorm (optional), rotation  csrc/rope_kv.cu, in place; k, v -> cache
    o    = softmax(q k^T * scale + mask) v        over the request's pages
    y    = o @ Wo^T

Formulas as in the reference (jllm/model/common.py:107-137,173-214): query head h reads kv
head h // (Hq/Hkv); key j is visible to the query at position p iff j <= p (and
j > p - window if the layer has a window); the scale is a parameter of the spec.  The
three projection matrices are stored packed so that one product reads the input once.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import PagedKVNeed, Part, TensorSpec
from .registry import POSITIONS, build, register_mixer


class Attention(Part):
    kernels = ("rope_kv", "attn_simt", "gemm_simt")

    def __init__(self, spec, prefix, ctx):
        self.spec, self.ctx = spec, ctx
        self.prefix = f"{prefix}.{spec.prefix}" if spec.prefix else prefix
        self.hq, self.hkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        if self.hq % self.hkv:
            raise ValueError(f"{self.hq} query heads are not a multiple of {self.hkv} kv heads")
        if self.d % 16 or not 16 <= self.d <= 256:
            raise ValueError(f"head size {self.d} is not supported: the attention kernels take multiples of 16 "
                             f"from 16 to 256")
        self.position = build(POSITIONS, "position encoding", spec.position, self.prefix, ctx) \
            if spec.position is not None else None
        if self.position is not None and self.position.dim > self.d:
            raise ValueError("rotary dim exceeds the head size")
        self.window = int(spec.window) if spec.window else 0
        self.writes_cache = True          # set False by the model for a layer that reads another's cache
        # bfloat16 with a head size the tensor-core kernels are built for; else the CUDA-core kernel
        self.use_mma = ops.attn_mma_supports(ctx.dtype, self.d)
        if self.use_mma:
            self.kernels = ("rope_kv", "attn_mma", "gemm_simt", "linear_skinny")
            if self.d == 128 and not self.window:
                self.kernels += ("attn_tcgen05", "attn_decode_tcgen05")
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    # -------------------------------------------------------------------- weights
    def _names(self):
        p = self.prefix
        return {k: f"{p}.{k}.weight" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")}

    def tensor_specs(self):
        n, s = self._names(), self.spec
        specs = {n["q_proj"]: TensorSpec((self.hq * self.d, s.hidden_size)),
                 n["o_proj"]: TensorSpec((s.hidden_size, self.hq * self.d))}
        if self.writes_cache:
            specs[n["k_proj"]] = TensorSpec((self.hkv * self.d, s.hidden_size))
            specs[n["v_proj"]] = TensorSpec((self.hkv * self.d, s.hidden_size))
        if s.qk_norm_eps is not None:
            specs[n["q_norm"]] = TensorSpec((self.d,), kind="vector", init="ones_normal")
            if self.writes_cache:
                specs[n["k_norm"]] = TensorSpec((self.d,), kind="vector", init="ones_normal")
        return specs

    def bind(self, tensors):
        n = self._names()
        mats = [tensors[n["q_proj"]]]
        if self.writes_cache:
            mats += [tensors[n["k_proj"]], tensors[n["v_proj"]]]
        mats = [self.compute_weight(m, self.ctx) for m in mats]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.to(torch.float32) for m in mats]
        self.w_qkv = torch.cat(mats, dim=0).contiguous()
        self.w_o = self.compute_weight(tensors[n["o_proj"]], self.ctx).contiguous()
        if self.spec.qk_norm_eps is not None:
            self.q_norm = tensors[n["q_norm"]].contiguous()
            self.k_norm = tensors[n["k_norm"]].contiguous() if self.writes_cache else None
            if self.k_norm is not None and self.k_norm.dtype != self.q_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    # ---------------------------------------------------------------------- cache
    def cache_need(self):
        return PagedKVNeed(self.hkv, self.d, self.window or None)

    FOREVER = 1 << 30

    def tile_classes(self, page_size: int):
        """Entries of several tokens: tiles of the mma.sync (or CUDA-core) kernel, and for portions that fill
        a 128-row tile of the tcgen05 kernel (head size 128, bfloat16, no window) tiles of that one."""
        small = (ops.attn_mma_tokens_per_tile if self.use_mma else ops.attn_simt_tokens_per_tile)(self.hq, self.hkv)
        if ops.attn_tcgen05_supports(self.ctx.dtype, self.d, self.hq, self.hkv, page_size, self.window):
            big = ops.attn_tcgen05_tokens_per_tile(self.hq, self.hkv)
            return [(small, 2, big), (big, big, self.FOREVER)]
        return [(small, 2, self.FOREVER)]

    # ----------------------------------------------------------------------- step
    def forward(self, x, step, cache):
        dt = self.ctx.dtype
        qkv = ops.linear(x, self.w_qkv, dt)
        table = step.block_tables[cache.group]
        writes = self.writes_cache and cache.writes
        out = torch.empty((step.n_tokens, self.hq * self.d), dtype=dt, device=x.device)
        dwork, n_dec = step.decode_work
        if writes and n_dec == step.n_tokens and self._decode_kernel_prepares(cache, n_dec):
            # single tokens only: the decode kernel does the norm, the rotation and the cache write itself
            freq = self.position.table() if self.position is not None else None
            ops.attn_decode_tcgen05(qkv, qkv.stride(0), out, cache.k, cache.v, table, step.cu_seqlens, step.start_pos,
                                    dwork, n_dec, self.hq, self.hkv, self.d, self.spec.scale,
                                    prepare=(freq, self.q_norm, self.k_norm, self.spec.qk_norm_eps or 0.0))
            return ops.linear(out, self.w_o, dt, parts_ok=True)
        ops.rope_kv(qkv, step.positions, step.token_entry, table,
                    self.position.table() if self.position is not None else None,
                    self.q_norm, self.k_norm, self.spec.qk_norm_eps or 0.0,
                    cache.k if writes else None, cache.v if writes else None, self.hq, self.hkv, self.d)
        self.attend(qkv, out, step, cache, table)
        return ops.linear(out, self.w_o, dt, parts_ok=True)    # maybe the parts of a sum, for the next norm to add

    # The decode kernel prepares a pair's queries in one warp, head after head; the separate kernel spreads the heads
    # of all tokens over the device.  Up to this many query heads per kv head the launch that the kernel saves is
    # worth more (a decode step at batch 8: 3 % faster with 2, equal with 4, 3 % slower with 5 and with 8).
    PREPARE_IN_DECODE_KERNEL_UP_TO = 4

    def _decode_kernel_prepares(self, cache, n_dec) -> bool:
        """Whether the tcgen05 decode kernel takes these tokens together with their preparation (it rotates whole
        heads only)."""
        return (self.hq // self.hkv <= self.PREPARE_IN_DECODE_KERNEL_UP_TO
                and ops.attn_decode_tcgen05_supports(self.ctx.dtype, self.d, self.hq, self.hkv, cache.k.shape[1], self.window,
                                                     n_dec)
                and (self.position is None or self.position.dim == self.d))

    def attend(self, qkv, out, step, cache, table):
        common = (cache.k, cache.v, table, step.cu_seqlens, step.start_pos)
        kernel = ops.attn_mma if self.use_mma else ops.attn_simt
        for cls in self.tile_classes(cache.k.shape[1]):
            work, n_work = step.tile_work[cls]
            if not n_work:
                continue
            if cls[2] == self.FOREVER and cls[1] > 2:      # the class of whole 128-row tiles
                ops.attn_tcgen05(qkv, qkv.stride(0), out, *common, work, n_work, self.hq, self.hkv, self.d,
                                 self.spec.scale)
            else:
                kernel(qkv, qkv.stride(0), out, *common, work, n_work, self.hq, self.hkv, self.d, self.window,
                       self.spec.scale)
        dwork, n_dec = step.decode_work
        if n_dec and ops.attn_decode_tcgen05_supports(self.ctx.dtype, self.d, self.hq, self.hkv, cache.k.shape[1],
                                                      self.window, n_dec):
            # single tokens, head size 128: one persistent launch over the key tiles of all requests
            ops.attn_decode_tcgen05(qkv, qkv.stride(0), out, *common, dwork, n_dec, self.hq, self.hkv, self.d,
                                    self.spec.scale)
        elif n_dec:
            split = self.ctx.decode_split_size
            n_splits = max(1, -(-step.max_seq_len // split))
            kernel(qkv, qkv.stride(0), out, *common, dwork, n_dec, self.hq, self.hkv, self.d,
                   self.window, self.spec.scale, split_size=split, n_splits=n_splits)


register_mixer("attention", Attention)
