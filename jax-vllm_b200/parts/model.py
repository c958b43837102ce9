"""A model put together from a `ModelSpec`: embedding, blocks in their run order, final
norm, output matrix (jllm/model/common.py:150-170).  It owns no cache and no batching: the
step hands it a `StepContext` and the per-layer cache views."""

from __future__ import annotations

import torch

from .. import ops
from .base import BuildContext, Part, TensorSpec
from .block import build_block
from .registry import NORMS, build


class Model(Part):
    def __init__(self, spec, ctx: BuildContext):
        spec.validate()
        self.spec, self.ctx = spec, ctx
        self.layers = [build_block(layer, ctx) for layer in spec.layers]
        self.final_norm = build(NORMS, "norm", spec.final_norm, "", ctx)
        self.embedding = self.lm_head = None

    # -------------------------------------------------------------------- weights
    def tensor_specs(self):
        s = self.spec
        out = {s.embedding_name: TensorSpec((s.vocab_size, s.hidden_size))}
        for layer in self.layers:
            out.update(layer.tensor_specs())
        out.update(self.final_norm.tensor_specs())
        if s.lm_head_name is not None:
            out[s.lm_head_name] = TensorSpec((s.vocab_size, s.hidden_size))
        return out

    def optional_tensors(self):
        """Names that may be in the folder without being used (the output matrix of a tied
        model is ignored, jllm/model/weights.py:142-146)."""
        return {"lm_head.weight"} if self.spec.lm_head_name is None else set()

    def bind(self, tensors):
        s = self.spec
        self.embedding = tensors[s.embedding_name].contiguous()
        for layer in self.layers:
            layer.bind(tensors)
        self.final_norm.bind(tensors)
        head = self.embedding if s.lm_head_name is None else tensors[s.lm_head_name]
        self.lm_head = self.compute_weight(head, self.ctx).contiguous()

    def kernels(self):
        names = {"embed", "norm", "gemm_simt"}
        for layer in self.layers:
            for part in layer.parts():
                names.update(part.kernels)
        return sorted(names)

    # ---------------------------------------------------------------------- cache
    def cache_needs(self):
        """Per layer: its need, or None; a layer with `cache_from` has none of its own."""
        return [None if layer.spec.cache_from is not None else layer.mixer.cache_need() for layer in self.layers]

    def cache_index(self, layer: int) -> int:
        src = self.layers[layer].spec.cache_from
        return layer if src is None else src

    def tile_token_sizes(self):
        sizes = set()
        for layer in self.layers:
            f = getattr(layer.mixer, "tile_tokens", None)
            if f is not None and f() is not None:
                sizes.add(f())
        return sorted(sizes)

    # ----------------------------------------------------------------------- step
    def forward(self, step, caches) -> torch.Tensor:
        """Logits [n_logit_rows, vocab] float32 for one batch; caches are updated in place."""
        h = ops.embed_gather(self.embedding, step.token_ids)
        delta = None
        for i in self.spec.run_order():
            cache = caches[self.cache_index(i)]
            h, delta = self.layers[i].forward(h, delta, step, cache)
        if step.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=h.device)
        x = self.final_norm.gather(h, delta, step.logit_rows)
        return ops.linear(x, self.lm_head, torch.float32)
