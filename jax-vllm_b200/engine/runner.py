"""The step function: one batch of (request, its next tokens) through the model.

Portions of prompts stand beside single decoded tokens, cut anywhere; only the tokens
given are run, against what earlier steps left in the cache; logits come back for the
wanted places only.  The reference needs two calls for this, a prefill step of padded
one-page rows and a decode step of padded single tokens (jllm/engine/generate.py:112-143,
233-265); here it is one flat batch without padding.
"""

from __future__ import annotations

import torch

from .. import ops
from ..cache import CacheManager
from ..csrc import build as kernel_build
from ..parts import BuildContext, Model
from .batch import BatchBuilder, StepEntry


class Runner:
    def __init__(self, model: Model, cache: CacheManager, device, dtype: torch.dtype):
        self.model, self.cache = model, cache
        self.device, self.dtype = torch.device(device), dtype
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only (there is no CPU path)")
        kernel_build.build_all(model.kernels() + ["sampling"])
        views = cache.allocate_storage(dtype, self.device)
        self.layer_caches = [views.get(i) for i in range(len(model.layers))]
        self.builder = BatchBuilder(len(cache.groups), cache.page_size, model.tile_token_sizes(), self.device)
        self.steps = 0

    @torch.no_grad()
    def step(self, entries: list) -> torch.Tensor:
        """Runs the entries as one batch.  Every entry's pages must have been allocated
        (`cache.grow`); the caller commits the new tokens afterwards (`cache.commit`).
        Returns float32 logits [sum of wanted places, vocab] in the order of the entries
        and of their `want`."""
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            ctx = self.builder.build(entries)
            logits = self.model.forward(ctx, self.layer_caches)
        self.steps += 1
        return logits

    def run(self, entries: list) -> torch.Tensor:
        """grow -> step -> commit, for callers that do not schedule (replay, tests)."""
        for e in entries:
            self.cache.grow(e.cache, e.cache.num_tokens + len(e.tokens))
        logits = self.step(entries)
        for e in entries:
            self.cache.commit(e.cache, e.tokens)
        return logits

    def check_kernels(self) -> None:
        ops.check_status(self.device)

    def status_word(self) -> torch.Tensor:
        return ops.status_word(self.device)

    def clear_status(self) -> None:
        ops.status_word(self.device).zero_()

    def warm_up(self) -> None:
        """One two-token portion and one single token through every kernel of the model."""
        if not self.cache.can_admit():
            return
        rc = self.cache.admit("__warm_up__")
        try:
            self.cache.grow(rc, 3)
            self.step([StepEntry(rc, [0, 0], (1,))])
            rc.num_tokens = 2
            self.step([StepEntry(rc, [0], (0,))])
            self.check_kernels()
        finally:
            rc.num_tokens = 0
            self.cache.release("__warm_up__")


def build_runner(spec, tensors_fn, *, dtype, device, page_size, num_pages, max_live, prefix_cache=True,
                 decode_split_size=256) -> Runner:
    """Model + cache + runner from a `ModelSpec`; `tensors_fn(specs, optional) -> {name: tensor}`
    supplies the weights (from a folder or at random)."""
    ctx = BuildContext(dtype=dtype, device=torch.device(device), decode_split_size=decode_split_size)
    model = Model(spec, ctx)
    model.bind(tensors_fn(model.tensor_specs(), model.optional_tensors()))
    cache = CacheManager(model.cache_needs(), page_size, num_pages, max_live, prefix_cache)
    return Runner(model, cache, device, dtype)
