"""The step function: one batch of (request, its next tokens) through the model.

Portions of prompts stand beside single decoded tokens, cut anywhere; only the tokens
given are run, against what earlier steps left in the cache; logits come back for the
wanted places only.  The reference needs two calls for this, a prefill step of padded
one-page rows and a decode step of padded single tokens (jllm/engine/generate.py:112-143,
233-265); here it is one flat batch without padding.
"""

from __future__ import annotations

import contextlib
import gc

import torch

from .. import ops
from ..cache import CacheManager
from ..csrc import build as kernel_build
from ..parts import BuildContext, Model
from .batch import BatchBuilder, StepEntry


@contextlib.contextmanager
def _capture(graph, pool=None):
    """`torch.cuda.graph(graph, pool)` with Python's cycle collector off: a collection that happened to run inside the
    capture and freed CUDA objects of some other owner (an old driver's graphs, pinned buffers) would invalidate it."""
    was_on = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, pool=pool):
            yield
    finally:
        if was_on:
            gc.enable()


class _DecodeGraph:
    """A captured step for `n` single-token entries: fixed buffers, fixed launch sizes.  With sampling in
    the graph, `out` holds the sampled tokens followed by the kernels' status word, and the sampling
    parameters lie behind the batch in the same buffer, from `samp_off` on: n seeds and n counters (64-bit),
    then n temperatures."""

    def __init__(self, layout, dev, logits, graph, launches, out=None, samp_off=0):
        self.layout, self.dev, self.logits, self.graph, self.launches = layout, dev, logits, graph, launches
        self.out, self.samp_off = out, samp_off
        self.total = layout.total if out is None else samp_off + 5 * layout.sections["token_ids"][1]


class Runner:
    def __init__(self, model: Model, cache: CacheManager, device, dtype: torch.dtype, max_model_len: int | None = None,
                 cuda_graphs: bool = False, max_graph_batch: int = 256):
        """With `cuda_graphs` (which needs `max_model_len`), a step whose entries are all single
        tokens with their logits wanted is replayed from a CUDA graph captured for that number
        of entries: block tables have the width of `max_model_len`, and the split attention is
        launched for `max_model_len` keys (blocks beyond a request's length leave at once)."""
        self.model, self.cache = model, cache
        self.max_model_len = max_model_len
        self.cuda_graphs = bool(cuda_graphs) and max_model_len is not None
        self.max_graph_batch = max_graph_batch
        self.graphs: dict[int, _DecodeGraph] = {}
        # All captured steps of this runner take their intermediate tensors from one pool: they never run at the same
        # time, and nothing but a graph's result (which stays allocated) is read after its replay, so the graphs of
        # all batch sizes together hold what the largest needs, not the sum.
        self.graph_pool = None
        self.graphs_sampled: dict[int, _DecodeGraph] = {}
        self.graph_warm: set[int] = set()
        self._ahead = None                 # (requests and lengths, graph) of a batch already laid out in the staging buffer
        self.launches_last_step = 0
        self.graph_replays = 0             # steps that were replayed from a captured graph
        # a part that reads the batch from the host lists of the step context (not from its device tensors)
        # would see, in a replay, the lists of the step that was captured: such a model is never captured
        self.capturable = model.capturable()
        self.device, self.dtype = torch.device(device), dtype
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only (there is no CPU path)")
        kernel_build.build_all(model.kernels() + ["sampling"])
        views = cache.allocate_storage(dtype, self.device)
        self.layer_caches = [views.get(k) for k in range(len(model.order))]
        self.builder = BatchBuilder(len(cache.groups), cache.page_size, model.tile_classes(cache.page_size), self.device)
        self.steps = 0

    @torch.no_grad()
    def step(self, entries: list) -> torch.Tensor:
        """Runs the entries as one batch.  Every entry's pages must have been allocated
        (`cache.grow`); the caller commits the new tokens afterwards (`cache.commit`).
        Returns float32 logits [sum of wanted places, vocab] in the order of the entries
        and of their `want`."""
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        self._ahead = None                 # the staging buffer is about to be written
        with torch.cuda.device(self.device):
            with ops.trace_range("step"):
                if self._graphable(entries):
                    logits = self._step_graph(entries)
                else:
                    ctx = self.builder.build(entries)
                    logits = self.model.forward(ctx, self.layer_caches)
        self.steps += 1
        return logits

    # ----------------------------------------------------------- captured decode steps
    def _graphable(self, entries) -> bool:
        if not self.cuda_graphs or not self.capturable or len(entries) > self.max_graph_batch:
            return False
        return all(len(e.tokens) == 1 and tuple(e.want) == (0,) and e.cache.num_tokens < self.max_model_len
                   for e in entries)

    def _pool(self):
        if self.graph_pool is None:
            self.graph_pool = torch.cuda.graph_pool_handle()
        return self.graph_pool

    def _graph_layout(self, entries):
        width = -(-self.max_model_len // self.cache.page_size)
        return self.builder.layout_for(entries, table_width=width)

    def _step_graph(self, entries) -> torch.Tensor:
        n = len(entries)
        b = self.builder
        g = self.graphs.get(n)
        if g is None and n not in self.graph_warm:
            # first time at this size: run it eagerly once (kernels get their one-time set-up
            # outside a capture), with the same fixed sizes that the capture will have
            self.graph_warm.add(n)
            layout = self._graph_layout(entries)
            pinned = b._staging(layout.total)
            b.fill(entries, pinned.numpy()[:layout.total], layout)
            dev = torch.empty(layout.total, dtype=torch.int32, device=self.device)
            dev.copy_(pinned[:layout.total], non_blocking=True)
            b._copied = torch.cuda.Event(); b._copied.record()
            return self.model.forward(b.context(entries, layout, dev, max_seq_len=self.max_model_len),
                                      self.layer_caches)
        if g is None:
            layout = self._graph_layout(entries)
            dev = torch.zeros(layout.total, dtype=torch.int32, device=self.device)
            pinned = b._staging(layout.total)
            b.fill(entries, pinned.numpy()[:layout.total], layout)
            dev.copy_(pinned[:layout.total], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            ctx = b.context(entries, layout, dev, max_seq_len=self.max_model_len)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            with _capture(graph, self._pool()):
                logits = self.model.forward(ctx, self.layer_caches)
            g = _DecodeGraph(layout, dev, logits, graph, ops.launch_count - before)
            ops.launch_count = before           # nothing ran yet: a replay counts them
            self.graphs[n] = g
        pinned = b._staging(g.layout.total)
        b.fill(entries, pinned.numpy()[:g.layout.total], g.layout)
        g.dev.copy_(pinned[:g.layout.total], non_blocking=True)
        b._copied = torch.cuda.Event(); b._copied.record()
        g.graph.replay()
        self.graph_replays += 1
        ops.launch_count += g.launches
        return g.logits

    # ------------------------------------------- captured decode steps that also sample
    @staticmethod
    def _key(entries):
        return tuple((e.cache.request_id, e.cache.num_tokens) for e in entries)

    def _fill_sampling(self, host, g: _DecodeGraph, temps, seeds, counters) -> None:
        n = len(temps)
        wide = host[g.samp_off:g.samp_off + 4 * n].view("int64")
        wide[:n] = [s & ((1 << 63) - 1) for s in seeds]
        wide[n:2 * n] = counters
        host[g.samp_off + 4 * n:g.samp_off + 5 * n].view("float32")[:] = temps

    @torch.no_grad()
    def step_sampled(self, entries: list, temps, seeds, counters):
        """A decode-only step with the sampling inside the replayed graph: returns the sampled tokens followed
        by the kernels' status word (int32, on the device), or None if this batch has to go the ordinary way
        (`step`, then the sampler): not all single tokens, or the first time at this batch size."""
        n = len(entries)
        if not self._graphable(entries) or n not in self.graph_warm:
            return None
        b = self.builder
        with torch.cuda.device(self.device):
            g = self.graphs_sampled.get(n)
            if g is None:
                layout = self._graph_layout(entries)
                samp_off = (layout.total + 1) // 2 * 2
                dev = torch.zeros(samp_off + 5 * n, dtype=torch.int32, device=self.device)
                out = torch.zeros(n + 1, dtype=torch.int32, device=self.device)
                g = _DecodeGraph(layout, dev, None, None, 0, out=out, samp_off=samp_off)
                pinned = b._staging(g.total)
                host = pinned.numpy()[:g.total]
                b.fill(entries, host, layout)
                self._fill_sampling(host, g, temps, seeds, counters)
                dev.copy_(pinned[:g.total], non_blocking=True)
                torch.cuda.current_stream().synchronize()
                ctx = b.context(entries, layout, dev, max_seq_len=self.max_model_len)
                seeds_d = dev[samp_off:samp_off + 2 * n].view(torch.int64)
                counters_d = dev[samp_off + 2 * n:samp_off + 4 * n].view(torch.int64)
                temps_d = dev[samp_off + 4 * n:samp_off + 5 * n].view(torch.float32)
                graph = torch.cuda.CUDAGraph()
                before = ops.launch_count
                with _capture(graph, self._pool()):
                    logits = self.model.forward(ctx, self.layer_caches)
                    out[:n].copy_(ops.sample(logits, temps_d, seeds_d, counters_d))
                    out[n:].copy_(ops.status_word(self.device))
                    del logits                  # only `out` is read after a replay: the logits' memory serves later captures
                g.graph, g.launches = graph, ops.launch_count - before
                ops.launch_count = before       # nothing ran yet: a replay counts them
                self.graphs_sampled[n] = g
                self._ahead = None
            ahead, self._ahead = self._ahead, None
            pinned = b._pinned
            if ahead is not None and ahead[1] is g and ahead[0] == self._key(entries):
                # the batch was laid out while the device ran the last step: only the tokens are new
                host = pinned.numpy()[:g.total]
                g.layout.view(host, "token_ids")[:] = [e.tokens[0] for e in entries]
            else:
                pinned = b._staging(g.total)
                host = pinned.numpy()[:g.total]
                b.fill(entries, host, g.layout)
                self._fill_sampling(host, g, temps, seeds, counters)
            g.dev.copy_(pinned[:g.total], non_blocking=True)
            b._copied = torch.cuda.Event(); b._copied.record()
            g.graph.replay()
            self.graph_replays += 1
            ops.launch_count += g.launches
        self.steps += 1
        return g.out

    def prefill_ahead(self, entries: list, temps, seeds, counters) -> None:
        """Lays out the next decode step (tokens not known yet) in the staging buffer while the device runs
        this one.  `entries` carry the lengths that the requests will have then; `step_sampled` uses the
        layout if it is called with exactly these requests at these lengths."""
        self._ahead = None
        g = self.graphs_sampled.get(len(entries))
        if g is None or not self._graphable(entries):
            return
        b = self.builder
        pinned = b._staging(g.total)          # waits until the last copy out of it has finished
        host = pinned.numpy()[:g.total]
        b.fill(entries, host, g.layout)
        self._fill_sampling(host, g, temps, seeds, counters)
        self._ahead = (self._key(entries), g)

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
        ops.clear_status(self.device)

    def warm_up(self, decode_batches: int = 0) -> None:
        """One two-token portion and one single token through every kernel of the model; then, with CUDA
        graphs, the decode steps of 1 .. `decode_batches` requests with their sampling are captured (a step
        of each size runs twice: once eagerly, once into the graph), so that no request pays for that."""
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
        if not self.cuda_graphs:
            return
        live = []
        try:
            for n in range(1, min(decode_batches, self.max_graph_batch, self.cache.max_live) + 1):
                if not self.cache.can_admit():
                    break
                rc = self.cache.admit(f"__warm_up_{n}__")
                live.append(rc)
                if not self.cache.can_grow(rc, 2):
                    break
                self.cache.grow(rc, 2)
                rc.num_tokens = 1              # as if one token were cached: the step adds the second
                entries = [StepEntry(r, [0], (0,)) for r in live]
                zeros = [0.0] * n
                if self.step_sampled(entries, zeros, [0] * n, [0] * n) is None:
                    self.step(entries)                                       # the first time at this size: eagerly
                    self.step_sampled(entries, zeros, [0] * n, [0] * n)      # then into the graph
            self.check_kernels()
        finally:
            for r in live:
                r.num_tokens = 0
                self.cache.release(r.request_id)


def build_runner(spec, tensors_fn, *, dtype, device, page_size, num_pages, max_live, prefix_cache=True,
                 decode_split_size=256) -> Runner:
    """Model + cache + runner from a `ModelSpec`; `tensors_fn(specs, optional) -> {name: tensor}`
    supplies the weights (from a folder or at random)."""
    ctx = BuildContext(dtype=dtype, device=torch.device(device), decode_split_size=decode_split_size)
    model = Model(spec, ctx)
    model.bind(tensors_fn(model.tensor_specs(), model.optional_tensors()))
    cache = CacheManager(model.cache_needs(), page_size, num_pages, max_live, prefix_cache)
    return Runner(model, cache, device, dtype)
