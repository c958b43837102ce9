"""The engine's programming entry point, in the manner of the reference's
(jllm/engine/engine.py:63-233): `make_driver`, `add_request`, `step`, `has_work`,
`stream`, `start`, `stop`, `prewarm`, with the same names and meanings of arguments
(max_num_seqs, max_model_len, max_prefill_len, block_size, num_blocks, dtype), token ids
in and out.  `step` admits, runs ONE batch on the device (decoded tokens and prompt
portions together) and returns the events of the tokens it produced.
"""

from __future__ import annotations

import threading
import time
import weakref
from typing import Iterator, Optional

import torch

from ..cache import CacheManager
from ..config import EngineConfig, parse_dtype
from ..sampling import Sampler
from .background import EventRouter
from .batch import StepEntry
from .request import EngineStats, Request, SamplingParams, StepEvent
from .runner import Runner
from .scheduler import Scheduler


class Driver:
    def __init__(self, model, config: EngineConfig, runner=None, sampler=None):
        """`runner` and `sampler` default to the device ones; tests of the scheduling pass
        stand-ins with the same `step`/`sample` methods."""
        self.model, self.config = model, config
        self.max_num_seqs, self.max_model_len = config.max_num_seqs, config.max_model_len
        self.max_prefill_len, self.block_size = config.prompt_limit, config.block_size
        self.stats = EngineStats()
        pages = config.pool_pages
        if config.num_blocks is None and config.memory_fraction is not None:
            # the pool is sized from the memory that is free now (the weights are loaded already)
            probe = CacheManager(model.cache_needs(), config.block_size, 1, 1, False)
            itemsize = 4 if config.dtype == torch.float32 else 2
            free_bytes = torch.cuda.mem_get_info(torch.device(config.device))[0]
            pages = config.pages_for_memory(probe.bytes_per_page(itemsize), free_bytes)
        self.num_blocks = pages
        self.cache = CacheManager(model.cache_needs(), config.block_size, pages, config.max_num_seqs,
                                  config.prefix_cache)
        self.runner = runner if runner is not None else Runner(
            model, self.cache, config.device, config.dtype, max_model_len=config.max_model_len,
            cuda_graphs=config.cuda_graphs)
        self.scheduler = Scheduler(self.cache, config.max_tokens_per_step, config.max_model_len, config.prompt_limit,
                                   self.stats)
        self.sampler = sampler if sampler is not None else Sampler(config.device)
        self.requests: dict[int, Request] = {}
        self.id_lock = threading.Lock()
        self.step_lock = threading.Lock()          # the scheduler and the cache are touched under it only
        self.next_id = 0
        # The router reaches the driver through a weak reference: a strong one would close a cycle, and a driver that
        # only the cycle collector frees may be freed at any moment, in the middle of another driver's graph capture
        # (where destroying this driver's captured graphs is an error).  A driver that is dropped stops its thread.
        me = weakref.ref(self)
        self.router = EventRouter(lambda: step(me()) if me() is not None else [],
                                  lambda: me() is not None and has_work(me()))
        weakref.finalize(self, self.router.stop, False)
        self.ahead = None                  # the next step's plan, made while the device ran the last one
        self.host_tokens = None            # pinned memory that the sampled tokens come back to


def make_driver(model, max_num_seqs: int = 4, max_model_len: int = 2048, max_prefill_len: Optional[int] = None,
                block_size: int = 16, num_blocks: Optional[int] = None, dtype=None, runner=None, sampler=None,
                **more) -> Driver:
    """A driver for a loaded model.  `dtype` defaults to the model's compute dtype and must
    equal it.  `more`: max_tokens_per_step, prefix_cache, decode_split_size, cuda_graphs, memory_fraction (with
    num_blocks None the pool takes that share of the free device memory instead of the worst case)."""
    model_dtype = model.ctx.dtype
    dtype = parse_dtype(dtype) if dtype is not None else model_dtype
    if dtype != model_dtype:
        raise ValueError(f"the model was loaded as {model_dtype}, the driver was asked for {dtype}")
    more.setdefault("decode_split_size", model.ctx.decode_split_size)
    if more["decode_split_size"] != model.ctx.decode_split_size:
        raise ValueError("decode_split_size is fixed when the model is loaded")
    cfg = EngineConfig(dtype=dtype, max_num_seqs=max_num_seqs, max_model_len=max_model_len,
                       max_prefill_len=max_prefill_len, block_size=block_size, num_blocks=num_blocks,
                       device=str(model.ctx.device), **more)
    return Driver(model, cfg, runner=runner, sampler=sampler)


def add_request(driver: Driver, prompt_ids, sampling: Optional[SamplingParams] = None) -> int:
    driver.router.raise_if_failed()
    sp = sampling or SamplingParams()
    prompt = [int(t) for t in prompt_ids]
    vocab = driver.model.spec.vocab_size
    if any(t < 0 or t >= vocab for t in prompt):
        raise ValueError(f"prompt holds token ids outside [0, {vocab})")
    driver.scheduler.validate(prompt, sp)
    with driver.id_lock:
        rid = driver.next_id
        driver.next_id += 1
    req = Request(request_id=rid, prompt_ids=prompt, sampling=sp, arrival=time.perf_counter())
    driver.router.open(rid)
    with driver.step_lock:
        driver.requests[rid] = req
        driver.scheduler.add(req)
    driver.router.wake()
    return rid


def has_work(driver: Driver) -> bool:
    return driver.scheduler.has_work()


def step(driver: Driver) -> list:
    """One scheduler iteration: at most one batch on the device; returns its StepEvents."""
    driver.router.raise_if_failed()
    with driver.step_lock:
        return _step_locked(driver)


def _step_locked(driver: Driver) -> list:
    sched = driver.scheduler
    ahead, driver.ahead = driver.ahead, None
    plan = sched.take_ahead(ahead) or sched.schedule()
    if not plan:
        return []
    entries = [StepEntry(driver.cache.live[s.request.request_id], s.tokens, (len(s.tokens) - 1,) if s.wants_logits else ())
               for s in plan]
    sampled = [s for s in plan if s.wants_logits]
    temps = [s.request.sampling.temperature for s in sampled]
    seeds = [s.request.sampling.seed if s.request.sampling.seed is not None else s.request.request_id for s in sampled]
    counters = [len(s.request.output_ids) for s in sampled]
    # a decode-only step samples inside its replayed graph; any other step hands back logits for the sampler
    fused = getattr(driver.runner, "step_sampled", None)
    both = fused(entries, temps, seeds, counters) if fused is not None and len(sampled) == len(plan) else None
    logits = driver.runner.step(entries) if both is None else None
    sched.committed(plan)
    st = driver.stats
    st.steps += 1
    st.last_step_tokens = sum(len(e.tokens) for e in entries)
    st.max_step_tokens = max(st.max_step_tokens, st.last_step_tokens)
    if driver.cache.groups:
        st.pages_total = driver.cache.num_pages
        st.pages_in_use = max(driver.cache.num_pages - g.pool.num_free for g in driver.cache.groups)
        st.max_pages_in_use = max(st.max_pages_in_use, st.pages_in_use)
    events: list = []
    if not sampled:
        return events
    if both is None:
        tokens = driver.sampler.sample(logits, temps, seeds, counters)
        both = torch.cat([tokens, driver.runner.status_word()])          # one copy back
    arrived = None
    if both.is_cuda:
        # the copy is on its way while the host plans the next step; waiting for it also synchronises
        if driver.host_tokens is None or driver.host_tokens.numel() < both.numel():
            driver.host_tokens = torch.empty(max(both.numel(), 64), dtype=both.dtype, pin_memory=True)
        back = driver.host_tokens[:both.numel()]
        back.copy_(both, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record()
        both = back
    driver.ahead = sched.plan_ahead(plan)
    if driver.ahead is not None and fused is not None:
        # its layout goes into the staging buffer now too; only the tokens are missing
        driver.runner.prefill_ahead([StepEntry(driver.cache.live[s.request.request_id], [0], (0,)) for s in driver.ahead[1]],
                                    temps, seeds, [c + 1 for c in counters])
    if arrived is not None:
        arrived.synchronize()
    both = both.tolist()
    toks, status = both[:-1], both[-1]
    if status:
        driver.runner.clear_status()
        from ..ops import raise_on_status
        raise_on_status(status)
    now = time.perf_counter()
    for s, tok in zip(sampled, toks):
        req = s.request
        req.output_ids.append(int(tok))
        if req.first_token_time is None:
            req.first_token_time = now
        driver.stats.emitted_tokens += 1
        done = len(req.output_ids) >= req.sampling.max_new_tokens or req.sampling.stops_at(int(tok))
        if done:
            sched.finish(req)
        events.append(StepEvent(req.request_id, int(tok), done))
    return events


def generate(driver: Driver, prompts, sampling=None) -> list:
    """Runs the prompts (lists of token ids) to completion; returns the generated token ids of
    each, in order.  `sampling`: one SamplingParams for all, or one per prompt."""
    if sampling is None or isinstance(sampling, SamplingParams):
        sampling = [sampling] * len(prompts)
    ids = [add_request(driver, p, sp) for p, sp in zip(prompts, sampling)]
    reqs = [driver.requests[i] for i in ids]
    while any(not r.finished for r in reqs):
        if not step(driver) and not has_work(driver):
            break
    for i in ids:
        driver.router.close(i)
        driver.requests.pop(i, None)
    return [list(r.output_ids) for r in reqs]


# --------------------------------------------------------------- streams and thread
def stream(driver: Driver, request_id: int) -> Iterator[StepEvent]:
    """The events of one request, until the one that finishes it.  With the background thread running they come
    from the thread; without one, the reader steps the engine itself (see engine/background.py)."""
    driver.router.raise_if_failed()
    for ev in driver.router.events(request_id):
        yield ev
    driver.requests.pop(request_id, None)


def start(driver: Driver) -> None:
    """Starts the background thread that steps the engine whenever there is work."""
    driver.router.start()


def stop(driver: Driver, join: bool = True) -> None:
    driver.router.stop(join)


def prewarm(driver: Driver) -> float:
    """Compiles what the model needs, runs one tiny batch and captures the decode graphs of every batch size up
    to `max_num_seqs`, so that no request pays for it (the reference compiles its shape buckets here,
    jllm/engine/engine.py:112-150).  Returns the seconds it took."""
    t0 = time.perf_counter()
    with driver.step_lock:
        driver.ahead = None
        driver.runner.warm_up(decode_batches=driver.max_num_seqs)
    return time.perf_counter() - t0
