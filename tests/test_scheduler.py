"""The scheduler's decisions, with a stand-in for the device (no GPU): admission, the token
budget, portions, decoding first, finishing and freeing, and what happens when pages run
out.  The stand-in checks that every request's tokens reach it exactly once and in order."""

import pytest
import torch

from jax_vllm_b200 import registry
from jax_vllm_b200.engine import SamplingParams, add_request, generate, has_work, make_driver, step
from jax_vllm_b200.engine import engine as eng
from jax_vllm_b200.parts import BuildContext, Model
from tests.util import TINY_A

VOCAB = TINY_A["vocab_size"]


def next_token(seq):
    return (sum(seq) * 31 + len(seq) * 7) % VOCAB


class FakeRunner:
    """Returns one-hot logits at next_token(everything the request was fed so far)."""

    def __init__(self):
        self.fed = {}
        self.batches = []

    def step(self, entries):
        rows = []
        self.batches.append([(e.cache.request_id, len(e.tokens), tuple(e.want)) for e in entries])
        for e in entries:
            seq = self.fed.setdefault(e.cache.request_id, [])
            if e.cache.num_tokens > len(seq):     # tokens taken over from another request's pages
                assert e.cache.tokens[:len(seq)] == seq
                seq[:] = e.cache.tokens[:e.cache.num_tokens]
            assert e.cache.num_tokens <= len(seq), "tokens were skipped"
            del seq[e.cache.num_tokens:]          # a preempted request starts again (after its cached prefix)
            seq.extend(e.tokens)
            for w in e.want:
                assert w == len(e.tokens) - 1
                row = torch.zeros(VOCAB)
                row[next_token(seq)] = 1.0
                rows.append(row)
        return torch.stack(rows) if rows else torch.zeros((0, VOCAB))

    def status_word(self):
        return torch.zeros(1, dtype=torch.int32)

    def clear_status(self):
        pass


class FakeSampler:
    def sample(self, logits, temperatures, seeds, counters):
        return logits.argmax(-1).to(torch.int32)


def expected(prompt, n, eos=None):
    seq, out = list(prompt), []
    for _ in range(n):
        t = next_token(seq)
        out.append(t); seq.append(t)
        if eos is not None and t == eos:
            break
    return out


def driver(**kw):
    model = Model(registry.config_from_dict(TINY_A).to_spec(), BuildContext(torch.float32, torch.device("cpu")))
    runner = FakeRunner()
    d = make_driver(model, runner=runner, sampler=FakeSampler(), **kw)
    return d, runner


def test_generates_what_the_stand_in_dictates_and_frees_everything():
    d, _ = driver(max_num_seqs=2, max_model_len=64, block_size=4)
    prompts = [[1, 2, 3], [9] * 17, [5], [7, 7]]
    outs = generate(d, prompts, SamplingParams(max_new_tokens=6))
    assert outs == [expected(p, 6) for p in prompts]
    assert not has_work(d) and not d.cache.live
    st = d.stats
    assert st.pages_total == d.cache.num_pages and 0 < st.max_pages_in_use <= st.pages_total
    assert 0 < st.last_step_tokens <= st.max_step_tokens <= d.config.max_tokens_per_step
    d.cache.check()
    assert d.stats.emitted_tokens == 24 and d.stats.finished == 4 and d.stats.admissions == 4


def test_budget_cuts_prompts_and_decodes_come_first():
    d, r = driver(max_num_seqs=3, max_model_len=64, block_size=4, max_tokens_per_step=8, prefix_cache=False)
    a = add_request(d, list(range(1, 4)), SamplingParams(max_new_tokens=4))      # 3 tokens
    step(d)
    assert r.batches[-1] == [(a, 3, (2,))]
    b = add_request(d, list(range(20)), SamplingParams(max_new_tokens=2))        # 20 tokens, cut to the budget
    step(d)
    assert r.batches[-1] == [(a, 1, (0,)), (b, 7, ())]                         # decode first, 7 = 8 - 1
    c = add_request(d, [4, 4], SamplingParams(max_new_tokens=2))
    step(d)
    assert r.batches[-1] == [(a, 1, (0,)), (b, 7, ())]                         # running portions before new requests
    step(d)
    assert r.batches[-1] == [(a, 1, (0,)), (b, 6, (5,)), (c, 1 + 0, ())] or \
        r.batches[-1] == [(a, 1, (0,)), (b, 6, (5,)), (c, 1, ())]
    while has_work(d):
        step(d)
    assert d.requests[b].output_ids == expected(list(range(20)), 2)
    assert d.requests[c].output_ids == expected([4, 4], 2)
    assert all(sum(n for _, n, _ in batch) <= 8 for batch in r.batches)


def test_first_token_comes_from_the_last_portion_and_eos_is_emitted():
    d, r = driver(max_num_seqs=1, max_model_len=64, block_size=4, max_tokens_per_step=5)
    prompt = list(range(11))
    free = expected(prompt, 8)
    eos = free[3]
    rid = add_request(d, prompt, SamplingParams(max_new_tokens=8, eos_id=eos))
    events = []
    while has_work(d):
        events += step(d)
    assert [b[0][1] for b in r.batches[:3]] == [5, 5, 1]
    assert [e.token for e in events] == free[: free.index(eos) + 1]
    assert [e.finished for e in events] == [False] * (len(events) - 1) + [True]
    assert events[0].request_id == rid


def test_stop_tokens_and_ignore_eos():
    d, _ = driver(max_num_seqs=2, max_model_len=64, block_size=4)
    prompt = [3, 1, 4, 1, 5]
    free = expected(prompt, 10)
    stop = free[4]
    first = free.index(stop)
    outs = generate(d, [prompt, prompt, prompt],
                    [SamplingParams(max_new_tokens=10, stop_token_ids=(stop, 999)),
                     SamplingParams(max_new_tokens=10, eos_id=stop, ignore_eos=True),
                     SamplingParams(max_new_tokens=10, eos_id=free[7], stop_token_ids=[stop])])
    assert outs == [free[:first + 1], free, free[:first + 1]]


def test_slots_limit_live_requests_first_come_first_served():
    d, r = driver(max_num_seqs=2, max_model_len=32, block_size=4)
    ids = [add_request(d, [i + 1] * 3, SamplingParams(max_new_tokens=3)) for i in range(5)]
    order = []
    while has_work(d):
        step(d)
        for rid, _, _ in r.batches[-1]:
            if rid not in order:
                order.append(rid)
        assert len(d.cache.live) <= 2
    assert order == ids


def test_request_that_can_never_fit_is_refused():
    d, _ = driver(max_num_seqs=2, max_model_len=64, block_size=4, num_blocks=5)
    with pytest.raises(ValueError, match="pages"):
        add_request(d, [1] * 16, SamplingParams(max_new_tokens=8))
    with pytest.raises(ValueError, match="max_model_len"):
        add_request(d, [1] * 60, SamplingParams(max_new_tokens=8))
    with pytest.raises(ValueError, match="empty"):
        add_request(d, [], SamplingParams())
    with pytest.raises(ValueError, match="token ids"):
        add_request(d, [VOCAB], SamplingParams())
    d2, _ = driver(max_num_seqs=2, max_model_len=64, max_prefill_len=8, block_size=4)
    with pytest.raises(ValueError, match="max_prefill_len"):
        add_request(d2, [1] * 9, SamplingParams(max_new_tokens=1))


@pytest.mark.parametrize("prefix_cache", [False, True])
def test_pages_run_out_youngest_is_preempted_and_tokens_stay_the_same(prefix_cache):
    # 6 pages of 4 tokens; two requests of 6 + 10 tokens each need 8 pages together
    d, r = driver(max_num_seqs=2, max_model_len=16, block_size=4, num_blocks=6, prefix_cache=prefix_cache)
    prompts = [[1, 2, 3, 4, 5, 6], [6, 5, 4, 3, 2, 1]]
    outs = generate(d, prompts, SamplingParams(max_new_tokens=10))
    assert outs == [expected(p, 10) for p in prompts]
    assert d.stats.preemptions >= 1
    d.cache.check()
    assert d.cache.groups[0].pool.num_free == 6
    # the older request was never preempted: it was fed each token exactly once
    fed_first = sum(n for batch in r.batches for rid, n, _ in batch if rid == 0)
    assert fed_first == 6 + 10 - 1


def test_the_next_decode_step_is_planned_under_the_running_one():
    d, r = driver(max_num_seqs=3, max_model_len=64, block_size=4, prefix_cache=False)
    sched = d.scheduler
    a = add_request(d, [1, 2, 3], SamplingParams(max_new_tokens=6))
    b = add_request(d, [4, 5, 6, 7, 8], SamplingParams(max_new_tokens=3))
    step(d)                                         # both prompts; both decode next and nobody waits
    assert d.ahead is not None and [s.request.request_id for s in d.ahead[1]] == [a, b]
    assert all(s.tokens is None for s in d.ahead[1])
    loops = d.stats.scheduler_loops
    step(d)
    assert r.batches[-1] == [(a, 1, (0,)), (b, 1, (0,))] and d.stats.scheduler_loops == loops + 1
    # a request that arrives makes the plan stale: the step is planned in the ordinary way, with the newcomer
    stale = d.ahead
    c = add_request(d, [9, 9], SamplingParams(max_new_tokens=2))
    assert sched.take_ahead(stale) is None
    step(d)
    assert r.batches[-1] == [(a, 1, (0,)), (b, 1, (0,)), (c, 2, (1,))]
    # b has its three tokens now: a request that finishes drops the plan too
    assert d.requests[b].finished and d.ahead is not None and sched.take_ahead(d.ahead) is None
    while has_work(d):
        step(d)
    assert d.requests[a].output_ids == expected([1, 2, 3], 6)
    assert d.requests[b].output_ids == expected([4, 5, 6, 7, 8], 3)
    assert d.requests[c].output_ids == expected([9, 9], 2)
    d.cache.check()
    assert not d.cache.live


def test_no_plan_ahead_when_it_would_take_pages_from_another():
    # 4 pages of 4 tokens; two requests at 8 tokens each hold them all, the ninth token needs a fifth page
    d, r = driver(max_num_seqs=2, max_model_len=16, block_size=4, num_blocks=4, prefix_cache=False)
    prompts = [[1] * 7, [2] * 7]
    ids = [add_request(d, p, SamplingParams(max_new_tokens=6)) for p in prompts]
    step(d)                                         # prompts: 7 tokens each, 2 pages each, the 8th fits
    assert d.ahead is not None
    step(d)                                         # 8 tokens each: the next token needs a page that is not there
    assert d.ahead is None and d.stats.preemptions == 0
    while has_work(d):
        step(d)
    assert d.stats.preemptions >= 1                 # decided by the ordinary plan, not by the one made ahead
    assert [d.requests[i].output_ids for i in ids] == [expected(p, 6) for p in prompts]
    d.cache.check()


def test_prompt_portion_waits_for_pages_instead_of_preempting():
    d, r = driver(max_num_seqs=2, max_model_len=24, block_size=4, num_blocks=6, max_tokens_per_step=64,
                  prefix_cache=False)
    a = add_request(d, [1] * 12, SamplingParams(max_new_tokens=4))      # 3 pages now, 4 at the end
    step(d)
    b = add_request(d, [2] * 14, SamplingParams(max_new_tokens=2))      # needs 4 pages: only 3 are free
    step(d)
    assert [x[0] for x in r.batches[-1]] == [a]                        # b is not admitted yet
    while has_work(d):
        step(d)
    assert d.requests[b].output_ids == expected([2] * 14, 2) and d.stats.preemptions == 0


def test_prefix_hits_skip_work():
    d, r = driver(max_num_seqs=2, max_model_len=64, block_size=4)
    p = list(range(30, 43))                                             # 13 tokens: 3 full pages
    first = generate(d, [p], SamplingParams(max_new_tokens=3))[0]
    n_batches = len(r.batches)
    second = generate(d, [p], SamplingParams(max_new_tokens=3))[0]
    assert first == second == expected(p, 3)
    assert r.batches[n_batches][0][1] == 1                              # 12 tokens came from the cache
    assert d.stats.cache_hit_blocks == 3 and d.stats.cache_hit_tokens == 12


class FailingRunner(FakeRunner):
    """The stand-in device, whose step raises from its `fail_at`-th call on."""

    def __init__(self, fail_at, error):
        super().__init__()
        self.fail_at, self.error, self.calls = fail_at, error, 0

    def step(self, entries):
        self.calls += 1
        if self.calls >= self.fail_at:
            raise self.error
        return super().step(entries)


def failing_driver(fail_at, error, **kw):
    model = Model(registry.config_from_dict(TINY_A).to_spec(), BuildContext(torch.float32, torch.device("cpu")))
    runner = FailingRunner(fail_at, error)
    return make_driver(model, runner=runner, sampler=FakeSampler(), **kw), runner


def test_an_exception_inside_the_background_thread_reaches_every_caller():
    """The third step raises inside the thread (as jllm's tests make its loop raise, tests/test_scheduler.py:335-366):
    the thread ends, the reader of a stream gets the error after the events that were delivered before it, a
    second reader and `add_request` and `step` get it too, and `stop` still joins."""
    from jax_vllm_b200.engine.background import EngineFailed
    d, runner = failing_driver(3, RuntimeError("boom in step three"), max_num_seqs=2, max_model_len=32, block_size=4)
    a = add_request(d, [1, 2, 3], SamplingParams(max_new_tokens=8))
    b = add_request(d, [4, 5], SamplingParams(max_new_tokens=8))
    eng.start(d)
    try:
        got = []
        with pytest.raises(EngineFailed, match="RuntimeError: boom in step three"):
            for ev in eng.stream(d, a):
                got.append(ev.token)
        assert got == expected([1, 2, 3], 8)[:len(got)] and len(got) == 2          # steps one and two delivered
        with pytest.raises(EngineFailed, match="boom in step three"):
            list(eng.stream(d, b))
        with pytest.raises(EngineFailed):
            add_request(d, [1], SamplingParams())
        with pytest.raises(EngineFailed):
            step(d)
        assert not d.router.running
    finally:
        eng.stop(d)                       # joins a thread that has already ended
    assert runner.calls == 3
    # starting again clears the latch; the stand-in keeps failing, so the next error is latched in turn
    eng.start(d)
    with pytest.raises(EngineFailed):
        list(eng.stream(d, b))
    eng.stop(d)


def test_the_allocator_running_dry_inside_the_thread_is_latched_too():
    from jax_vllm_b200.cache.page_pool import OutOfPages
    from jax_vllm_b200.engine.background import EngineFailed
    d, _ = failing_driver(2, OutOfPages("no free pages"), max_num_seqs=1, max_model_len=16, block_size=4)
    a = add_request(d, [1, 2, 3], SamplingParams(max_new_tokens=4))
    eng.start(d)
    try:
        with pytest.raises(EngineFailed, match="OutOfPages: no free pages"):
            list(eng.stream(d, a))
    finally:
        eng.stop(d)


def test_streams_without_a_thread_and_after_a_stop():
    """Without a background thread the reader of a stream drives the engine itself; the events of the other
    request wait in its queue.  A stream read after `stop` with its request unfinished says so."""
    d, _ = driver(max_num_seqs=2, max_model_len=32, block_size=4)
    a = add_request(d, [1, 2], SamplingParams(max_new_tokens=5))
    b = add_request(d, [3], SamplingParams(max_new_tokens=3))
    assert [ev.token for ev in eng.stream(d, a)] == expected([1, 2], 5)
    assert [ev.token for ev in eng.stream(d, b)] == expected([3], 3)
    with pytest.raises(KeyError, match="no events to read"):
        list(eng.stream(d, a))
    eng.start(d)
    eng.stop(d)
    c = add_request(d, [9, 9, 9], SamplingParams(max_new_tokens=2))
    with pytest.raises(RuntimeError, match="stopped with request"):
        list(eng.stream(d, c))


def test_background_thread_streams_events():
    d, _ = driver(max_num_seqs=2, max_model_len=32, block_size=4)
    eng.start(d)
    try:
        ids = [add_request(d, [i + 1, 2], SamplingParams(max_new_tokens=4)) for i in range(3)]
        got = {i: [ev.token for ev in eng.stream(d, i)] for i in ids}
    finally:
        eng.stop(d)
    assert got == {i: expected([i + 1, 2], 4) for i in range(3)}
