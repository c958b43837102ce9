"""Generation through the entry point on the GPU: greedy tokens equal the plain
implementation's, alone and batched, through prompt portions, preemption and prefix reuse;
temperature sampling is reproducible and does not depend on the batch; long decoding; the
first tokens of a sequence."""

import pytest
import torch

from tests.plain.qwen3_plain import PlainModel
from tests.util import PAGE_SIZE, TINY, make_folder, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["a", "b", "d"])
def setup(request, tmp_path_factory):
    tag = request.param
    folder = make_folder(tmp_path_factory.mktemp(f"gen_{tag}"), tag, seed=5)
    return tag, folder, PlainModel(folder)


def load(folder, dtype):
    from jax_vllm_b200 import load_from_path
    return load_from_path(folder, dtype=dtype)


def test_greedy_equals_plain_alone_batched_and_chunked(setup):
    from jax_vllm_b200 import SamplingParams, generate, make_driver
    tag, folder, plain = setup
    vocab = TINY[tag]["vocab_size"]
    prompts = [random_tokens(n, vocab, seed=20 + n) for n in (5, 17, 33, 1, 40)]
    want = [plain.greedy(p, 8) for p in prompts]
    model = load(folder, "fp32")
    sp = SamplingParams(max_new_tokens=8)
    solo = make_driver(model, max_num_seqs=1, max_model_len=64, block_size=PAGE_SIZE[tag])
    assert [generate(solo, [p], sp)[0] for p in prompts] == want
    batched = make_driver(model, max_num_seqs=4, max_model_len=64, block_size=PAGE_SIZE[tag])
    assert generate(batched, prompts, sp) == want
    chunked = make_driver(model, max_num_seqs=3, max_model_len=64, block_size=PAGE_SIZE[tag], max_tokens_per_step=7)
    assert generate(chunked, prompts, sp) == want
    assert chunked.stats.steps > batched.stats.steps
    for d in (solo, batched, chunked):
        d.cache.check()
        assert not d.cache.live


def test_bf16_greedy_follows_plain_where_the_choice_is_clear(setup):
    """In bfloat16 the engine must pick the plain implementation's token wherever the plain top-1
    leads the runner-up by more than the bfloat16 error bound (3 % of the largest logit)."""
    from jax_vllm_b200 import SamplingParams, generate, make_driver
    tag, folder, plain = setup
    vocab = TINY[tag]["vocab_size"]
    model = load(folder, "bf16")
    d = make_driver(model, max_num_seqs=2, max_model_len=64, block_size=PAGE_SIZE[tag])
    checked = 0
    for seed in range(6):
        p = random_tokens(12, vocab, seed=40 + seed)
        got = generate(d, [p], SamplingParams(max_new_tokens=6))[0]
        seq = list(p)
        for tok in got:
            logits = plain.logits(seq)[-1]
            top = logits.topk(2).values
            if (top[0] - top[1]).item() > 0.06 * logits.abs().max().item():
                assert tok == int(logits.argmax())
                checked += 1
            seq.append(tok)
    assert checked >= 10


def test_preemption_and_prefix_reuse_leave_tokens_unchanged(setup):
    from jax_vllm_b200 import SamplingParams, generate, make_driver
    tag, folder, plain = setup
    vocab, P = TINY[tag]["vocab_size"], PAGE_SIZE[tag]
    shared = random_tokens(2 * P, vocab, seed=70)
    prompts = [shared + random_tokens(P // 2 + 1, vocab, seed=71), shared + random_tokens(P + 1, vocab, seed=72),
               random_tokens(2 * P + 3, vocab, seed=73)]
    want = [plain.greedy(p, 2 * P) for p in prompts]
    model = load(folder, "fp32")
    sp = SamplingParams(max_new_tokens=2 * P)
    # each request ends with more than 4P tokens (5 or 6 pages); 10 pages cannot hold all three to the end
    tight = make_driver(model, max_num_seqs=3, max_model_len=6 * P, block_size=P, num_blocks=10)
    assert generate(tight, prompts, sp) == want
    assert tight.stats.preemptions >= 1
    tight.cache.check()
    roomy = make_driver(model, max_num_seqs=3, max_model_len=6 * P, block_size=P)
    assert generate(roomy, prompts[:1], sp) == want[:1]
    assert generate(roomy, prompts, sp) == want
    assert roomy.stats.cache_hit_tokens >= 2 * P + 2 * P      # the same prompt again, and the shared prefix
    no_reuse = make_driver(model, max_num_seqs=3, max_model_len=6 * P, block_size=P, prefix_cache=False)
    assert generate(no_reuse, prompts, sp) == want and no_reuse.stats.cache_hit_tokens == 0


def test_temperature_sampling_is_reproducible_and_batch_independent(setup):
    from jax_vllm_b200 import SamplingParams, generate, make_driver
    tag, folder, _ = setup
    vocab = TINY[tag]["vocab_size"]
    model = load(folder, "fp32")
    prompts = [random_tokens(n, vocab, seed=80 + n) for n in (1, 9, 40, 23, 7)]
    sps = [SamplingParams(max_new_tokens=12, temperature=0.8, seed=4 + i) for i in range(5)]
    a = make_driver(model, max_num_seqs=1, max_model_len=64, block_size=PAGE_SIZE[tag])
    solo = [generate(a, [p], sp)[0] for p, sp in zip(prompts, sps)]
    b = make_driver(model, max_num_seqs=4, max_model_len=64, block_size=PAGE_SIZE[tag], max_tokens_per_step=7)
    assert generate(b, prompts, sps) == solo
    greedy = generate(b, prompts, SamplingParams(max_new_tokens=12))
    assert greedy != solo
    other = generate(b, prompts, [SamplingParams(max_new_tokens=12, temperature=0.8, seed=99 + i) for i in range(5)])
    assert other != solo


def test_long_decoding_and_first_tokens(setup):
    """Two hundred tokens decoded one by one (crossing many pages and several splits) equal the
    plain implementation's logits; so do the logits of the very first positions."""
    from jax_vllm_b200.cache import CacheManager
    from jax_vllm_b200.engine import Runner, StepEntry
    tag, folder, plain = setup
    vocab, P = TINY[tag]["vocab_size"], PAGE_SIZE[tag]
    toks = random_tokens(230, vocab, seed=90)
    want = plain.logits(toks)
    from jax_vllm_b200 import load_from_path
    model = load_from_path(folder, dtype="fp32", decode_split_size=48)
    cache = CacheManager(model.cache_needs(), P, -(-230 // P), 2, prefix_cache=False)
    runner = Runner(model, cache, "cuda:0", torch.float32)
    rc = cache.admit("x")
    first = runner.run([StepEntry(rc, toks[:3], (0, 1, 2))]).cpu()
    lim = 1e-4 * max(1.0, want.abs().max().item())
    assert (first - want[:3]).abs().max().item() <= lim
    for i in range(3, 230):
        row = runner.run([StepEntry(rc, [toks[i]], (0,))]).cpu()[0]
        assert (row - want[i]).abs().max().item() <= lim, f"position {i}"
    runner.check_kernels()


def test_layers_of_the_benchmarked_size_in_bfloat16_follow_the_32_bit_path(tmp_path):
    """Two layers with the widths that the kernels are tuned for (4,096 wide, 32/8 heads of 128, feed-forward
    12,288): a prompt long enough for the product with the gate in its epilogue and the 128-row attention
    tiles, then single tokens through the replayed graph (persistent decode attention that prepares its own
    queries and keys, products whose k is cut into parts).  The bfloat16 engine must stay within the bfloat16
    bound of the same engine in true 32-bit on the same weights, position by position."""
    from jax_vllm_b200 import load_from_path, registry, write_model_folder
    from jax_vllm_b200.engine import StepEntry, make_driver
    cfg = dict(architectures=["Qwen3ForCausalLM"], vocab_size=2048, hidden_size=4096, intermediate_size=12288,
               num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
               rope_theta=1e6, max_position_embeddings=4096, tie_word_embeddings=False)
    folder = write_model_folder(tmp_path / "wide", registry.config_from_dict(cfg), seed=7)
    lens, n_new = (1100, 300, 37), 24
    seqs = [random_tokens(n + n_new, 2048, seed=90 + i) for i, n in enumerate(lens)]
    logits = {}
    for dtype in ("fp32", "bf16"):
        model = load_from_path(folder, dtype=dtype)
        d = make_driver(model, max_num_seqs=3, max_model_len=1280, block_size=16, prefix_cache=False,
                        max_tokens_per_step=2048)
        rcs = [d.cache.admit(i) for i in range(len(lens))]
        rows = [d.runner.run([StepEntry(rc, s[:n], (n - 1,))]).float().cpu() for rc, s, n in zip(rcs, seqs, lens)]
        for i in range(n_new):       # the three requests side by side, one token each
            rows.append(d.runner.run([StepEntry(rc, s[n + i:n + i + 1], (0,)) for rc, s, n in zip(rcs, seqs, lens)]).float().cpu())
        d.runner.check_kernels()
        logits[dtype] = torch.cat(rows)
        if dtype == "bf16":
            assert d.runner.graphs, "single tokens were not replayed from a graph"
        for i in range(len(lens)):
            d.cache.release(i)
        del d, model
        torch.cuda.empty_cache()
    want, got = logits["fp32"], logits["bf16"]
    assert want.abs().max() > 1.0
    lim = 3e-2 * max(1.0, want.abs().max().item())
    assert (got - want).abs().max().item() <= lim
    # and the 32-bit path at these widths against the plain implementation (on the CPU): the shortest request,
    # its prompt's last position and every decoded position
    plain = PlainModel(folder)
    n = lens[2]
    oracle = plain.logits(seqs[2])[n - 1:]
    mine = torch.cat([want[2:3]] + [want[3 + 3 * i + 2:3 + 3 * i + 3] for i in range(n_new)])
    assert (mine - oracle).abs().max().item() <= 1e-4 * max(1.0, oracle.abs().max().item())


def test_command_line_generates_what_plain_generates(setup):
    """cli.py as a user runs it: a model folder, prompts as token ids, 32-bit; the printed token ids are the
    plain implementation's greedy continuation."""
    import json, os, subprocess, sys
    from pathlib import Path
    tag, folder, plain = setup
    vocab = TINY[tag]["vocab_size"]
    prompts = [random_tokens(9, vocab, seed=130), random_tokens(21, vocab, seed=131)]
    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, str(root / "cli.py"), "--model-path", str(folder), "--dtype", "fp32", "--max-tokens", "6",
           "--max-model-len", "64", "--block-size", str(PAGE_SIZE[tag])]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(root), env=dict(os.environ))
    assert out.returncode == 0, out.stderr[-2000:]
    got = [json.loads(line)["output_ids"] for line in out.stdout.splitlines() if line.startswith("{")]
    assert got == [plain.greedy(p, 6) for p in prompts]


def test_llm_class_and_background_thread_on_the_device(setup):
    """The convenience class, and the entry point's background thread with streams (start, stream, stop), give
    the plain greedy continuation."""
    from jax_vllm_b200 import LLM, SamplingParams, add_request, start, stop, stream
    tag, folder, plain = setup
    vocab = TINY[tag]["vocab_size"]
    prompts = [random_tokens(7, vocab, seed=140), random_tokens(18, vocab, seed=141)]
    want = [plain.greedy(p, 5) for p in prompts]
    llm = LLM(folder, dtype="fp32", max_num_seqs=2, max_model_len=64, block_size=PAGE_SIZE[tag])
    assert llm.generate(prompts, SamplingParams(max_new_tokens=5)) == want
    assert not llm.has_work() and llm.stats.finished == 2
    start(llm.driver)
    try:
        ids = [add_request(llm.driver, p, SamplingParams(max_new_tokens=5)) for p in prompts]
        got = [[ev.token for ev in stream(llm.driver, i)] for i in ids]
    finally:
        stop(llm.driver)
    assert got == want
    llm.driver.cache.check()


def test_replayed_graphs_and_planning_ahead_change_no_token(tmp_path):
    """Many requests of mixed lengths in bfloat16 on the configuration that takes the tcgen05 kernels, with few
    pages (requests are preempted) and more requests than slots: the engine with replayed decode graphs, sampling
    inside the graph and the next step planned ahead gives exactly the tokens of the same engine stepping
    eagerly.  Same kernels, same schedule: any difference is a fault of the machinery around them."""
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    folder = make_folder(tmp_path / "c", "c", seed=21)
    vocab, P = TINY["c"]["vocab_size"], PAGE_SIZE["c"]
    model = load_from_path(folder, dtype="bf16")
    lens = [5, 140, 33, 270, 18, 64, 129, 7, 200, 90, 31, 256]
    prompts = [random_tokens(n, vocab, seed=300 + i) for i, n in enumerate(lens)]
    sps = [SamplingParams(max_new_tokens=24 + (i % 5) * 9, temperature=0.0 if i % 3 else 0.7, seed=11 + i)
           for i in range(len(prompts))]
    outs = []
    for graphs in (False, True):
        d = make_driver(model, max_num_seqs=4, max_model_len=352, block_size=P, num_blocks=30, cuda_graphs=graphs,
                        max_tokens_per_step=192)
        outs.append(generate(d, prompts, sps))
        d.cache.check()
        assert not d.cache.live and d.stats.finished == len(prompts)
        if graphs:
            assert d.runner.graphs_sampled, "no decode step was replayed with its sampling"
            assert d.stats.preemptions >= 1
    assert outs[0] == outs[1]
    assert [len(o) for o in outs[1]] == [sp.max_new_tokens for sp in sps]


def test_prewarm_captures_the_decode_graphs_and_changes_nothing(tmp_path):
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver, prewarm
    folder = make_folder(tmp_path / "c", "c", seed=33)
    vocab, P = TINY["c"]["vocab_size"], PAGE_SIZE["c"]
    model = load_from_path(folder, dtype="bf16")
    prompts = [random_tokens(n, vocab, seed=400 + n) for n in (9, 40, 3)]
    sp = SamplingParams(max_new_tokens=12)
    cold = make_driver(model, max_num_seqs=3, max_model_len=96, block_size=P)
    want = generate(cold, prompts, sp)
    warm = make_driver(model, max_num_seqs=3, max_model_len=96, block_size=P)
    assert prewarm(warm) > 0
    assert sorted(warm.runner.graphs_sampled) == [1, 2, 3]
    warm.cache.check()
    assert not warm.cache.live and warm.cache.groups[0].pool.num_free == warm.cache.num_pages
    assert generate(warm, prompts, sp) == want


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_many_requests_at_once(setup, dtype):
    """Twenty-four requests decode together, with CUDA graphs: batches of 9 and more rows take other kernels than
    small ones (the tcgen05 product for larger batches, the decode attention over many requests).  32-bit tokens
    equal the plain implementation's; bfloat16 tokens equal it wherever the plain choice is clear."""
    from jax_vllm_b200 import SamplingParams, generate, make_driver, prewarm
    tag, folder, plain = setup
    vocab, P = TINY[tag]["vocab_size"], PAGE_SIZE[tag]
    new = 6
    prompts = [random_tokens(3 + (7 * i) % 23, vocab, seed=300 + i) for i in range(24)]
    model = load(folder, dtype)
    d = make_driver(model, max_num_seqs=24, max_model_len=-(-(26 + new) // P) * P, block_size=P, prefix_cache=False)
    prewarm(d)
    got = generate(d, prompts, SamplingParams(max_new_tokens=new))
    assert d.stats.steps < 24 * new                      # they did run together
    d.cache.check()
    assert not d.cache.live
    checked = 0
    for p, out in zip(prompts, got):
        assert len(out) == new
        if dtype == "fp32":
            assert out == plain.greedy(p, new)
            continue
        seq = list(p)
        for tok in out:
            logits = plain.logits(seq)[-1]
            top = logits.topk(2).values
            if (top[0] - top[1]).item() > 0.06 * logits.abs().max().item():
                assert tok == int(logits.argmax())
                checked += 1
            seq.append(tok)
    assert dtype == "fp32" or checked >= 40


def test_pool_sized_from_the_free_memory(setup):
    """`memory_fraction` instead of a page count: the pool gets what fits into that share of the memory that is free
    (here a share so small that it is fewer pages than the worst case), and generation goes on as ever."""
    from jax_vllm_b200 import SamplingParams, generate, make_driver
    tag, folder, plain = setup
    vocab, P = TINY[tag]["vocab_size"], PAGE_SIZE[tag]
    model = load(folder, "fp32")
    roomy = make_driver(model, max_num_seqs=3, max_model_len=8 * P, block_size=P)
    assert roomy.num_blocks == 24
    per_page = roomy.cache.bytes_per_page(4)
    free = torch.cuda.mem_get_info()[0]
    tight = make_driver(model, max_num_seqs=3, max_model_len=8 * P, block_size=P, memory_fraction=10.5 * per_page / free)
    assert tight.num_blocks == tight.cache.num_pages == 10
    prompts = [random_tokens(2 * P + 1, vocab, seed=500 + i) for i in range(3)]
    sp = SamplingParams(max_new_tokens=2 * P)
    assert generate(tight, prompts, sp) == generate(roomy, prompts, sp) == [plain.greedy(p, 2 * P) for p in prompts]
    assert tight.stats.preemptions >= 1
    with pytest.raises(MemoryError, match="one request of max_model_len"):
        make_driver(model, max_num_seqs=3, max_model_len=8 * P, block_size=P, memory_fraction=3.5 * per_page / free)
