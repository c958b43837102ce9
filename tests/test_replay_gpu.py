"""Trace replay against the plain implementation: the same requests whole, with the last 32
tokens one by one, in portions of changing size down to two tokens, and mixed with other
requests in a pool so small that pages are used again (with and without reuse of known
prefixes, eagerly and through the captured decode graph); in 32-bit and in bfloat16; for
tiny configurations that differ in every size, one of them with the head layout of the
benchmarked model.  The largest |difference| of every case is recorded and printed at the end
of the run (tests/conftest.py)."""

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.plain.qwen3_plain import PlainModel
from tests.util import PAGE_SIZE, TINY, collect, make_folder, portions, prefix_then_single, random_tokens, whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"a": [70, 45, 100, 33], "b": [90, 38, 64, 51], "c": [200, 70, 300, 130], "d": [61, 40, 83, 35],
           "e": [200, 70, 300, 130], "f": [180, 66, 270, 110]}
ABSOLUTE_UPTO = 50.0      # logits up to this size are held to 1e-4 absolute in 32-bit


def limits(dtype, want: torch.Tensor):
    """Largest allowed |difference| of logits.  32-bit: 1e-4 absolute while no logit of the request exceeds
    ABSOLUTE_UPTO in size (every configuration here: they reach 5 to 12), beyond that 1e-4 * size / ABSOLUTE_UPTO
    (a float32 of size 50 is spaced 4e-6).  bfloat16: 3 % of the largest logit (8 bits of mantissa through a few
    layers)."""
    size = want.abs().max().item()
    if dtype == "float32":
        return 1e-4 * max(1.0, size / ABSOLUTE_UPTO)
    return 3e-2 * max(1.0, size)


@pytest.fixture(scope="module", params=["a", "b", "c", "d", "e", "f"])
def setup(request, tmp_path_factory):
    tag = request.param
    folder = make_folder(tmp_path_factory.mktemp(f"model_{tag}"), tag, seed=3)
    plain = PlainModel(folder)           # the folder holds bfloat16 weights; both sides read the same values
    seqs = {f"r{i}": random_tokens(n, TINY[tag]["vocab_size"], seed=10 + i) for i, n in enumerate(LENGTHS[tag])}
    want = {rid: plain.logits(t) for rid, t in seqs.items()}
    assert all(w.abs().max() > 1.0 for w in want.values())     # logits of order one, not a flat model
    if tag in ("c", "e", "f"):
        # the product with the gate in its epilogue is taken from 1,024 rows on; these prompts are shorter, so
        # for this configuration the bar is lowered and portions of 17 tokens or more go through it
        from jax_vllm_b200.parts.feed_forward import GatedMLP
        before, GatedMLP.FUSED_GATE_ROWS = GatedMLP.FUSED_GATE_ROWS, 17
        yield tag, folder, seqs, want
        GatedMLP.FUSED_GATE_ROWS = before
        return
    yield tag, folder, seqs, want


def replay(folder, tag, dtype, steps, out_dir, max_tokens, **switches):
    from jax_vllm_b200.engine.replay import Replayer

    rep = Replayer(folder, dtype, out_dir, max_tokens=max_tokens, page_size=PAGE_SIZE[tag], **switches)
    rep.run_stream(json.dumps(s) for s in steps)
    rep.cache.check()
    assert not rep.cache.live
    for s in steps:       # what every step did is on disk beside its logits
        meta = json.loads((Path(out_dir) / f"{s['step']}.json").read_text())
        assert meta["step"] == s["step"] and meta["entries"] == len(s["entries"])
    return rep


def compare(steps, out_dir, vocab, want, dtype, case=None):
    """Every written row against the oracle's; returns what was read and the largest |difference|, which is
    recorded under `case` for the summary at the end of the run."""
    from tests.conftest import record_worst

    got = collect(steps, out_dir, vocab)
    worst, lim_of_worst = 0.0, 0.0
    for rid, rows in got.items():
        lim = limits(dtype, want[rid])
        for pos, row in rows.items():
            w = want[rid][pos]
            diff = (torch.from_numpy(row.copy()) - w).abs().max().item()
            assert diff <= lim, f"{rid} position {pos}: |diff| {diff:.3e} > {lim:.3e}"
            if diff >= worst:
                worst, lim_of_worst = diff, lim
            if dtype == "float32":
                assert int(row.argmax()) == int(w.argmax())
    assert worst <= lim_of_worst or not got
    if case is not None:
        record_worst(case, dtype, worst, lim_of_worst)
    return got, worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_request_alone_and_whole(setup, dtype, tmp_path):
    tag, folder, seqs, want = setup
    for rid, toks in seqs.items():
        steps = whole(rid, toks)
        out = tmp_path / rid
        replay(folder, tag, dtype, steps, out, max_tokens=320)
        got, _ = compare(steps, out, TINY[tag]["vocab_size"], want, dtype, case=f"{tag} whole")
        assert sorted(got[rid]) == list(range(len(toks)))


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graph"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_tokens_one_by_one(setup, dtype, graphs, tmp_path):
    """Most of a request in one step, then single tokens: stepped eagerly, and replayed from the captured
    graph that generation uses for such steps (the first step at a batch size runs eagerly, the second is
    captured, the others replay it)."""
    tag, folder, seqs, want = setup
    for rid, toks in list(seqs.items())[:3]:
        steps = prefix_then_single(rid, toks, tail=32)
        out = tmp_path / rid
        rep = replay(folder, tag, dtype, steps, out, max_tokens=320, cuda_graphs=graphs)
        compare(steps, out, TINY[tag]["vocab_size"], want, dtype, case=f"{tag} last 32 one by one" + (", graph" if graphs else ""))
        replayed = sum(1 for m in rep.records if m["replayed_graph"])
        assert replayed == (31 if graphs else 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(7, 2, 13, 5, 2, 3), (2,), (16, 1, 15, 17), (31, 2, 33), (64, 3, 130, 2)])
def test_portions_of_changing_size(setup, dtype, sizes, tmp_path):
    tag, folder, seqs, want = setup
    rid, toks = "r2", seqs["r2"]
    steps = portions(rid, toks, sizes)
    replay(folder, tag, dtype, steps, tmp_path, max_tokens=320)
    got, _ = compare(steps, tmp_path, TINY[tag]["vocab_size"], want, dtype, case=f"{tag} portions {sizes}")
    assert sorted(got[rid]) == list(range(len(toks)))


REST = 1 << 20      # "all that is left of the request"
# A portion that fills at least one 128-row tile of the tcgen05 prompt attention (64 tokens with 2 query heads per
# kv head, 32 with 4, 25 with 5) for the configurations that take it, beside single tokens of other requests in the same step.
TILE_AND_MORE = {"c": (69, 130), "e": (37, 70), "f": (29, 55)}
FIRST_WANTED_OF_R4 = 33      # with prefix reuse r4's first portion wants its logits from here on (its start is r0's)


def mixed_trace(seqs, tag="a", reuse_prefix=False):
    """Up to four live requests; portions of some beside single tokens of others; requests
    end and new ones start, in a pool that the sum of all requests would overflow."""
    ids = list(seqs)
    fed = {r: 0 for r in ids}
    big, bigger = TILE_AND_MORE.get(tag, (24, 20))
    plan = [  # (request, tokens to feed) per step; a request may sit a step out
        [("r0", 9), ("r1", 2)],
        [("r0", 1), ("r1", 17), ("r2", 5)],
        [("r0", 1), ("r1", 1), ("r2", 30), ("r3", 2)],
        [("r0", big), ("r1", 1), ("r3", 7)],      # a whole tile and more beside a single token and a short portion
        [("r0", 1), ("r1", 1), ("r2", 1), ("r3", 1)],
        [("r0", 1), ("r2", bigger), ("r1", 1)],  # two tiles beside two single tokens
        [("r1", REST), ("r0", REST)],            # both finish here: their pages go back
        [("r2", 3), ("r3", REST), ("r4", 40)],   # r4 and r5 repeat r0 and r1 in reused pages
        [("r2", 1), ("r4", 1), ("r5", 2)],
        [("r2", REST), ("r4", REST), ("r5", REST)],
    ]
    seqs = dict(seqs, r4=seqs["r0"], r5=seqs["r1"])
    fed.update(r4=0, r5=0)
    steps = []
    for i, row in enumerate(plan):
        entries, end = [], []
        for rid, n in row:
            toks = seqs[rid][fed[rid]:fed[rid] + n]
            if not toks:
                continue
            first = FIRST_WANTED_OF_R4 if reuse_prefix and rid == "r4" and fed[rid] == 0 else 0
            entries.append({"id": rid, "tokens": toks, "want": list(range(first, len(toks)))})
            fed[rid] += len(toks)
            if fed[rid] == len(seqs[rid]):
                end.append(rid)
        steps.append({"step": i, "entries": entries, "end": end})
    assert all(fed[r] == len(seqs[r]) for r in seqs)
    return steps, seqs


def pool_tokens(seqs):
    """The most tokens that live requests hold at any time in `mixed_trace`, each request's
    count rounded up to a multiple of 64: the first four requests together.  The whole trace
    needs more pages than that, so pages are used again."""
    return sum(-(-len(s) // 64) * 64 for s in list(seqs.values())[:4])


@pytest.mark.parametrize("reuse", [False, True], ids=["no reuse", "prefix reuse"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_requests_in_reused_pages(setup, dtype, reuse, tmp_path):
    tag, folder, seqs, want = setup
    steps, all_seqs = mixed_trace(seqs, tag, reuse_prefix=reuse)
    want = dict(want, r4=want["r0"], r5=want["r1"])
    rep = replay(folder, tag, dtype, steps, tmp_path, max_tokens=pool_tokens(seqs), prefix_cache=reuse)
    got, _ = compare(steps, tmp_path, TINY[tag]["vocab_size"], want, dtype,
                     case=f"{tag} mixed" + (", prefix reuse" if reuse else ""))
    first_of = {r: (FIRST_WANTED_OF_R4 if reuse and r == "r4" else 0) for r in all_seqs}
    assert all(sorted(got[r]) == list(range(first_of[r], len(all_seqs[r]))) for r in all_seqs)
    # pages were handed out again: afresh, or (with reuse) with what an earlier request had left in them
    assert rep.cache.stats["pages_allocated"] + rep.cache.stats["prefix_hit_pages"] > rep.cache.num_pages
    meta = {m["step"]: m for m in rep.records}
    assert sum(m["pages_allocated"] for m in rep.records) == rep.cache.stats["pages_allocated"]
    assert sum(m["pages_released"] for m in rep.records) == rep.cache.stats["pages_released"]
    assert meta[6]["pages_released"] > 0 and meta[6]["live_requests"] == 2      # r0 and r1 ended there
    hit = meta[7]["prefix_hit_tokens"]          # the step in which r4 arrives with r0's first tokens
    P = PAGE_SIZE[tag]
    assert hit == (FIRST_WANTED_OF_R4 // P * P if reuse else 0)
    assert hit == sum(m["prefix_hit_tokens"] for m in rep.records)
    if tag in TILE_AND_MORE and dtype == "bfloat16":
        # the step that this configuration is here for: whole tcgen05 prompt tiles and single tokens in one batch
        whole_tiles = lambda m: sum(n for k, n in m["tiles"].items() if k.startswith(f"{128 // GROUP[tag]} tokens"))
        assert whole_tiles(meta[3]) >= 2 and meta[3]["single_token_entries"] == 1
        assert whole_tiles(meta[5]) >= 3 and meta[5]["single_token_entries"] == 2


GROUP = {"c": 2, "e": 4, "f": 5}     # query heads per kv head of the configurations with head size 128


def test_schedules_agree_with_each_other_in_32_bit(setup, tmp_path):
    """Differences between ways of cutting are rounding only: far below the distance to the oracle's limit."""
    tag, folder, seqs, want = setup
    rid, toks = "r0", seqs["r0"]
    vocab = TINY[tag]["vocab_size"]
    a = whole(rid, toks); replay(folder, tag, "float32", a, tmp_path / "a", 320)
    b = portions(rid, toks, (3, 2, 11)); replay(folder, tag, "float32", b, tmp_path / "b", 320)
    ga, gb = collect(a, tmp_path / "a", vocab)[rid], collect(b, tmp_path / "b", vocab)[rid]
    worst = max(np.abs(ga[p] - gb[p]).max() for p in ga)
    assert worst <= 2e-5 * max(1.0, want[rid].abs().max().item())


def test_trace_run_program(setup, tmp_path):
    """bin/trace_run as a program: stdin steps, `done <step>` lines, files on disk, exit 0."""
    tag, folder, seqs, want = setup
    steps, all_seqs = mixed_trace(seqs, tag)
    env = dict(os.environ)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(tmp_path), "--max-tokens", str(pool_tokens(seqs)), "--page-size", str(PAGE_SIZE[tag])],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, env=env,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    compare(steps, tmp_path, TINY[tag]["vocab_size"], dict(want, r4=want["r0"], r5=want["r1"]), "float32")
    assert all((tmp_path / f"{s['step']}.json").exists() for s in steps)


@pytest.mark.parametrize("head_dim,heads,kv_heads", [(80, 3, 1), (144, 2, 2), (256, 2, 1), (112, 4, 2)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_head_sizes_in_steps_of_16(head_dim, heads, kv_heads, dtype, tmp_path):
    """Head sizes that no tensor-core kernel of the engine is built for run on the CUDA-core kernels, in both
    modes: whole, and the last tokens one by one."""
    from tests.util import write_folder, make_weights
    cfg = dict(architectures=["Qwen3ForCausalLM"], vocab_size=200, hidden_size=88, intermediate_size=120,
               num_hidden_layers=2, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
               rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=256, tie_word_embeddings=True)
    folder = write_folder(tmp_path / "model", cfg, make_weights(cfg, seed=head_dim))
    toks = random_tokens(50, 200, seed=head_dim + 1)
    want = {"r": PlainModel(folder).logits(toks)}
    from jax_vllm_b200.engine.replay import Replayer
    for i, steps in enumerate((whole("r", toks), prefix_then_single("r", toks, tail=12))):
        out = tmp_path / f"out{i}"
        rep = Replayer(folder, dtype, out, max_tokens=64, page_size=8)
        rep.run_stream(json.dumps(s) for s in steps)
        rep.cache.check()
        compare(steps, out, 200, want, dtype)


@pytest.mark.parametrize("heads,kv_heads", [(5, 1), (6, 2), (7, 1)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_group_sizes_that_do_not_divide_the_tile(heads, kv_heads, dtype, tmp_path):
    """Head size 128 with 5, 3 and 7 query heads per kv head: the 128-row tiles of the tcgen05 kernels hold 25, 42
    and 18 tokens and leave rows over.  Whole, in portions, and the last tokens one by one."""
    from tests.util import write_folder, make_weights
    cfg = dict(architectures=["Qwen3ForCausalLM"], vocab_size=200, hidden_size=96, intermediate_size=128,
               num_hidden_layers=2, num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=128,
               rms_norm_eps=1e-6, rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=True)
    folder = write_folder(tmp_path / "model", cfg, make_weights(cfg, seed=heads))
    toks = random_tokens(230, 200, seed=heads + 1)
    want = {"r": PlainModel(folder).logits(toks)}
    from jax_vllm_b200.engine.replay import Replayer
    for i, steps in enumerate((whole("r", toks), portions("r", toks, [97, 2, 51, 30, 26, 24]), prefix_then_single("r", toks, tail=12))):
        out = tmp_path / f"out{i}"
        rep = Replayer(folder, dtype, out, max_tokens=256, page_size=16)
        rep.run_stream(json.dumps(s) for s in steps)
        rep.cache.check()
        compare(steps, out, 200, want, dtype)
