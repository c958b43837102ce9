"""A whole architecture added from outside the package: a configuration class with config.json keys of its own,
registered under its architecture name, and nothing else.  Its model has layers of different kinds (a windowed
attention beside full ones, a layer that reads another layer's keys and values, a layer that runs twice), so the
loader, the cache groups, the step function, the replay program and the entry point all have to work from the
spec alone.  It is a toy for this test and no model of anyone's."""

import json
import math
from dataclasses import asdict, dataclass

import pytest
import torch

from tests.test_parts_gpu import plain_layers
from tests.test_replay_gpu import compare
from tests.util import portions, random_tokens, whole

pytestmark = pytest.mark.gpu
NAME = "ToyWindowedForCausalLM"


@dataclass(frozen=True)
class ToyConfig:
    """config.json of the toy: its own key names, none of Qwen3's."""
    vocab: int
    width: int
    ff: int
    depth: int
    heads: int
    groups: int
    head_size: int
    eps: float
    base: float
    window: int                  # every odd layer sees only this many keys
    reader: int                  # this layer reads the keys and values of layer 0
    twice: int                   # this layer runs a second time at the end

    @classmethod
    def from_dict(cls, c: dict) -> "ToyConfig":
        return cls(**{k: c[k] for k in cls.__dataclass_fields__})

    def to_dict(self) -> dict:
        return dict(asdict(self), architectures=[NAME])

    def to_spec(self):
        from jax_vllm_b200.config import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, RopeSpec
        layers = []
        for i in range(self.depth):
            attn = AttentionSpec(hidden_size=self.width, num_heads=self.heads, num_kv_heads=self.groups,
                                 head_dim=self.head_size, scale=1.0 / math.sqrt(self.head_size),
                                 position=RopeSpec(dim=self.head_size, theta=self.base), qk_norm_eps=self.eps,
                                 window=self.window if i % 2 else None)
            layers.append(LayerSpec(prefix=f"model.layers.{i}", mixer=attn,
                                    feed_forward=GatedMLPSpec(self.width, self.ff),
                                    mixer_norm=NormSpec(self.width, self.eps, "input_layernorm.weight"),
                                    ffn_norm=NormSpec(self.width, self.eps, "post_attention_layernorm.weight"),
                                    cache_from=0 if i == self.reader else None))
        spec = ModelSpec(architecture=NAME, vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers),
                         final_norm=NormSpec(self.width, self.eps, "model.norm.weight"),
                         schedule=tuple(range(self.depth)) + (self.twice,))
        spec.validate()
        return spec

    def order(self):
        return tuple(range(self.depth)) + (self.twice,)


TOY = ToyConfig(vocab=211, width=80, ff=144, depth=3, heads=4, groups=2, head_size=32, eps=2e-6, base=3e4, window=11,
                reader=2, twice=1)


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    """Registers the architecture, writes a model folder for it (config.json in its own keys, tensors by the names its
    parts ask for) and returns (folder, float32 weights, sequences, their logits by the plain implementation)."""
    from safetensors.torch import save_file
    from jax_vllm_b200 import registry
    from jax_vllm_b200.parts import BuildContext, Model

    registry.register_architecture(NAME, ToyConfig)
    folder = tmp_path_factory.mktemp("toy_architecture")
    (folder / "config.json").write_text(json.dumps(TOY.to_dict()))
    model = Model(TOY.to_spec(), BuildContext(dtype=torch.bfloat16, device=torch.device("cpu")))
    g = torch.Generator().manual_seed(31)
    w = {}
    for name, ts in model.tensor_specs().items():
        z = torch.randn(ts.shape, generator=g)
        w[name] = ((1 + 0.1 * z) if ts.kind == "vector" else z * 1.5 / ts.shape[-1] ** 0.5).to(torch.bfloat16)
    assert "model.layers.2.self_attn.k_proj.weight" not in w           # the reader has no keys of its own
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    w32 = {k: v.float() for k, v in w.items()}
    cfg = dict(num_heads=TOY.heads, num_kv_heads=TOY.groups, head_dim=TOY.head_size, rms_norm_eps=TOY.eps,
               rope_theta=TOY.base, num_hidden_layers=TOY.depth, tie_word_embeddings=False)
    seqs = {f"r{i}": random_tokens(n, TOY.vocab, seed=40 + i) for i, n in enumerate((70, 33, 91))}
    windows = {i: TOY.window for i in range(TOY.depth) if i % 2}
    want = {r: plain_layers(w32, cfg, t, TOY.order(), windows=windows, cache_from={TOY.reader: 0}) for r, t in seqs.items()}
    assert all(v.abs().max() > 1.0 for v in want.values())
    yield folder, w32, cfg, seqs, want, windows
    registry.ARCHITECTURES.pop(NAME, None)


def test_the_registry_knows_it_and_says_what_else_it_knows(toy):
    from jax_vllm_b200 import registry
    folder = toy[0]
    assert isinstance(registry.config_from_path(folder), ToyConfig)
    with pytest.raises(ValueError, match=f"Supported: .*Qwen3ForCausalLM.*{NAME}"):
        registry.config_from_dict({"architectures": ["NoSuchForCausalLM"]})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_the_toy_architecture_equals_plain(toy, dtype, tmp_path):
    """Through the replay program's own class: whole, in portions down to two tokens, and two requests side by side
    in a pool whose pages are used again; windowed layers give their pages back as the window passes them."""
    from jax_vllm_b200.engine.replay import Replayer
    folder, w32, cfg, seqs, want, windows = toy
    traces = {"whole": whole("r0", seqs["r0"]), "portions": portions("r2", seqs["r2"], (7, 2, 13, 1, 1, 5))}
    side = []
    a, b, fa, fb = seqs["r0"], seqs["r1"], 0, 0
    for step, (na, nb) in enumerate([(9, 2), (1, 17), (30, 1), (1, 1), (29, 12)]):
        entries = []
        if na:
            entries.append({"id": "r0", "tokens": a[fa:fa + na], "want": list(range(len(a[fa:fa + na])))}); fa += na
        if nb:
            entries.append({"id": "r1", "tokens": b[fb:fb + nb], "want": list(range(len(b[fb:fb + nb])))}); fb += nb
        side.append({"step": step, "entries": entries, "end": [r for r, f, s in (("r0", fa, a), ("r1", fb, b)) if f == len(s)]})
    assert fa == len(a) and fb == len(b)
    traces["side by side"] = side
    for name, steps in traces.items():
        out = tmp_path / name.replace(" ", "_")
        rep = Replayer(folder, dtype, out, max_tokens=128, page_size=8)
        assert [grp.need.window for grp in rep.cache.groups] == [None, TOY.window]      # two groups of layers by need
        assert [grp.layers for grp in rep.cache.groups] == [[0], [1, 3]]               # places in the run order
        rep.run_stream(json.dumps(s) for s in steps)
        rep.cache.check()
        assert not rep.cache.live
        compare(steps, out, TOY.vocab, want, dtype, case=f"toy architecture, {name}")
        if name == "portions":       # the windowed layers gave pages back long before the request ended
            assert sum(m["pages_released"] for m in rep.records[:-1]) >= 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_known_prefix_is_taken_over_where_the_window_still_reaches(toy, dtype, tmp_path):
    """Prefix reuse with a windowed group: a second request that starts like a finished one takes its pages, in the
    windowed layers only those the window of its first computed token reaches; the rest of its table says given back."""
    from jax_vllm_b200.engine.replay import Replayer
    folder, w32, cfg, seqs, want, windows = toy
    again = seqs["r0"][:52] + random_tokens(25, TOY.vocab, seed=77)
    first_wanted = 43                           # five pages of eight tokens lie before it
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": seqs["r0"], "want": [69]}], "end": ["r0"]},
             {"step": 1, "entries": [{"id": "r1", "tokens": seqs["r1"], "want": [32]}], "end": ["r1"]},
             {"step": 2, "entries": [{"id": "again", "tokens": again[:60], "want": list(range(first_wanted, 60))}], "end": []},
             {"step": 3, "entries": [{"id": "again", "tokens": again[60:], "want": list(range(len(again) - 60))}], "end": ["again"]}]
    rep = Replayer(folder, dtype, tmp_path, max_tokens=128, page_size=8, prefix_cache=True)
    assert rep.cache.prefix_cache is True
    for s in steps[:3]:
        rep.run_step(s)
    rc = rep.cache.live["again"]
    assert rep.records[2]["prefix_hit_tokens"] == 40 and rep.records[2]["tokens"] == 20
    # the first computed token is at 40 and sees keys from 30 on in the windowed layers: of the five known pages only
    # 3 and 4 were taken there; after the step (60 tokens, keys from 50 on) they and page 5 have been given back
    assert rep.records[2]["pages_allocated"] == 3 + 3 and rep.records[2]["pages_released"] == 3
    assert [p >= 0 for p in rc.tables[1]] == [False] * 6 + [True] * 2 and all(p >= 0 for p in rc.tables[0])
    rep.run_step(steps[3])
    rep.cache.check()
    assert not rep.cache.live
    want_all = dict(want, again=plain_layers(w32, cfg, again, TOY.order(), windows=windows, cache_from={TOY.reader: 0}))
    compare(steps, tmp_path, TOY.vocab, want_all, dtype, case="toy architecture, prefix reuse under a window")


def test_generation_of_the_toy_architecture_equals_plain(toy):
    from jax_vllm_b200 import SamplingParams, generate, load_from_path, make_driver
    folder, w32, cfg, seqs, want, windows = toy
    model = load_from_path(folder, dtype="fp32")
    d = make_driver(model, max_num_seqs=2, max_model_len=64, block_size=8, max_tokens_per_step=16)
    prompts = [seqs["r0"][:21], seqs["r1"][:5]]
    got = generate(d, prompts, SamplingParams(max_new_tokens=7))

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(7):
            seq.append(int(plain_layers(w32, cfg, seq, TOY.order(), windows=windows, cache_from={TOY.reader: 0})[-1].argmax()))
        return seq[len(prompt):]

    assert got == [plain_greedy(p) for p in prompts]
    assert d.cache.prefix_cache is True             # a windowed group does not switch prefix reuse off
    d.cache.check()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_arrivals_with_few_pages_known_prefixes_and_a_window(toy, seed):
    """Everything at once, through the entry point, in 32-bit where tokens must be equal: requests arrive at random
    steps, many start alike (known prefixes are taken over, in the windowed layers only as far as the window reaches),
    prompts are cut by a small token budget, the pool is too small for three requests (the youngest is preempted and
    run again), pages come back as the window passes and are used again, decode-only steps replay captured graphs.
    Greedy tokens depend on none of it."""
    import random
    from jax_vllm_b200 import SamplingParams, add_request, has_work, load_from_path, make_driver, step
    folder, w32, cfg, seqs, want, windows = toy
    rng = random.Random(seed)
    model = load_from_path(folder, dtype="fp32")
    d = make_driver(model, max_num_seqs=3, max_model_len=64, block_size=8, num_blocks=9, max_tokens_per_step=24)
    shared = seqs["r2"][:40]
    prompts = [shared[:rng.choice([0, 8, 17, 24])] + random_tokens(rng.randrange(1, 14), TOY.vocab, seed=100 * seed + i)
               for i in range(10)]
    new_tokens = [rng.randrange(6, 27) for _ in prompts]
    waiting, ids = list(range(len(prompts))), {}
    while waiting or has_work(d):
        if waiting and (rng.random() < 0.4 or not has_work(d)):
            i = waiting.pop(0)
            ids[i] = add_request(d, prompts[i], SamplingParams(max_new_tokens=new_tokens[i]))
        step(d)
        d.cache.check()
    assert not d.cache.live and all(g.pool.num_free == 9 for g in d.cache.groups)
    assert d.stats.preemptions > 0 and d.stats.cache_hit_tokens > 0

    def plain_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(plain_layers(w32, cfg, seq, TOY.order(), windows=windows, cache_from={TOY.reader: 0})[-1].argmax()))
        return seq[len(prompt):]

    for i, prompt in enumerate(prompts):
        assert d.requests[ids[i]].output_ids == plain_greedy(prompt, new_tokens[i]), f"request {i} of seed {seed}"
