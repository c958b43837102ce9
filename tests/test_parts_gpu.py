"""Each part of a model alone against the plain formulas, and the generality of the
assembly: a layer run twice, a layer that reads another layer's cache, a windowed layer
beside a full one, and a toy mixer with state of its own that is defined here, registered,
built and stepped without any change to the package."""

from dataclasses import dataclass, replace

import pytest
import torch

from tests.plain import qwen3_plain as plain
from tests.util import TINY_B, random_tokens

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def pkg():
    import jax_vllm_b200 as j
    from jax_vllm_b200 import cache, config, engine, parts, weights
    return j, cache, config, engine, parts, weights


def make_runner(spec, seed=0, dtype=torch.float32, page=8, pages=64, std=None):
    """A runner for `spec` with random float32 weights; returns (runner, weights on the CPU)."""
    j, cache, config, engine, parts, weights = pkg()
    ctx = parts.BuildContext(dtype=dtype, device=DEV, decode_split_size=32)
    model = parts.Model(spec, ctx)
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, ts in model.tensor_specs().items():
        z = torch.randn(ts.shape, generator=g)
        w[name] = (1 + 0.1 * z) if ts.kind == "vector" else z * (std or 1.5 / ts.shape[-1] ** 0.5)
    model.bind({k: v.to(DEV) for k, v in w.items()})
    cm = cache.CacheManager(model.cache_needs(), page, pages, 4, prefix_cache=False)
    return engine.Runner(model, cm, DEV, dtype), w


def run_cut(runner, toks, cuts):
    """Feeds `toks` in portions of the sizes in `cuts` (cycled); returns logits of all positions."""
    j, cache, config, engine, parts, weights = pkg()
    rc = runner.cache.admit(object())
    rows, i, k = [], 0, 0
    while i < len(toks):
        n = min(cuts[k % len(cuts)], len(toks) - i)
        rows.append(runner.run([engine.StepEntry(rc, toks[i:i + n], tuple(range(n)))]).cpu())
        i += n; k += 1
    runner.check_kernels()
    runner.cache.release(rc.request_id)
    return torch.cat(rows)


def qwen_cfg(c):
    return dict(num_heads=c["num_attention_heads"], num_kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
                rms_norm_eps=c["rms_norm_eps"], rope_theta=c["rope_theta"], num_hidden_layers=c["num_hidden_layers"],
                tie_word_embeddings=c["tie_word_embeddings"])


def spec_b():
    j = pkg()[0]
    return j.registry.config_from_dict(TINY_B).to_spec()


# ----------------------------------------------------------------- parts, one by one
def test_norm_and_position_parts():
    j, cache, config, engine, parts, weights = pkg()
    ctx = parts.BuildContext(torch.float32, DEV)
    norm = parts.NORMS["rmsnorm"](config.NormSpec(72, 1e-5, "n.weight"), "pre", ctx)
    assert list(norm.tensor_specs()) == ["pre.n.weight"]
    w = 1 + 0.1 * torch.randn(72)
    norm.bind({"pre.n.weight": w.to(DEV)})
    h, d = torch.randn(5, 72), torch.randn(5, 72)
    hd = h.clone().to(DEV)
    y = norm.norm(hd, d.to(DEV))
    torch.testing.assert_close(y.cpu(), plain.rms_norm(h + d, w, 1e-5), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(hd.cpu(), h + d)
    rope = parts.POSITIONS["rope"](config.RopeSpec(dim=48, theta=1e6), "", ctx)
    want = 1.0 / (1e6 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert torch.equal(rope.table().cpu(), want)
    with pytest.raises(ValueError):
        parts.POSITIONS["rope"](config.RopeSpec(dim=7, theta=1e4), "", ctx)


@pytest.mark.parametrize("window", [None, 11])
def test_attention_mixer_alone(window):
    """The mixer stepped in portions equals the plain attention block over the whole sequence."""
    j, cache, config, engine, parts, weights = pkg()
    spec = config.AttentionSpec(hidden_size=40, num_heads=6, num_kv_heads=2, head_dim=16, scale=0.25,
                                position=config.RopeSpec(16, 1e4), qk_norm_eps=1e-5, window=window)
    ctx = parts.BuildContext(torch.float32, DEV, decode_split_size=16)
    mixer = parts.MIXERS["attention"](spec, "L", ctx)
    g = torch.Generator().manual_seed(1)
    w = {n: (1 + 0.1 * torch.randn(ts.shape, generator=g)) if ts.kind == "vector" else torch.randn(ts.shape, generator=g) * 0.3
         for n, ts in mixer.tensor_specs().items()}
    mixer.bind({k: v.to(DEV) for k, v in w.items()})
    cm = cache.CacheManager([mixer.cache_need()], 8, 16, 2, prefix_cache=False)
    views = cm.allocate_storage(torch.float32, DEV)
    builder = engine.BatchBuilder(1, 8, mixer.tile_classes(8), DEV)
    x = torch.randn(37, 40, generator=g)
    rc = cm.admit("r")
    outs, i = [], 0
    for n in (5, 1, 2, 17, 1, 11):
        cm.grow(rc, i + n)
        step = builder.build([engine.StepEntry(rc, [0] * n, ())])
        outs.append(mixer.forward(x[i:i + n].to(DEV), step, views[0]).cpu())
        cm.commit(rc, [0] * n)
        i += n
    pcfg = dict(num_heads=6, num_kv_heads=2, head_dim=16, rms_norm_eps=1e-5, rope_theta=1e4)
    pw = {k.replace("L.self_attn", "p"): v for k, v in w.items()}
    T = x.shape[0]
    q = plain.linear(x, pw["p.q_proj.weight"]).reshape(T, 6, 16).transpose(0, 1)
    k = plain.linear(x, pw["p.k_proj.weight"]).reshape(T, 2, 16).transpose(0, 1)
    v = plain.linear(x, pw["p.v_proj.weight"]).reshape(T, 2, 16).transpose(0, 1)
    cos, sin = plain.rope_cos_sin(torch.arange(T), 16, 1e4)
    q = plain.apply_rope(plain.rms_norm(q, pw["p.q_norm.weight"], 1e-5), cos, sin)
    k = plain.apply_rope(plain.rms_norm(k, pw["p.k_norm.weight"], 1e-5), cos, sin)
    # head size 16 gives the plain scale 0.25 as well
    o = plain.causal_attention(q, k, v, 6, 2, 16, window=window).transpose(0, 1).reshape(T, 96)
    want = plain.linear(o, pw["p.o_proj.weight"])
    torch.testing.assert_close(torch.cat(outs), want, atol=2e-4, rtol=2e-4)
    if window:
        assert sum(p >= 0 for p in rc.tables[0]) <= 3          # pages behind the window went back


def test_feed_forward_and_block_alone():
    j, cache, config, engine, parts, weights = pkg()
    ctx = parts.BuildContext(torch.float32, DEV)
    ff = parts.FEED_FORWARDS["gated_mlp"](config.GatedMLPSpec(40, 56), "L", ctx)
    g = torch.Generator().manual_seed(2)
    w = {n: torch.randn(ts.shape, generator=g) * 0.3 for n, ts in ff.tensor_specs().items()}
    ff.bind({k: v.to(DEV) for k, v in w.items()})
    x = torch.randn(9, 40, generator=g)
    torch.testing.assert_close(ff.forward(x.to(DEV), None).cpu(), plain.swiglu(x, w, "L.mlp"), atol=1e-4, rtol=1e-4)
    with pytest.raises(ValueError, match="activation"):
        parts.FEED_FORWARDS["gated_mlp"](config.GatedMLPSpec(40, 56, activation="gelu"), "L", ctx)


@pytest.mark.parametrize("rows", [3, 16, 17, 150, 1100])
def test_feed_forward_bf16_with_the_gate_in_the_product(rows):
    """An intermediate size that is a multiple of 128 takes the interleaved gate|up weight: prompt steps apply
    the gate in the epilogue of the tcgen05 product (here from 1,024 rows on; the part itself goes by the product's
    tiles per multiprocessor), smaller batches in the separate kernel; both equal plain."""
    j, cache, config, engine, parts, weights = pkg()
    ctx = parts.BuildContext(torch.bfloat16, DEV)
    ff = parts.FEED_FORWARDS["gated_mlp"](config.GatedMLPSpec(72, 384), "L", ctx)
    g = torch.Generator().manual_seed(8)
    w = {n: (torch.randn(ts.shape, generator=g) * 0.2).to(torch.bfloat16) for n, ts in ff.tensor_specs().items()}
    ff.bind({k: v.to(DEV) for k, v in w.items()})
    assert ff.block == 128
    assert not ff._fuse_gate(4096)           # 32 x 3 tiles are far fewer than nine per multiprocessor
    ff.FUSED_GATE_ROWS = 1024                # so that this small part takes both ways
    x = torch.randn(rows, 72, generator=g).to(torch.bfloat16)
    got = ff.forward(x.to(DEV), None).float().cpu()
    # the plain formula with the engine's rounding points: the activations are bfloat16 where they reach
    # memory (gate|up only on the small-batch path, silu(g) * u on both), sums are 32-bit or better
    rnd = lambda t: t.to(torch.bfloat16).double()
    wd = {k: v.double() for k, v in w.items()}
    gate, up = x.double() @ wd["L.mlp.gate_proj.weight"].T, x.double() @ wd["L.mlp.up_proj.weight"].T
    if not ff._fuse_gate(rows):
        gate, up = rnd(gate), rnd(up)
    want = (rnd(torch.nn.functional.silu(gate) * up) @ wd["L.mlp.down_proj.weight"].T).float()
    torch.testing.assert_close(got, want, atol=2e-2, rtol=1e-2)
    loose = plain.swiglu(x.float(), {k: v.float() for k, v in w.items()}, "L.mlp")
    assert (got - loose).abs().max().item() <= 0.02 * loose.abs().max().item()      # and near the unrounded formula
    from jax_vllm_b200 import ops
    ops.check_status()


@pytest.mark.parametrize("rows", [1, 7, 16, 40])
def test_feed_forward_bf16_whose_down_product_comes_as_the_parts_of_a_sum(rows):
    """A feed-forward wide enough that the decode product cuts the k of the down product (few strips, long k): the
    part hands back the parts of a sum, which the next norm adds to the stream as it reads them."""
    j, cache, config, engine, parts, weights = pkg()
    from jax_vllm_b200 import ops
    ctx = parts.BuildContext(torch.bfloat16, DEV)
    ff = parts.FEED_FORWARDS["gated_mlp"](config.GatedMLPSpec(1024, 2048), "L", ctx)
    g = torch.Generator().manual_seed(9)
    w = {n: (torch.randn(ts.shape, generator=g) * 0.05).to(torch.bfloat16) for n, ts in ff.tensor_specs().items()}
    ff.bind({k: v.to(DEV) for k, v in w.items()})
    x = torch.randn(rows, 1024, generator=g).to(torch.bfloat16)
    got = ff.forward(x.to(DEV), None)
    plan = ops.linear_stream_splits
    assert isinstance(got, ops.PartialSum) and got.parts.shape[0] == plan(DEV, 1024, 2048) > 1
    rnd = lambda t: t.to(torch.bfloat16).double()
    wd = {k: v.double() for k, v in w.items()}
    gate, up = x.double() @ wd["L.mlp.gate_proj.weight"].T, x.double() @ wd["L.mlp.up_proj.weight"].T
    if plan(DEV, 2 * 2048, 1024) == 1:                   # gate|up reaches memory as bfloat16; as the parts of a sum it does not
        gate, up = rnd(gate), rnd(up)
    want = (rnd(torch.nn.functional.silu(gate) * up) @ wd["L.mlp.down_proj.weight"].T).float()
    torch.testing.assert_close(got.tensor().cpu(), want, atol=2e-2, rtol=1e-2)
    # through a norm: norm(h + delta) with the stream updated in place
    norm = parts.NORMS["rmsnorm"](config.NormSpec(1024, 1e-6, "weight"), "N", ctx)
    norm.bind({"N.weight": torch.ones(1024, dtype=torch.bfloat16, device=DEV)})
    h = torch.randn(rows, 1024, generator=g)
    hd = h.to(DEV)
    y = norm.norm(hd, got).float().cpu()
    torch.testing.assert_close(hd.cpu(), h + want, atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(y, plain.rms_norm(h + want, torch.ones(1024), 1e-6), atol=3e-2, rtol=2e-2)
    ops.check_status()


def test_kinds_are_looked_up_in_the_registries():
    j, cache, config, engine, parts, weights = pkg()
    spec = spec_b()
    bad = replace(spec, layers=(replace(spec.layers[0], mixer=replace(spec.layers[0].mixer, kind="nonesuch")),))
    with pytest.raises(ValueError, match="unknown mixer kind 'nonesuch'"):
        parts.Model(bad, parts.BuildContext(torch.float32, DEV))


# --------------------------------------------------- arrangements of layers as data
def plain_layers(w, cfg, toks, order, windows=None, cache_from=None):
    """Plain forward with a run order, per-layer windows and layers that read another layer's keys/values."""
    ids = torch.as_tensor(toks)
    T = len(toks)
    pos = torch.arange(T)
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    Hq, Hkv, D, eps = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    cos, sin = plain.rope_cos_sin(pos, D, cfg["rope_theta"])
    kv = {}
    for i in order:
        p = f"model.layers.{i}"
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
        q = plain.linear(x, w[f"{p}.self_attn.q_proj.weight"]).reshape(T, Hq, D).transpose(0, 1)
        q = plain.apply_rope(plain.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], eps), cos, sin)
        src = (cache_from or {}).get(i)
        if src is None:
            k = plain.linear(x, w[f"{p}.self_attn.k_proj.weight"]).reshape(T, Hkv, D).transpose(0, 1)
            v = plain.linear(x, w[f"{p}.self_attn.v_proj.weight"]).reshape(T, Hkv, D).transpose(0, 1)
            k = plain.apply_rope(plain.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], eps), cos, sin)
            kv[i] = (k, v)
        else:
            k, v = kv[src]
        o = plain.causal_attention(q, k, v, Hq, Hkv, D, window=(windows or {}).get(i))
        h = h + plain.linear(o.transpose(0, 1).reshape(T, Hq * D), w[f"{p}.self_attn.o_proj.weight"])
        h = h + plain.swiglu(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    h = plain.rms_norm(h, w["model.norm.weight"], eps)
    return plain.linear(h, w["lm_head.weight"])


def test_a_layer_run_twice_a_shared_cache_and_a_window_beside_full_layers():
    spec = spec_b()
    layers = list(spec.layers)
    layers[1] = replace(layers[1], mixer=replace(layers[1].mixer, window=13))   # its own cache group
    layers[2] = replace(layers[2], cache_from=0)                                 # reads layer 0's keys and values
    spec = replace(spec, layers=tuple(layers), schedule=(0, 1, 2, 1))
    runner, w = make_runner(spec, seed=3)
    assert [g.layers for g in runner.cache.groups] == [[0], [1, 3]]      # caches belong to places in the order
    assert "model.layers.2.self_attn.k_proj.weight" not in w
    toks = random_tokens(61, TINY_B["vocab_size"], seed=4)
    want = plain_layers(w, qwen_cfg(TINY_B), toks, (0, 1, 2, 1), windows={1: 13}, cache_from={2: 0})
    lim = 1e-4 * max(1.0, want.abs().max().item())
    for cuts in [(61,), (7, 2, 13, 1, 1, 5), (29, 1)]:
        got = run_cut(runner, toks, cuts)
        assert (got - want).abs().max().item() <= lim, cuts
    runner.cache.check()


# --------------------------------------------- a toy mixer with state of its own
@dataclass(frozen=True)
class DecaySpec:
    hidden_size: int
    decay: float
    kind: str = "toy_decay"


def register_toy():
    j, cache, config, engine, parts, weights = pkg()

    class DecayMixer(parts.Part):
        """y_t = s_t * w with s_t = decay * s_{t-1} + x_t: a running sum kept per request in a
        fixed-size state row, carried from step to step (torch ops: a toy for this test).  It loops over the
        entries on the host, from the host lists of the step context, so it says that it cannot be captured."""

        capturable = False

        def __init__(self, spec, prefix, ctx):
            self.spec, self.name, self.ctx = spec, f"{prefix}.decay.weight", ctx

        def tensor_specs(self):
            return {self.name: parts.TensorSpec((self.spec.hidden_size,), kind="vector", init="ones_normal")}

        def bind(self, tensors):
            self.w = tensors[self.name].float()

        def cache_need(self):
            return parts.FixedStateNeed((self.spec.hidden_size,), torch.float32)

        def forward(self, x, step, cache):
            out = torch.empty_like(x)
            i = 0
            for q, slot in zip(step.host_q_lens, step.host_slots):
                s = cache.state[slot]
                for t in range(i, i + q):
                    s = self.spec.decay * s + x[t].float()
                    out[t] = (s * self.w).to(x.dtype)
                cache.state[slot] = s
                i += q
            return out

    parts.register_mixer("toy_decay", DecayMixer)

    class DecayMixerOnDevice(DecayMixer):
        """The same recurrence from the device tensors of the step context only (positions, entry of each token,
        state slots, offsets of the entries), with shapes that depend on the numbers of tokens and entries alone:
        a step of it can be captured into a CUDA graph and replayed."""

        capturable = True

        def forward(self, x, step, cache):
            d = self.spec.decay
            pos, ent = step.positions.long(), step.token_entry.long()
            slots, start = step.state_slots.long(), step.start_pos.long()
            xf = x.float()
            same = ent[:, None] == ent[None, :]
            lag = (pos[:, None] - pos[None, :]).clamp(min=0).float()
            weight = torch.where(same & (pos[None, :] <= pos[:, None]), torch.pow(torch.full_like(lag, d), lag),
                                 torch.zeros_like(lag))
            carried = cache.state[slots[ent]] * torch.pow(torch.full_like(pos, d, dtype=torch.float32),
                                                          (pos - start[ent] + 1).float())[:, None]
            s = weight @ xf + carried
            last = step.cu_seqlens.long()[1:] - 1
            cache.state.index_copy_(0, slots, s[last])
            return (s * self.w).to(x.dtype)

    parts.register_mixer("toy_decay_on_device", DecayMixerOnDevice)


def plain_with_toy(w, cfg, toks, toy_layers, decay):
    ids = torch.as_tensor(toks)
    T = len(toks)
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    eps = cfg["rms_norm_eps"]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
        if i in toy_layers:
            s, ys = torch.zeros(x.shape[1]), []
            for t in range(T):
                s = decay * s + x[t]
                ys.append(s * w[f"{p}.decay.weight"])
            h = h + torch.stack(ys)
        else:
            h = h + plain.attention_block(x, w, f"{p}.self_attn", cfg, torch.arange(T))
        h = h + plain.swiglu(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])


def test_toy_mixer_with_own_state_registers_builds_and_steps():
    j, cache, config, engine, parts, weights = pkg()
    register_toy()
    spec = spec_b()
    layers = list(spec.layers)
    layers[1] = replace(layers[1], mixer=DecaySpec(spec.hidden_size, 0.9))
    spec = replace(spec, layers=tuple(layers))
    runner, w = make_runner(spec, seed=5)
    assert runner.cache.state_layers.keys() == {1} and [g.layers for g in runner.cache.groups] == [[0, 2]]
    assert runner.cache.prefix_cache is False
    toks = random_tokens(45, TINY_B["vocab_size"], seed=6)
    want = plain_with_toy(w, qwen_cfg(TINY_B), toks, {1}, 0.9)
    lim = 1e-4 * max(1.0, want.abs().max().item())
    for cuts in [(45,), (6, 1, 2, 9)]:
        got = run_cut(runner, toks, cuts)          # a fresh request each time: its state row starts at zero
        assert (got - want).abs().max().item() <= lim, cuts
    # two requests side by side keep their states apart
    other = random_tokens(20, TINY_B["vocab_size"], seed=7)
    want_other = plain_with_toy(w, qwen_cfg(TINY_B), other, {1}, 0.9)
    a, b = runner.cache.admit("a"), runner.cache.admit("b")
    la = runner.run([engine.StepEntry(a, toks[:10], ()), engine.StepEntry(b, other[:7], (6,))])
    lb = runner.run([engine.StepEntry(b, other[7:], tuple(range(13))), engine.StepEntry(a, toks[10:12], (1,))]).cpu()
    assert (la.cpu()[0] - want_other[6]).abs().max().item() <= lim
    assert (lb[:13] - want_other[7:]).abs().max().item() <= lim
    assert (lb[13] - want[11]).abs().max().item() <= lim
    runner.check_kernels()


@pytest.mark.parametrize("kind,replays", [("toy_decay", False), ("toy_decay_on_device", True)])
def test_toy_mixer_through_the_entry_point_with_captured_graphs(kind, replays):
    """Two requests decode side by side through `make_driver` with CUDA graphs on.  The toy that reads the
    host lists of the step says so (`capturable = False`) and its model is stepped eagerly; the toy written on
    the device tensors is captured and replayed.  Both give the plain toy's greedy tokens."""
    j, cache, config, engine, parts, weights = pkg()
    register_toy()
    spec = spec_b()
    layers = list(spec.layers)
    layers[1] = replace(layers[1], mixer=DecaySpec(spec.hidden_size, 0.9, kind=kind))
    spec = replace(spec, layers=tuple(layers))
    ctx = parts.BuildContext(dtype=torch.float32, device=DEV, decode_split_size=32)
    model = parts.Model(spec, ctx)
    g = torch.Generator().manual_seed(21)
    w = {}
    for name, ts in model.tensor_specs().items():
        z = torch.randn(ts.shape, generator=g)
        w[name] = (1 + 0.1 * z) if ts.kind == "vector" else z * (1.5 / ts.shape[-1] ** 0.5)
    model.bind({k: v.to(DEV) for k, v in w.items()})
    assert model.capturable() is replays
    cfg = qwen_cfg(TINY_B)
    prompts = [random_tokens(9, TINY_B["vocab_size"], seed=22), random_tokens(4, TINY_B["vocab_size"], seed=23)]
    new = 10

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(plain_with_toy(w, cfg, seq, {1}, 0.9)[-1].argmax()))
        return seq[len(prompt):]

    d = engine.make_driver(model, max_num_seqs=2, max_model_len=32, block_size=8, cuda_graphs=True)
    got = engine.generate(d, prompts, engine.SamplingParams(max_new_tokens=new))
    assert got == [plain_greedy(p) for p in prompts]
    assert (d.runner.graph_replays > 0) is replays
    d.cache.check()
    assert not d.cache.live


# ------------------------------------- a toy feed-forward with routing, defined here
@dataclass(frozen=True)
class RoutedSpec:
    hidden_size: int
    intermediate_size: int
    num_experts: int
    prefix: str = "moe"
    kind: str = "toy_routed"


def register_toy_routed():
    j, cache, config, engine, parts, weights = pkg()

    class Top1Experts(parts.Part):
        """Every token goes to the expert with the largest router logit (32-bit), whose gated feed-forward
        output is scaled by that expert's softmax weight (torch ops: a toy for this test)."""

        def __init__(self, spec, prefix, ctx):
            self.spec, self.p, self.ctx = spec, f"{prefix}.{spec.prefix}", ctx

        def tensor_specs(self):
            s, out = self.spec, {f"{self.p}.router.weight": parts.TensorSpec((self.spec.num_experts, self.spec.hidden_size))}
            for e in range(s.num_experts):
                out[f"{self.p}.experts.{e}.gate_up.weight"] = parts.TensorSpec((2 * s.intermediate_size, s.hidden_size))
                out[f"{self.p}.experts.{e}.down.weight"] = parts.TensorSpec((s.hidden_size, s.intermediate_size))
            return out

        def bind(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items() if k.startswith(self.p + ".")}

        def forward(self, x, step):
            xf = x.float()
            probs = torch.softmax(xf @ self.t[f"{self.p}.router.weight"].T, dim=-1)
            weight, expert = probs.max(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.spec.num_experts):
                rows = (expert == e).nonzero().flatten()
                if rows.numel():
                    gu = xf[rows] @ self.t[f"{self.p}.experts.{e}.gate_up.weight"].T
                    g, u = gu.chunk(2, dim=-1)
                    out[rows] = (torch.nn.functional.silu(g) * u) @ self.t[f"{self.p}.experts.{e}.down.weight"].T
            return (out * weight[:, None]).to(x.dtype)

    parts.register_feed_forward("toy_routed", Top1Experts)


def plain_routed(x, w, p, n_experts):
    probs = torch.softmax(x @ w[f"{p}.router.weight"].T, dim=-1)
    weight, expert = probs.max(dim=-1)
    ys = []
    for t in range(x.shape[0]):
        e = int(expert[t])
        g, u = (w[f"{p}.experts.{e}.gate_up.weight"] @ x[t]).chunk(2)
        ys.append(weight[t] * (w[f"{p}.experts.{e}.down.weight"] @ (torch.nn.functional.silu(g) * u)))
    return torch.stack(ys)


def test_toy_feed_forward_with_routing_registers_builds_and_steps():
    j, cache, config, engine, parts, weights = pkg()
    register_toy_routed()
    spec = spec_b()
    layers = list(spec.layers)
    layers[2] = replace(layers[2], feed_forward=RoutedSpec(spec.hidden_size, 40, 3))
    spec = replace(spec, layers=tuple(layers))
    runner, w = make_runner(spec, seed=11)
    assert any(".moe.experts.2.down.weight" in n for n in w) and not any("layers.2.mlp" in n for n in w)
    cfg = qwen_cfg(TINY_B)
    toks = random_tokens(41, TINY_B["vocab_size"], seed=12)
    ids, T, eps = torch.as_tensor(toks), len(toks), cfg["rms_norm_eps"]
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        h = h + plain.attention_block(plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", cfg,
                                      torch.arange(T))
        x = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)
        h = h + (plain_routed(x, w, f"{p}.moe", 3) if i == 2 else plain.swiglu(x, w, f"{p}.mlp"))
    want = plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])
    lim = 1e-4 * max(1.0, want.abs().max().item())
    for cuts in [(41,), (5, 1, 1, 13, 2)]:
        got = run_cut(runner, toks, cuts)
        assert (got - want).abs().max().item() <= lim, cuts


# --------------------------------------- another position encoding, defined here
@dataclass(frozen=True)
class HarmonicSpec:
    dim: int                       # rotated elements of a head (here fewer than the head has)
    base: float
    kind: str = "toy_harmonic"


def register_toy_position():
    j, cache, config, engine, parts, weights = pkg()

    class Harmonic(parts.Part):
        """Angles position * base / (j + 1) instead of the geometric table: only the table differs, the
        rotation kernel is the same."""

        def __init__(self, spec, prefix, ctx):
            self.dim = int(spec.dim)
            self.freq = (float(spec.base) / torch.arange(1, self.dim // 2 + 1, dtype=torch.float32)).to(ctx.device)

        def table(self):
            return self.freq

    parts.register_position("toy_harmonic", Harmonic)


def test_toy_position_encoding_registers_builds_and_steps():
    j, cache, config, engine, parts, weights = pkg()
    register_toy_position()
    spec = spec_b()
    D = TINY_B["head_dim"]
    rot = D // 2                   # half of the head rotates, the rest passes
    layers = tuple(replace(l, mixer=replace(l.mixer, position=HarmonicSpec(rot, 0.7))) for l in spec.layers)
    spec = replace(spec, layers=layers)
    runner, w = make_runner(spec, seed=13)
    cfg = qwen_cfg(TINY_B)
    toks = random_tokens(37, TINY_B["vocab_size"], seed=14)
    ids, T, eps = torch.as_tensor(toks), len(toks), cfg["rms_norm_eps"]
    Hq, Hkv = cfg["num_heads"], cfg["num_kv_heads"]
    ang = torch.arange(T, dtype=torch.float32)[:, None] * (0.7 / torch.arange(1, rot // 2 + 1, dtype=torch.float32))[None]
    cos, sin = torch.cos(torch.cat([ang, ang], -1)), torch.sin(torch.cat([ang, ang], -1))
    rotate = lambda u: torch.cat([plain.apply_rope(u[..., :rot], cos, sin), u[..., rot:]], dim=-1)
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)
        q = plain.linear(x, w[f"{p}.self_attn.q_proj.weight"]).reshape(T, Hq, D).transpose(0, 1)
        k = plain.linear(x, w[f"{p}.self_attn.k_proj.weight"]).reshape(T, Hkv, D).transpose(0, 1)
        v = plain.linear(x, w[f"{p}.self_attn.v_proj.weight"]).reshape(T, Hkv, D).transpose(0, 1)
        q = rotate(plain.rms_norm(q, w[f"{p}.self_attn.q_norm.weight"], eps))
        k = rotate(plain.rms_norm(k, w[f"{p}.self_attn.k_norm.weight"], eps))
        o = plain.causal_attention(q, k, v, Hq, Hkv, D).transpose(0, 1).reshape(T, Hq * D)
        h = h + plain.linear(o, w[f"{p}.self_attn.o_proj.weight"])
        h = h + plain.swiglu(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    want = plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])
    lim = 1e-4 * max(1.0, want.abs().max().item())
    for cuts in [(37,), (4, 1, 9, 2)]:
        got = run_cut(runner, toks, cuts)
        assert (got - want).abs().max().item() <= lim, cuts
