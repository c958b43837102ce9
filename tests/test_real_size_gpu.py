"""The true 32-bit path at the widths and the vocabulary of Qwen3-8B (4,096 wide, 32 query heads in 8 groups,
head size 128, feed-forward 12,288, 151,936 tokens), with fewer layers than the 36 of that model so that the test
stays within seconds: RUN_LAYERS of FULL_LAYERS.  The oracle is the plain implementation of tests/plain with its
tensors on the device, torch's float32 products and TF32 switched off: unfused, whole sequences, no cache, no
code of the package.  Three requests are cut two ways: most of each in one step and the last 32 tokens one by
one, and mixed (portions of some beside single tokens of others) in a pool so small that pages are used again.
A one-layer model runs the output matrix of that vocabulary tied to the embedding and untied."""

import pytest
import torch

from tests.plain.qwen3_plain import PlainModel, read_config
from tests.util import random_tokens, tensor_shapes

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
FULL_LAYERS, RUN_LAYERS = 36, 6
QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                num_hidden_layers=FULL_LAYERS, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=40960, tie_word_embeddings=False)
PAGE = 16
LIMIT = 1e-4        # absolute: the logits of these models stay below 10 in size


def device_weights(cfg: dict, seed: int) -> dict:
    """Float32 weights drawn on the device: matrices N(0, 0.02), norm weights 1 + N(0, 0.1)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32, device=DEV)
        out[name] = (1.0 + 0.1 * z) if len(shape) == 1 else 0.02 * z
    return out


class Case:
    """The engine in 32-bit and the plain oracle over the same tensors."""

    def __init__(self, cfg: dict, seed: int, pool_tokens: int):
        from jax_vllm_b200 import registry
        from jax_vllm_b200.cache import CacheManager
        from jax_vllm_b200.engine import Runner
        from jax_vllm_b200.parts import BuildContext, Model

        self.cfg = cfg
        w = device_weights(cfg, seed)
        model = Model(registry.config_from_dict(cfg).to_spec(), BuildContext(dtype=torch.float32, device=DEV))
        assert set(model.tensor_specs()) == set(w)
        model.bind(w)
        self.cache = CacheManager(model.cache_needs(), PAGE, -(-pool_tokens // PAGE), 4, prefix_cache=False)
        self.runner = Runner(model, self.cache, DEV, torch.float32)
        plain_cfg = dict(vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"],
                         intermediate_size=cfg["intermediate_size"], num_hidden_layers=cfg["num_hidden_layers"],
                         num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
                         head_dim=cfg["head_dim"], rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"],
                         tie_word_embeddings=cfg["tie_word_embeddings"])
        self.plain = PlainModel(cfg=plain_cfg, weights=w)
        self.worst = 0.0

    def oracle(self, toks) -> torch.Tensor:
        return self.plain.logits(toks)

    def feed(self, rows):
        """One step: rows of (request cache, tokens); logits are asked for at every place."""
        from jax_vllm_b200.engine import StepEntry
        out = self.runner.run([StepEntry(rc, list(t), tuple(range(len(t)))) for rc, t in rows])
        return out.split([len(t) for _, t in rows])

    def hold(self, got: torch.Tensor, want: torch.Tensor, what: str) -> None:
        diff = (got - want).abs().max().item()
        self.worst = max(self.worst, diff)
        assert want.abs().max().item() < 10.0
        assert diff <= LIMIT, f"{what}: |diff| {diff:.3e}"
        assert torch.equal(got.argmax(-1), want.argmax(-1)), f"{what}: another greedy token"


@pytest.fixture
def true_float32_products():
    before = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = torch.backends.cudnn.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = before


def test_float32_at_full_widths_and_vocabulary_under_two_schedules(true_float32_products):
    from tests.conftest import record_worst

    cfg = dict(QWEN3_8B, num_hidden_layers=RUN_LAYERS)
    lens = (150, 90, 41)
    seqs = [random_tokens(n, cfg["vocab_size"], seed=500 + i) for i, n in enumerate(lens)]
    # the pool holds the three requests rounded up to pages and no more: the fourth (the first again) gets
    # pages that others gave back
    case = Case(cfg, seed=11, pool_tokens=sum(-(-n // PAGE) * PAGE for n in lens))
    with torch.no_grad():
        want = [case.oracle(s) for s in seqs]
    assert all(w.abs().max() > 1.0 for w in want)
    # --- most of each request in one step, the last 32 tokens one by one
    for i, (s, w) in enumerate(zip(seqs, want)):
        rc = case.cache.admit(f"single{i}")
        head = len(s) - 32
        case.hold(case.feed([(rc, s[:head])])[0], w[:head], f"request {i}, first {head} tokens")
        for t in range(head, len(s)):
            case.hold(case.feed([(rc, s[t:t + 1])])[0], w[t:t + 1], f"request {i}, token {t} alone")
        case.cache.release(rc.request_id)
    case.cache.check()
    # --- mixed: portions beside single tokens; requests end and the first comes again in pages given back
    a, b, c = (case.cache.admit(k) for k in "abc")
    fed = {"a": 0, "b": 0, "c": 0, "d": 0}
    seq_of = {"a": (seqs[0], want[0]), "b": (seqs[1], want[1]), "c": (seqs[2], want[2]), "d": (seqs[0], want[0])}
    live = {"a": a, "b": b, "c": c}
    plan = [[("a", 33), ("b", 2)], [("a", 1), ("b", 40), ("c", 7)], [("a", 1), ("b", 1), ("c", 1)],
            [("a", 70), ("b", 1), ("c", 1)], [("a", 999), ("b", 999)], [("c", 2), ("d", 50)], [("c", 1), ("d", 1)],
            [("c", 999), ("d", 999)]]
    allocated_before = case.cache.stats["pages_allocated"]
    for step, row in enumerate(plan):
        if step == 5:
            live["d"] = case.cache.admit("d")
        rows, spans = [], []
        for k, n in row:
            s, _ = seq_of[k]
            toks = s[fed[k]:fed[k] + n]
            rows.append((live[k], toks))
            spans.append((k, fed[k], fed[k] + len(toks)))
            fed[k] += len(toks)
        for (k, lo, hi), got in zip(spans, case.feed(rows)):
            case.hold(got, seq_of[k][1][lo:hi], f"mixed step {step}, request {k}, places {lo}..{hi}")
        for k, lo, hi in spans:
            if hi == len(seq_of[k][0]):
                case.cache.release(k)
    case.runner.check_kernels()
    case.cache.check()
    assert not case.cache.live
    assert case.cache.stats["pages_allocated"] - allocated_before > case.cache.num_pages     # pages were used again
    record_worst(f"Qwen3-8B widths, vocabulary 151,936, {RUN_LAYERS} of {FULL_LAYERS} layers", "float32", case.worst, LIMIT)


@pytest.mark.parametrize("tied", [True, False], ids=["tied", "untied"])
def test_output_matrix_of_the_full_vocabulary_tied_and_untied(true_float32_products, tied):
    from tests.conftest import record_worst

    cfg = dict(QWEN3_8B, num_hidden_layers=1, tie_word_embeddings=tied)
    toks = random_tokens(48, cfg["vocab_size"], seed=520)
    case = Case(cfg, seed=12, pool_tokens=64)
    with torch.no_grad():
        want = case.oracle(toks)
    rc = case.cache.admit("r")
    case.hold(case.feed([(rc, toks[:40])])[0], want[:40], "the first 40 tokens")
    for t in range(40, 48):
        case.hold(case.feed([(rc, toks[t:t + 1])])[0], want[t:t + 1], f"token {t} alone")
    case.runner.check_kernels()
    record_worst(f"Qwen3-8B widths, vocabulary 151,936, 1 layer, {'tied' if tied else 'untied'}", "float32", case.worst, LIMIT)
