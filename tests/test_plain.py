"""The plain implementation against the reference's own model code (golden file made
by tests/golden/make_golden.py), and against itself."""

from pathlib import Path

import numpy as np
import pytest
import torch

from tests.plain import qwen3_plain as plain

GOLDEN = Path(__file__).parent / "golden" / "qwen3_reference_logits.npz"


def _load(tag):
    z = np.load(GOLDEN)
    cfg = {k.split("/")[-1]: z[k].item() for k in z.files if k.startswith(f"{tag}/cfg/")}
    w = {k[len(f"{tag}/w/"):]: torch.from_numpy(z[k]) for k in z.files if k.startswith(f"{tag}/w/")}
    return cfg, w, z[f"{tag}/ids"].tolist(), torch.from_numpy(z[f"{tag}/logits"])


@pytest.mark.parametrize("tag", ["a", "b"])
def test_plain_matches_reference_model_code(tag):
    cfg, w, ids, want = _load(tag)
    got = plain.forward(cfg, w, ids)
    scale = want.abs().max().item()
    assert scale > 1.0  # the golden model is not degenerate
    assert (got - want).abs().max().item() <= 2e-5 * max(1.0, scale)
    assert torch.equal(got.argmax(-1), want.argmax(-1))


def test_plain_is_causal():
    cfg, w, ids, _ = _load("a")
    whole = plain.forward(cfg, w, ids)
    part = plain.forward(cfg, w, ids[:9])
    assert (whole[:9] - part).abs().max().item() < 1e-5


def test_plain_window_equals_full_when_wide():
    q = torch.randn(4, 10, 8); k = torch.randn(2, 10, 8); v = torch.randn(2, 10, 8)
    a = plain.causal_attention(q, k, v, 4, 2, 8)
    b = plain.causal_attention(q, k, v, 4, 2, 8, window=10)
    c = plain.causal_attention(q, k, v, 4, 2, 8, window=3)
    assert torch.allclose(a, b) and not torch.allclose(a, c)


def test_plain_greedy_stops_at_eos():
    cfg, w, ids, _ = _load("b")
    free = plain.greedy(cfg, w, ids[:5], 6)
    stopped = plain.greedy(cfg, w, ids[:5], 6, eos_id=free[2])
    assert stopped == free[: free.index(free[2]) + 1]
