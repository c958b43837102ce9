"""Shared test material: two tiny Qwen3 configurations that differ in every size and
option, a model-folder writer that is independent of the product's, and trace helpers."""

from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

# Two tiny configurations: layers 2/3, hidden 64/96, query heads 4/6, kv heads 2/1, head size
# 16 (= hidden/heads) / 32 (explicit), intermediate 160/224, vocabulary 256/384 (B: no power of
# two), theta 1e4/1e6, eps 1e-6/1e-5, tied/untied.  Page sizes 16/8 are chosen by the tests.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=160,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-6,
              rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=True)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], vocab_size=384, hidden_size=96, intermediate_size=224,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32, rms_norm_eps=1e-5,
              rope_theta=1e6, max_position_embeddings=512, tie_word_embeddings=False)
# A third one with the head size (128) and the feed-forward width (a multiple of 128) at which the bfloat16
# path takes its tcgen05 kernels (prompt attention in tensor memory, the gate in the product's epilogue).
TINY_C = dict(architectures=["Qwen3ForCausalLM"], vocab_size=300, hidden_size=192, intermediate_size=384,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
              rope_theta=5e5, max_position_embeddings=1024, tie_word_embeddings=False)
# A fourth one with sizes that are not even multiples of 16: width 120, 5 heads without grouping, head size 48
# (the tensor-core kernels do not take it: the bfloat16 path then runs the CUDA-core attention), one layer,
# an odd vocabulary, pages of 4 tokens.
TINY_D = dict(architectures=["Qwen3ForCausalLM"], vocab_size=301, hidden_size=120, intermediate_size=136,
              num_hidden_layers=1, num_attention_heads=5, num_key_value_heads=5, head_dim=48, rms_norm_eps=3e-6,
              rope_theta=2e4, max_position_embeddings=512, tie_word_embeddings=True)
# A fifth one with the head layout of the benchmarked model (32 query heads in 8 groups of 4, head size 128): the
# 128-row tiles of the tcgen05 prompt attention hold 32 tokens, the decode attention has 4 query rows per kv head.
TINY_E = dict(architectures=["Qwen3ForCausalLM"], vocab_size=320, hidden_size=512, intermediate_size=1024,
              num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
              rope_theta=1e6, max_position_embeddings=1024, tie_word_embeddings=False)
# A sixth one with five query heads per kv head, as the 14B shape has them: a number that does not divide the 128 rows
# of a tile (25 tokens a tile, three rows left over), more heads per group than the decode kernel prepares itself
# (the separate kernel runs before it), pages of 32 tokens.
TINY_F = dict(architectures=["Qwen3ForCausalLM"], vocab_size=310, hidden_size=320, intermediate_size=640,
              num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=2, head_dim=128, rms_norm_eps=2e-6,
              rope_theta=3e5, max_position_embeddings=1024, tie_word_embeddings=True)
TINY = {"a": TINY_A, "b": TINY_B, "c": TINY_C, "d": TINY_D, "e": TINY_E, "f": TINY_F}
PAGE_SIZE = {"a": 16, "b": 8, "c": 16, "d": 4, "e": 16, "f": 32}


def tensor_shapes(c: dict) -> dict:
    H, I = c["hidden_size"], c["intermediate_size"]
    Hq = c["num_attention_heads"]
    Hkv = c.get("num_key_value_heads", Hq)
    D = c.get("head_dim", H // Hq)
    shapes = {"model.embed_tokens.weight": (c["vocab_size"], H), "model.norm.weight": (H,)}
    if not c.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (c["vocab_size"], H)
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}"
        shapes.update({
            f"{p}.self_attn.q_proj.weight": (Hq * D, H), f"{p}.self_attn.k_proj.weight": (Hkv * D, H),
            f"{p}.self_attn.v_proj.weight": (Hkv * D, H), f"{p}.self_attn.o_proj.weight": (H, Hq * D),
            f"{p}.self_attn.q_norm.weight": (D,), f"{p}.self_attn.k_norm.weight": (D,),
            f"{p}.mlp.gate_proj.weight": (I, H), f"{p}.mlp.up_proj.weight": (I, H),
            f"{p}.mlp.down_proj.weight": (H, I), f"{p}.input_layernorm.weight": (H,),
            f"{p}.post_attention_layernorm.weight": (H,)})
    return shapes


def make_weights(c: dict, seed: int, matrix_std: float | None = None) -> dict:
    """Random float32 weights.  Matrices are N(0, std) with std = 1.5/sqrt(fan_in) unless given
    (large enough that attention is far from uniform and logits are of order one, so that a
    wrong key or a stale page shows); norm weights are 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        z = torch.randn(shape, generator=g, dtype=torch.float32)
        if len(shape) == 1:
            out[name] = 1.0 + 0.1 * z
        else:
            std = matrix_std if matrix_std is not None else 1.5 / (shape[1] ** 0.5)
            out[name] = std * z
    return out


def write_folder(folder, c: dict, weights: dict, dtype=torch.bfloat16) -> Path:
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(c))
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder


def make_folder(folder, tag: str, seed: int = 0, dtype=torch.bfloat16, matrix_std=None) -> Path:
    c = TINY[tag]
    return write_folder(folder, c, make_weights(c, seed, matrix_std), dtype)


def random_tokens(n: int, vocab: int, seed: int) -> list:
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


# ------------------------------------------------------------------------ traces
def whole(rid, tokens, step=0):
    """One request in one step, logits wanted everywhere."""
    return [{"step": step, "entries": [{"id": rid, "tokens": list(tokens), "want": list(range(len(tokens)))}],
             "end": [rid]}]


def prefix_then_single(rid, tokens, tail=32):
    """Most of the request in one step, the last `tail` tokens one by one."""
    head = len(tokens) - tail
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": list(tokens[:head]), "want": list(range(head))}], "end": []}]
    for i in range(head, len(tokens)):
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}],
                      "end": [rid] if i == len(tokens) - 1 else []})
    return steps


def portions(rid, tokens, sizes):
    """The request in portions of the given sizes (cycled), logits wanted everywhere."""
    steps, i, k = [], 0, 0
    while i < len(tokens):
        n = min(sizes[k % len(sizes)], len(tokens) - i)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(tokens[i:i + n]),
                                                       "want": list(range(n))}],
                      "end": [rid] if i + n == len(tokens) else []})
        i += n
        k += 1
    return steps


def collect(steps, out_dir, vocab: int) -> dict:
    """Reads the logits written for `steps` back into {request id: [position -> row]}."""
    got: dict = {}
    fed: dict = {}
    for s in steps:
        n_want = sum(len(e.get("want", [])) for e in s["entries"])
        rows = None
        if n_want:
            rows = np.fromfile(Path(out_dir) / f"{s['step']}.f32", dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            for w in e.get("want", []):
                got.setdefault(e["id"], {})[base + w] = rows[r]
                r += 1
            fed[e["id"]] = base + len(e["tokens"])
    return got
