"""Makes tests/golden/qwen3_reference_logits.npz from the reference's own model code.

JAX and Equinox are not installed where this was run, so the reference's
`jllm/model/common.py` and `jllm/model/qwen3.py` are imported unmodified under a
small stand-in for the few `jax`, `jax.numpy`, `jax.nn`, `jax.lax` and `equinox`
names they use, all mapped to numpy in 32-bit.  The arithmetic is therefore numpy's,
not XLA's; at the 1e-5 level that the test asks for this makes no difference.

    python tests/golden/make_golden.py --reference <checkout of alec-tschantz/jax-vllm>

The file holds the configuration, every weight, the token ids and the logits that
`jllm.model.qwen3.forward` returned, for two small random Qwen3 models that differ
in every size.  tests/test_plain.py compares the plain implementation with it.
"""

from __future__ import annotations

import argparse
import dataclasses
import sys
import types
from pathlib import Path

import numpy as np


def install_numpy_stand_in() -> None:
    jnp = types.ModuleType("jax.numpy")
    for name in dir(np):
        if not name.startswith("_"):
            setattr(jnp, name, getattr(np, name))
    jnp.bfloat16 = np.float32  # never used by this script; the name must exist

    nn = types.ModuleType("jax.nn")
    nn.silu = lambda x: x / (1.0 + np.exp(-x))

    def softmax(x, axis=-1):
        m = np.max(x, axis=axis, keepdims=True)
        e = np.exp(x - m)
        return e / np.sum(e, axis=axis, keepdims=True)

    nn.softmax = softmax
    lax = types.ModuleType("jax.lax")
    lax.rsqrt = lambda x: (1.0 / np.sqrt(x)).astype(np.float32)

    jax = types.ModuleType("jax")
    jax.Array = np.ndarray
    jax.numpy = jnp
    jax.nn = nn
    jax.lax = lax

    eqx = types.ModuleType("equinox")

    class Module:
        def __init_subclass__(cls, **kw):
            super().__init_subclass__(**kw)
            dataclasses.dataclass(cls)

    eqx.Module = Module
    eqx.filter_jit = lambda f=None, **kw: f if f is not None else (lambda g: g)
    sys.modules.update(
        {"jax": jax, "jax.numpy": jnp, "jax.nn": nn, "jax.lax": lax, "equinox": eqx}
    )


CONFIGS = {
    "a": dict(vocab_size=96, hidden_size=32, intermediate_size=80, num_hidden_layers=2,
              num_heads=4, num_kv_heads=2, head_dim=8, rms_norm_eps=1e-6, rope_theta=10000.0,
              max_position_embeddings=128, tie_word_embeddings=True),
    "b": dict(vocab_size=72, hidden_size=48, intermediate_size=56, num_hidden_layers=3,
              num_heads=6, num_kv_heads=1, head_dim=16, rms_norm_eps=1e-5, rope_theta=1e6,
              max_position_embeddings=64, tie_word_embeddings=False),
}
SEEDS = {"a": 11, "b": 12}
LENGTHS = {"a": 21, "b": 19}


def tensor_shapes(c: dict) -> dict[str, tuple]:
    H, I, D = c["hidden_size"], c["intermediate_size"], c["head_dim"]
    Hq, Hkv = c["num_heads"], c["num_kv_heads"]
    shapes = {"model.embed_tokens.weight": (c["vocab_size"], H), "model.norm.weight": (H,)}
    if not c["tie_word_embeddings"]:
        shapes["lm_head.weight"] = (c["vocab_size"], H)
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}"
        shapes.update({
            f"{p}.self_attn.q_proj.weight": (Hq * D, H),
            f"{p}.self_attn.k_proj.weight": (Hkv * D, H),
            f"{p}.self_attn.v_proj.weight": (Hkv * D, H),
            f"{p}.self_attn.o_proj.weight": (H, Hq * D),
            f"{p}.self_attn.q_norm.weight": (D,),
            f"{p}.self_attn.k_norm.weight": (D,),
            f"{p}.mlp.gate_proj.weight": (I, H),
            f"{p}.mlp.up_proj.weight": (I, H),
            f"{p}.mlp.down_proj.weight": (H, I),
            f"{p}.input_layernorm.weight": (H,),
            f"{p}.post_attention_layernorm.weight": (H,),
        })
    return shapes


def random_weights(c: dict, seed: int) -> dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(c).items():
        z = rng.standard_normal(shape).astype(np.float32)
        # matrices N(0, 0.3) so that attention is far from uniform; norms 1 + N(0, 0.1)
        out[name] = (1.0 + 0.1 * z) if len(shape) == 1 else 0.3 * z
    return out


def build_reference_model(c: dict, w: dict[str, np.ndarray]):
    from jllm.model import common as cm
    from jllm.model.qwen3 import Qwen3Config, Qwen3Model

    eps = c["rms_norm_eps"]
    lin = lambda n: cm.Linear(weight=w[n], bias=None)
    rms = lambda n: cm.RMSNorm(weight=w[n], eps=eps)
    layers = []
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}"
        layers.append(cm.DecoderLayer(
            self_attn=cm.Attention(
                q_proj=lin(f"{p}.self_attn.q_proj.weight"), k_proj=lin(f"{p}.self_attn.k_proj.weight"),
                v_proj=lin(f"{p}.self_attn.v_proj.weight"), o_proj=lin(f"{p}.self_attn.o_proj.weight"),
                q_norm=rms(f"{p}.self_attn.q_norm.weight"), k_norm=rms(f"{p}.self_attn.k_norm.weight"),
                num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"], head_dim=c["head_dim"]),
            mlp=cm.SwiGLU(gate_proj=lin(f"{p}.mlp.gate_proj.weight"), up_proj=lin(f"{p}.mlp.up_proj.weight"),
                          down_proj=lin(f"{p}.mlp.down_proj.weight")),
            input_layernorm=rms(f"{p}.input_layernorm.weight"),
            post_attention_layernorm=rms(f"{p}.post_attention_layernorm.weight")))
    embed = cm.Embedding(weight=w["model.embed_tokens.weight"])
    head = embed.weight if c["tie_word_embeddings"] else w["lm_head.weight"]
    cfg = Qwen3Config(**c)
    return Qwen3Model(embed_tokens=embed, layers=layers, norm=rms("model.norm.weight"),
                      rotary_emb=cm.RotaryEmbedding(dim=c["head_dim"], theta=c["rope_theta"]),
                      lm_head=cm.Linear(weight=head, bias=None), cfg=cfg)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of alec-tschantz/jax-vllm")
    ap.add_argument("--out", default=str(Path(__file__).with_name("qwen3_reference_logits.npz")))
    args = ap.parse_args()
    install_numpy_stand_in()
    sys.path.insert(0, args.reference)
    from jllm.model.qwen3 import forward

    blob = {}
    for tag, c in CONFIGS.items():
        w = random_weights(c, SEEDS[tag])
        ids = np.random.default_rng(SEEDS[tag] + 100).integers(0, c["vocab_size"], LENGTHS[tag])
        model = build_reference_model(c, w)
        logits = np.asarray(forward(model, ids[None, :].astype(np.int32)))[0]
        assert logits.dtype == np.float32 and logits.shape == (LENGTHS[tag], c["vocab_size"])
        blob[f"{tag}/ids"] = ids.astype(np.int32)
        blob[f"{tag}/logits"] = logits
        for name, arr in w.items():
            blob[f"{tag}/w/{name}"] = arr
        for key, val in c.items():
            blob[f"{tag}/cfg/{key}"] = np.asarray(val)
    np.savez_compressed(args.out, **blob)
    print("wrote", args.out, Path(args.out).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
