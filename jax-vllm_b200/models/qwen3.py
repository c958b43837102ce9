"""Qwen3 dense: config.json -> typed configuration -> `ModelSpec`.

Keys and defaults are those the reference reads (jllm/model/qwen3.py:37-56): required
vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
rms_norm_eps, max_position_embeddings; num_key_value_heads defaults to the number of
heads, head_dim to hidden_size // heads, rope_theta to 1e6, tie_word_embeddings to
False.  The architecture is fixed where the reference fixes it: no bias on any
projection, RMSNorm of every query and key head before the rotation, the rotation over
the whole head, SiLU gating, full causal attention (jllm/model/weights.py:113-155,
jllm/model/common.py:107-147).  Keys of config.json that would ask for something else
(attention_bias, a rope_scaling, use_sliding_window, another hidden_act) are refused
rather than ignored.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from pathlib import Path

from ..config.model_spec import AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NormSpec, RopeSpec

ARCHITECTURE = "Qwen3ForCausalLM"
_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
             "rms_norm_eps", "max_position_embeddings")


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, c: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in c]
        if missing:
            raise KeyError(f"config.json lacks {missing} (required for {ARCHITECTURE})")
        contradictions = []
        if c.get("attention_bias"):
            contradictions.append("attention_bias=true (Qwen3 projections have no bias)")
        if c.get("rope_scaling") not in (None, {}):
            contradictions.append(f"rope_scaling={c['rope_scaling']!r} (only the plain rotation is built)")
        if c.get("use_sliding_window"):
            contradictions.append("use_sliding_window=true (Qwen3 dense attends to all earlier tokens)")
        if c.get("hidden_act", "silu") != "silu":
            contradictions.append(f"hidden_act={c['hidden_act']!r} (the gate is SiLU)")
        if contradictions:
            raise ValueError("config.json asks for what this architecture does not do: " + "; ".join(contradictions))
        heads = int(c["num_attention_heads"])
        cfg = cls(
            vocab_size=int(c["vocab_size"]), hidden_size=int(c["hidden_size"]),
            intermediate_size=int(c["intermediate_size"]), num_hidden_layers=int(c["num_hidden_layers"]),
            num_attention_heads=heads, num_key_value_heads=int(c.get("num_key_value_heads", heads)),
            head_dim=int(c.get("head_dim", int(c["hidden_size"]) // heads)),
            rms_norm_eps=float(c["rms_norm_eps"]), rope_theta=float(c.get("rope_theta", 1_000_000.0)),
            max_position_embeddings=int(c["max_position_embeddings"]),
            tie_word_embeddings=bool(c.get("tie_word_embeddings", False)))
        cfg.validate()
        return cfg

    @classmethod
    def from_path(cls, path) -> "Qwen3Config":
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        return cls.from_dict(json.loads(p.read_text()))

    def validate(self) -> None:
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, k) < 1:
                raise ValueError(f"{k} must be positive, got {getattr(self, k)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError(f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                             f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ValueError(f"head_dim={self.head_dim} must be even for the rotation")
        if not (self.rms_norm_eps > 0 and self.rope_theta > 0):
            raise ValueError("rms_norm_eps and rope_theta must be positive")

    def to_dict(self) -> dict:
        """config.json content for this configuration."""
        d = asdict(self)
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = "qwen3"
        d["hidden_act"] = "silu"
        d["attention_bias"] = False
        return d

    # ----------------------------------------------------------------- the model
    def to_spec(self) -> ModelSpec:
        eps = self.rms_norm_eps
        attn = AttentionSpec(
            hidden_size=self.hidden_size, num_heads=self.num_attention_heads, num_kv_heads=self.num_key_value_heads,
            head_dim=self.head_dim, scale=1.0 / math.sqrt(self.head_dim),
            position=RopeSpec(dim=self.head_dim, theta=self.rope_theta), qk_norm_eps=eps, window=None)
        mlp = GatedMLPSpec(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)
        layers = tuple(
            LayerSpec(prefix=f"model.layers.{i}", mixer=attn, feed_forward=mlp,
                      mixer_norm=NormSpec(self.hidden_size, eps, "input_layernorm.weight"),
                      ffn_norm=NormSpec(self.hidden_size, eps, "post_attention_layernorm.weight"))
            for i in range(self.num_hidden_layers))
        spec = ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab_size, hidden_size=self.hidden_size, layers=layers,
            final_norm=NormSpec(self.hidden_size, eps, "model.norm.weight"),
            lm_head_name=None if self.tie_word_embeddings else "lm_head.weight",
            max_position=self.max_position_embeddings)
        spec.validate()
        return spec
