"""Plain, slow, whole-sequence implementation of Qwen3 dense in 32-bit (on the CPU, or for
shapes of real size on the device that its tensors are moved to, with torch's float32
products and TF32 switched off by the caller).

This is the oracle that the engine is compared with.  It has no cache, no batching
and no kernels: one function for each part, each written from the formula that the
reference computes (cited as file:line within alec-tschantz/jax-vllm).  It shares no
code with the product package: it reads config.json keys and safetensors names
itself.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# --------------------------------------------------------------------------- config
def read_config(folder) -> dict:
    """config.json keys with the reference's defaults (jllm/model/qwen3.py:37-56)."""
    c = json.loads((Path(folder) / "config.json").read_text())
    heads = c["num_attention_heads"]
    return {
        "vocab_size": c["vocab_size"],
        "hidden_size": c["hidden_size"],
        "intermediate_size": c["intermediate_size"],
        "num_hidden_layers": c["num_hidden_layers"],
        "num_heads": heads,
        "num_kv_heads": c.get("num_key_value_heads", heads),
        "head_dim": c.get("head_dim", c["hidden_size"] // heads),
        "rms_norm_eps": c["rms_norm_eps"],
        "rope_theta": c.get("rope_theta", 1_000_000.0),
        "tie_word_embeddings": c.get("tie_word_embeddings", False),
    }


def read_weights(folder) -> dict[str, torch.Tensor]:
    """Every tensor of every *.safetensors shard, upcast to float32
    (jllm/model/weights.py:21-37)."""
    from safetensors import safe_open

    out = {}
    for shard in sorted(Path(folder).glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as f:
            for key in f.keys():
                out[key] = f.get_tensor(key).to(torch.float32)
    return out


# ---------------------------------------------------------------------------- parts
def embedding(weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Row gather, no scaling (jllm/model/common.py:35-36)."""
    return weight[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight, over the last axis
    (jllm/model/common.py:44-48)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * inv) * weight


def rope_cos_sin(positions: torch.Tensor, dim: int, theta: float):
    """inv_freq[j] = 1/theta^(2j/dim); angles = pos * inv_freq, repeated twice along
    the last axis (jllm/model/common.py:51-55)."""
    inv_freq = (1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))).to(positions.device)
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return torch.cos(emb), torch.sin(emb)


def rotate_half(u: torch.Tensor) -> torch.Tensor:
    """concat(-second half, first half) (jllm/model/common.py:58-60)."""
    half = u.shape[-1] // 2
    return torch.cat([-u[..., half:], u[..., :half]], dim=-1)


def apply_rope(u: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """u*cos + rotate_half(u)*sin; u is [heads, T, D], cos/sin [T, D]
    (jllm/model/common.py:63-66)."""
    return u * cos[None] + rotate_half(u) * sin[None]


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x @ W.T, no bias for Qwen3 (jllm/model/common.py:39-41,
    jllm/model/weights.py:124-127)."""
    return x @ weight.T


def causal_attention(q, k, v, num_heads, num_kv_heads, head_dim, window=None):
    """Grouped-query causal attention over a whole sequence.

    q: [Hq, T, D], k, v: [Hkv, T, D].  Query head h reads kv head h // (Hq/Hkv)
    (jllm/model/common.py:191-200); scores scaled by 1/sqrt(D), masked with -inf
    above the diagonal, softmax in 32-bit (jllm/model/common.py:173-178).  `window`
    (not part of the reference's Qwen3, used only for the toy architectures in the
    tests) keeps keys j with i - window < j <= i.
    """
    rep = num_heads // num_kv_heads
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    T = q.shape[1]
    scores = torch.einsum("hqd,hkd->hqk", q, k) * (1.0 / math.sqrt(head_dim))
    i = torch.arange(T, device=q.device)[:, None]
    j = torch.arange(T, device=q.device)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,hkd->hqd", probs, v)


def attention_block(x, w, prefix, cfg, positions, window=None):
    """q/k/v projections, per-head q/k RMSNorm before RoPE, attention, output
    projection (jllm/model/common.py:114-137; q/k norm :107-111)."""
    T = x.shape[0]
    Hq, Hkv, D = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    q = linear(x, w[f"{prefix}.q_proj.weight"]).reshape(T, Hq, D).transpose(0, 1)
    k = linear(x, w[f"{prefix}.k_proj.weight"]).reshape(T, Hkv, D).transpose(0, 1)
    v = linear(x, w[f"{prefix}.v_proj.weight"]).reshape(T, Hkv, D).transpose(0, 1)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = rope_cos_sin(positions, D, cfg["rope_theta"])
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, Hq, Hkv, D, window=window)
    o = o.transpose(0, 1).reshape(T, Hq * D)
    return linear(o, w[f"{prefix}.o_proj.weight"])


def swiglu(x, w, prefix):
    """down(silu(gate(x)) * up(x)) (jllm/model/common.py:75-76)."""
    g = linear(x, w[f"{prefix}.gate_proj.weight"])
    u = linear(x, w[f"{prefix}.up_proj.weight"])
    return linear(torch.nn.functional.silu(g) * u, w[f"{prefix}.down_proj.weight"])


def decoder_layer(h, w, i, cfg, positions):
    """Pre-norm block with two residual sums (jllm/model/common.py:140-147)."""
    p = f"model.layers.{i}"
    eps = cfg["rms_norm_eps"]
    h = h + attention_block(
        rms_norm(h, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", cfg, positions
    )
    h = h + swiglu(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    return h


def forward(cfg: dict, w: dict[str, torch.Tensor], token_ids) -> torch.Tensor:
    """Logits [T, vocab] for one whole sequence (jllm/model/common.py:150-170); the
    output matrix is the embedding table when tied (jllm/model/weights.py:142-146)."""
    dev = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(list(token_ids), dtype=torch.long, device=dev)
    positions = torch.arange(ids.shape[0], device=dev)
    h = embedding(w["model.embed_tokens.weight"], ids)
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, i, cfg, positions)
    h = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(h, head)


def greedy(cfg, w, prompt, max_new_tokens, eos_id=None) -> list[int]:
    """Greedy decoding by recomputing the whole sequence for every new token; stops
    after max_new_tokens or once eos_id was produced, the end token included
    (jllm/engine/engine.py:507-512)."""
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        tok = int(forward(cfg, w, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
        if eos_id is not None and tok == eos_id:
            break
    return out


class PlainModel:
    """A model folder read for the plain implementation."""

    def __init__(self, folder=None, round_to_bf16: bool = False, cfg: dict | None = None, weights: dict | None = None):
        """From a model folder, or from `cfg` (keys as `read_config` returns them) and a dict of float32 tensors
        by safetensors name, on whatever device they lie."""
        self.cfg = read_config(folder) if cfg is None else cfg
        self.w = read_weights(folder) if weights is None else weights
        if round_to_bf16:
            self.w = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in self.w.items()}

    def logits(self, token_ids) -> torch.Tensor:
        with torch.no_grad():
            return forward(self.cfg, self.w, token_ids)

    def greedy(self, prompt, max_new_tokens, eos_id=None):
        with torch.no_grad():
            return greedy(self.cfg, self.w, prompt, max_new_tokens, eos_id)
