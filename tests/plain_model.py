"""A plain, slow implementation of the Qwen2 decoder: whole sequences, no cache, one function
for each part, on the CPU. It shares no code with the package: it reads config.json and
model.safetensors itself. Every function is written from the reference's formulas and cites
them as file:line of ktfth/smolmoe-c99.

The reference's own engine cannot serve as the oracle directly: it stores weights as Q8 and
re-quantizes every matrix input to Q8 (docs/FORMAT.md:152-159), so its logits are those of
another model. ``tests/golden/`` holds one loose comparison with it (see the header there);
everything else rests on the formulas below.

Conventions that differ from the reference on purpose, with the same mathematics:
* RoPE rotates pairs (i, i + R/2) of the checkpoint's own row order; the reference rotates
  adjacent pairs of rows that its converter permuted from that order
  (scripts/hf/permute.ts:14-28, src/model.c:439-450).
* Token ids are the checkpoint's (the reference remaps them for its tokenizer).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ---- reading the folder ------------------------------------------------------------------
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        return json.load(f)


def read_safetensors(path: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """8-byte length, JSON header, raw bytes (scripts/hf/safetensors.ts:73-111)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = np.frombuffer(blob, dtype=np.uint8, count=e - b, offset=8 + n + b)
        if info["dtype"] == "BF16":  # bf16 is the upper half of a float32 (scripts/hf/decode.ts)
            u16 = raw.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u16.view(np.float32).copy())
        elif info["dtype"] == "F32":
            t = torch.from_numpy(raw.view(np.float32).copy())
        elif info["dtype"] == "F16":
            t = torch.from_numpy(raw.view(np.float16).astype(np.float32))
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = t.reshape(info["shape"]).to(dtype)
    return out


# ---- the parts ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x_t = embed[token_t], no scaling for this architecture (src/model.c:667,671-679)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)].clone()


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """sq = sum x^2; inv = 1/sqrt(sq/n + eps); y = x*inv*w (src/model.c:334-342)."""
    sq = (x * x).sum(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(sq / x.shape[-1] + eps)
    return x * inv * w


def rope_tables(n: int, rotary_dim: int, theta: float):
    """inv_freq_i = theta^(-2i/R), angle = pos * inv_freq_i in double; cos and sin rounded
    to float (src/model.c:166-169,425-437)."""
    half = rotary_dim // 2
    inv_freq = [math.pow(float(theta), -(2.0 * i) / rotary_dim) for i in range(half)]
    cos = torch.empty(n, half, dtype=torch.float64)
    sin = torch.empty(n, half, dtype=torch.float64)
    for t in range(n):
        for i in range(half):
            cos[t, i] = math.cos(t * inv_freq[i])
            sin[t, i] = math.sin(t * inv_freq[i])
    return cos.float(), sin.float()


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """a' = a c - b s, b' = a s + b c on each pair (src/model.c:439-450); the pair of
    element i is element i + R/2 here (see the module header). x: [n, heads, head_dim]."""
    half = cos.shape[1]
    a, b = x[..., :half], x[..., half:2 * half]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    out = x.clone()
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = a * s + b * c
    return out


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int, kv_heads: int, window: Optional[int]) -> torch.Tensor:
    """For the query at position pos and head h: kv head h // (heads/kv_heads); keys from
    start to pos, start = pos - window + 1 once pos >= window (src/model.c:459-472);
    s_p = dot(q, K_p) / sqrt(head_dim); softmax with the maximum subtracted; weighted sum
    of the values (src/kernels.c:1138-1176). q: [n, heads, hd]; k, v: [n, kv_heads, hd]."""
    n, _, hd = q.shape
    factor = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    group = heads // kv_heads
    for pos in range(n):
        start = pos - window + 1 if (window and pos >= window) else 0
        for h in range(heads):
            kh = h // group
            scores = (k[start:pos + 1, kh] @ q[pos, h]) * factor
            e = torch.exp(scores - scores.max())
            out[pos, h] = (e / e.sum()) @ v[start:pos + 1, kh]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """up * (gate / (1 + exp(-gate))) (src/vecmath.c:78-81)."""
    return up * (gate / (1.0 + torch.exp(-gate)))


def attention_block(x, w, prefix, cfg, layer, cos, sin):
    """norm -> q,k,v with bias -> RoPE on q and k -> attention -> o projection -> residual
    (src/model.c:493-542)."""
    heads, kv_heads, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    n = x.shape[0]
    y = rmsnorm(x, w[f"{prefix}.input_layernorm.weight"], cfg["rms_norm_eps"])
    q = y @ w[f"{prefix}.self_attn.q_proj.weight"].T + w[f"{prefix}.self_attn.q_proj.bias"]
    k = y @ w[f"{prefix}.self_attn.k_proj.weight"].T + w[f"{prefix}.self_attn.k_proj.bias"]
    v = y @ w[f"{prefix}.self_attn.v_proj.weight"].T + w[f"{prefix}.self_attn.v_proj.bias"]
    q = rope(q.view(n, heads, hd), cos, sin)
    k = rope(k.view(n, kv_heads, hd), cos, sin)
    v = v.view(n, kv_heads, hd)
    att = attend(q, k, v, heads, kv_heads, layer_window(cfg, layer))
    return x + att.reshape(n, heads * hd) @ w[f"{prefix}.self_attn.o_proj.weight"].T


def ffn_block(x, w, prefix, cfg, act_store):
    """norm -> gate, up -> SwiGLU -> down -> residual (src/model.c:547-561,625-638)."""
    y = rmsnorm(x, w[f"{prefix}.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    if act_store is not None:
        y = act_store(y)
    h = swiglu(y @ w[f"{prefix}.mlp.gate_proj.weight"].T, y @ w[f"{prefix}.mlp.up_proj.weight"].T)
    if act_store is not None:
        h = act_store(h)
    return x + h @ w[f"{prefix}.mlp.down_proj.weight"].T


def head_dim_of(cfg: dict) -> int:
    """head_dim defaults to dim / heads (src/config.c:116-120)."""
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    """The sliding window of a layer, if any: layers from max_window_layers on see only the
    last sliding_window positions (window start as in src/model.c:462)."""
    if cfg.get("use_sliding_window") and layer >= cfg["max_window_layers"]:
        return cfg["sliding_window"]
    return None


def forward(model_dir: str, tokens: Sequence[int], *, compute=torch.float32, round_like_bf16_engine=False,
            weights: Optional[Dict[str, torch.Tensor]] = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of one whole sequence (src/model.c:664-690,654-662).

    ``round_like_bf16_engine`` rounds activations to bfloat16 at the places where the
    bfloat16 engine stores them (norm outputs, q/k/v, attention output, the gated
    activation), which makes the comparison with that engine tighter; the mathematics is
    unchanged."""
    cfg = read_config(model_dir)
    w = weights if weights is not None else read_safetensors(os.path.join(model_dir, "model.safetensors"), compute)
    n = len(tokens)
    store = (lambda t: t.to(torch.bfloat16).to(compute)) if round_like_bf16_engine else None
    cos, sin = rope_tables(n, head_dim_of(cfg), cfg["rope_theta"])
    x = embed(w["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        prefix = f"model.layers.{layer}"
        if store is not None:
            x = attention_block_rounded(x, w, prefix, cfg, layer, cos, sin, store)
        else:
            x = attention_block(x, w, prefix, cfg, layer, cos, sin)
        x = ffn_block(x, w, prefix, cfg, store)
    y = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    if store is not None:
        y = store(y)
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return y @ head.T


def attention_block_rounded(x, w, prefix, cfg, layer, cos, sin, store):
    """attention_block with the norm output rounded first, as the bfloat16 engine stores it."""
    heads, kv_heads, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    n = x.shape[0]
    y = store(rmsnorm(x, w[f"{prefix}.input_layernorm.weight"], cfg["rms_norm_eps"]))
    q = y @ w[f"{prefix}.self_attn.q_proj.weight"].T + w[f"{prefix}.self_attn.q_proj.bias"]
    k = y @ w[f"{prefix}.self_attn.k_proj.weight"].T + w[f"{prefix}.self_attn.k_proj.bias"]
    v = y @ w[f"{prefix}.self_attn.v_proj.weight"].T + w[f"{prefix}.self_attn.v_proj.bias"]
    q = store(rope(q.view(n, heads, hd), cos, sin))
    k = store(rope(k.view(n, kv_heads, hd), cos, sin))
    v = store(v.view(n, kv_heads, hd))
    att = store(attend(q, k, v, heads, kv_heads, layer_window(cfg, layer)))
    return x + att.reshape(n, heads * hd) @ w[f"{prefix}.self_attn.o_proj.weight"].T


# ---- sampling (src/sampler.c) ------------------------------------------------------------
def xorshift32(state: int) -> int:
    """src/sampler.c:48-55."""
    x = state & 0xFFFFFFFF
    x ^= (x << 13) & 0xFFFFFFFF
    x ^= x >> 17
    x ^= (x << 5) & 0xFFFFFFFF
    return x & 0xFFFFFFFF


def argmax(logits: Sequence[float], banned: Optional[Sequence[int]] = None) -> int:
    """The best allowed id; the lowest id wins ties (src/sampler.c:57-63)."""
    best = -1
    for i, l in enumerate(logits):
        if banned is not None and banned[i]:
            continue
        if best < 0 or l > logits[best]:
            best = i
    return best


def sample(logits: Sequence[float], temperature: float, top_k: int, top_p: float, state: int,
           banned: Optional[Sequence[int]] = None):
    """Returns (token, new state) (src/sampler.c:103-127): rank by (logit desc, id asc), keep
    top_k (0 or >= vocab: all), p = exp((l - l0)/T) in double, keep the shortest prefix with
    cumulative >= top_p * total, draw u = (xorshift32 >> 8) / 2^24, walk the prefix."""
    vocab = len(logits)
    if temperature == 0:
        return argmax(logits, banned), state
    ranked = sorted((i for i in range(vocab) if not (banned is not None and banned[i])),
                    key=lambda i: (-float(logits[i]), i))
    k = top_k if (top_k and top_k < vocab) else 0
    if k:
        ranked = ranked[:k]
    t = float(np.float32(temperature))
    probs = [math.exp((float(logits[i]) - float(logits[ranked[0]])) / t) for i in ranked]
    total = 0.0
    for p in probs:
        total += p
    kept = len(ranked)
    if float(np.float32(top_p)) < 1.0:
        cumulative = 0.0
        for i, p in enumerate(probs):
            cumulative += p
            if cumulative >= float(np.float32(top_p)) * total:
                kept = i + 1
                break
        total = cumulative
    state = xorshift32(state)
    target = (state >> 8) / 16777216.0 * total
    for i in range(kept):
        target -= probs[i]
        if target < 0:
            return ranked[i], state
    return ranked[kept - 1], state
