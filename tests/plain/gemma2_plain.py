"""Plain, slow Gemma-2 forward pass: whole sequences, no cache, float32, CPU.

This file rests on the reference's formulas only: the reference (a Rust crate)
cannot be compiled or imported where these tests run (no Rust toolchain, no
network), so nothing here was compared against its binary.  Every function
cites the reference lines it restates.  Two things are not in the reference's
Gemma-2 path and follow the model family's config keys instead: the attention
scale `query_pre_attn_scalar ** -0.5` (the reference uses `1/sqrt(head_dim)`,
src/forward.rs:287, which is the same number whenever the key is absent) and
the sliding window on even layers (the reference attends to every earlier key,
src/forward.rs:342).

Nothing in this file imports the library under test.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass
class PlainConfig:
    """The numbers the forward pass needs, read from a config.json dict."""
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    sliding_window: int
    query_pre_attn_scalar: float
    attn_logit_softcapping: float
    final_logit_softcapping: float

    @staticmethod
    def from_json(cfg: dict) -> "PlainConfig":
        # defaults as in src/hf.rs:173-181 and src/model.rs:753-757
        nh = int(cfg["num_attention_heads"])
        hd = int(cfg.get("head_dim", int(cfg["hidden_size"]) // nh))
        return PlainConfig(
            num_hidden_layers=int(cfg["num_hidden_layers"]),
            hidden_size=int(cfg["hidden_size"]),
            num_attention_heads=nh,
            num_key_value_heads=int(cfg.get("num_key_value_heads", nh)),
            head_dim=hd,
            intermediate_size=int(cfg["intermediate_size"]),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            rope_theta=float(cfg.get("rope_theta", 10000.0)),
            sliding_window=int(cfg.get("sliding_window", 4096)),
            query_pre_attn_scalar=float(cfg.get("query_pre_attn_scalar", hd)),
            attn_logit_softcapping=float(cfg.get("attn_logit_softcapping") or 0.0),
            final_logit_softcapping=float(cfg.get("final_logit_softcapping") or 0.0),
        )


def embed(table: torch.Tensor, tokens: List[int], hidden: int) -> torch.Tensor:
    """x = E[token] * sqrt(hidden), the scale taken in float32.
    src/forward.rs:271-281, scale from src/model.rs:899."""
    scale = torch.tensor(float(hidden), dtype=torch.float32).sqrt()
    rows = table[torch.tensor(tokens, dtype=torch.long)].to(torch.float32)
    return rows * scale


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * (1 + w), row by row.
    src/forward.rs:166-174 with add_one (Gemma's convention, src/hf.rs:101-107)."""
    x = x.to(torch.float32)
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(ss + torch.tensor(eps, dtype=torch.float32))
    return x * scale * (w.to(torch.float32) + 1.0)


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))).  src/forward.rs:186-189."""
    c = torch.tensor(2.0 / math.pi, dtype=torch.float32).sqrt()
    return 0.5 * x * (1.0 + torch.tanh(c * (x + 0.044715 * x * x * x)))


def softcap(v: torch.Tensor, c: float) -> torch.Tensor:
    """c * tanh(v / c) when c > 0, else v.  src/forward.rs:193-199."""
    if c > 0.0:
        return c * torch.tanh(v / c)
    return v


def rope_rotate_half(v: torch.Tensor, positions: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """Rotate-half rotary encoding per head.  v: [T, heads, head_dim].
    freq_i = 1 / theta^(2i/head_dim); pairs (i, i + head_dim/2).
    src/forward.rs:203-222 with neox = true (src/model.rs:80-82)."""
    half = head_dim // 2
    i = torch.arange(half, dtype=torch.float32)
    freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2.0 * i / float(head_dim))
    angle = positions.to(torch.float32)[:, None] * freq[None, :]          # [T, half]
    s, c = torch.sin(angle)[:, None, :], torch.cos(angle)[:, None, :]
    x0, x1 = v[..., :half], v[..., half:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def softmax_rows(x: torch.Tensor) -> torch.Tensor:
    """exp(x - max) / sum, over the last axis.  src/forward.rs:224-234."""
    m = x.max(dim=-1, keepdim=True).values
    e = torch.exp(x - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: float,
              window: Optional[int]) -> torch.Tensor:
    """Causal (optionally windowed) grouped-query attention over a whole sequence.
    q: [T, nh, hd] and k, v: [T, nkv, hd], already rotated.
    Scores (q.k)*scale, soft-capped, softmax over the visible keys, weighted sum
    of values; query head h reads kv head h // (nh/nkv).
    src/forward.rs:336-361 (head map :340, cap :348).  The window keeps keys
    t in [max(0, pos+1-W), pos]."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    pos = torch.arange(T)
    visible = pos[None, :] <= pos[:, None]
    if window is not None:
        visible &= pos[None, :] > (pos[:, None] - window)
    out = torch.empty(T, nh, hd, dtype=torch.float32)
    for h in range(nh):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        s = softcap((q[:, h, :] @ kh.T) * scale, cap)
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h, :] = softmax_rows(s) @ vh
    return out


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = W x with W stored [out, in].  src/model.rs:179-180, src/forward.rs:300-302."""
    return x @ w.to(torch.float32).T


def attention_block(x, w: Dict[str, torch.Tensor], prefix: str, cfg: PlainConfig, layer: int,
                    positions: torch.Tensor) -> torch.Tensor:
    """input norm -> q,k,v -> rotary -> attention -> o_proj.  src/forward.rs:291-363."""
    T = x.shape[0]
    h = rmsnorm(x, w[prefix + "input_layernorm.weight"], cfg.rms_norm_eps)
    q = linear(h, w[prefix + "self_attn.q_proj.weight"]).view(T, cfg.num_attention_heads, cfg.head_dim)
    k = linear(h, w[prefix + "self_attn.k_proj.weight"]).view(T, cfg.num_key_value_heads, cfg.head_dim)
    v = linear(h, w[prefix + "self_attn.v_proj.weight"]).view(T, cfg.num_key_value_heads, cfg.head_dim)
    q = rope_rotate_half(q, positions, cfg.head_dim, cfg.rope_theta)
    k = rope_rotate_half(k, positions, cfg.head_dim, cfg.rope_theta)
    window = cfg.sliding_window if layer % 2 == 0 else None
    scale = float(torch.tensor(cfg.query_pre_attn_scalar, dtype=torch.float32) ** -0.5)
    att = attention(q, k, v, scale, cfg.attn_logit_softcapping, window)
    return linear(att.reshape(T, -1), w[prefix + "self_attn.o_proj.weight"])


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(gelu(gate(h)) * up(h)).  src/forward.rs:384-398."""
    g = linear(h, w[prefix + "mlp.gate_proj.weight"])
    u = linear(h, w[prefix + "mlp.up_proj.weight"])
    return linear(gelu_tanh(g) * u, w[prefix + "mlp.down_proj.weight"])


def forward_hidden(weights: Dict[str, torch.Tensor], cfg: PlainConfig, tokens: List[int]) -> torch.Tensor:
    """The residual stream after the last layer, [T, hidden].  src/forward.rs:271-415."""
    T = len(tokens)
    positions = torch.arange(T)
    x = embed(weights["model.embed_tokens.weight"], tokens, cfg.hidden_size)
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        a = attention_block(x, weights, p, cfg, l, positions)
        x = x + rmsnorm(a, weights[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)   # :364-373
        h = rmsnorm(x, weights[p + "pre_feedforward_layernorm.weight"], cfg.rms_norm_eps)      # :375-383
        f = feed_forward(h, weights, p)
        x = x + rmsnorm(f, weights[p + "post_feedforward_layernorm.weight"], cfg.rms_norm_eps)  # :399-414
    return x


def forward_logits(weights: Dict[str, torch.Tensor], cfg: PlainConfig, tokens: List[int]) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, vocab], float32.
    Final norm, head (the embedding table again unless lm_head.weight exists),
    final soft-cap.  src/forward.rs:417-435, tie rule src/model.rs:879-883."""
    x = forward_hidden(weights, cfg, tokens)
    h = rmsnorm(x, weights["model.norm.weight"], cfg.rms_norm_eps)
    head = weights.get("lm_head.weight", weights["model.embed_tokens.weight"])
    return softcap(linear(h, head), cfg.final_logit_softcapping)


# ---- sampling, restated from src/lib.rs:78-172 -------------------------------------------

def next_rand(state: int):
    """xorshift64 (13, 7, 17); top 24 bits -> [0, 1).  src/lib.rs:78-85."""
    mask = (1 << 64) - 1
    x = state
    x ^= (x << 13) & mask
    x ^= x >> 7
    x ^= (x << 17) & mask
    return x, float(x >> 40) / float(1 << 24)


def sample(logits: torch.Tensor, temp: float, top_k: int, top_p: float, rep_penalty: float,
           recent: List[int], rng: int):
    """Returns (token, new rng state).  src/lib.rs:91-172."""
    l = logits.to(torch.float32).clone()
    if rep_penalty != 1.0 and recent:
        for t in recent:
            if t < l.numel():
                l[t] = l[t] / rep_penalty if l[t] > 0 else l[t] * rep_penalty
    if temp <= 0.0:
        best = 0
        for i in range(1, l.numel()):
            if l[i] > l[best]:
                best = i
        return best, rng
    probs = torch.exp((l - l.max()) / temp)
    probs = probs / probs.sum()
    order = sorted(range(probs.numel()), key=lambda i: (-float(probs[i]), i))
    if 0 < top_k < len(order):
        order = order[:top_k]
    if top_p < 1.0:
        cum, cut = 0.0, len(order)
        cum = torch.tensor(0.0)
        for i, idx in enumerate(order):
            cum = cum + probs[idx]
            if float(cum) >= top_p:
                cut = i + 1
                break
        order = order[:cut]
    total = torch.tensor(0.0)
    for idx in order:
        total = total + probs[idx]
    rng, u = next_rand(rng)
    r = torch.tensor(u, dtype=torch.float32) * total
    cdf = torch.tensor(0.0)
    for idx in order:
        cdf = cdf + probs[idx]
        if float(r) < float(cdf):
            return idx, rng
    return order[-1], rng


def greedy_generate(weights, cfg: PlainConfig, prompt: List[int], max_new: int,
                    stop_ids=()) -> List[int]:
    """Greedy continuation by re-running the whole sequence for every token.
    The stop token ends the sequence and is not returned (src/lib.rs:456-457, :475-478)."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(max_new):
        nxt = int(torch.argmax(forward_logits(weights, cfg, ids)[-1]))
        if nxt in stop_ids:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
