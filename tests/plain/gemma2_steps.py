"""A second restatement of the reference's Gemma-2 arithmetic, in another shape: ONE token at a
time on top of a key/value cache, in numpy float32, with explicit loops over heads and keys.

`gemma2_plain.py` restates the prompt driver (src/forward.rs:247-438: whole sequences, no
cache, matrix products); this file restates the one-token driver (src/forward.rs:443-616) and
its primitives (src/forward.rs:166-234) line by line.  The two were written from different
parts of the reference and share no code; `tests/test_plain.py` asserts that they agree, which
is the reference's own invariant (src/forward.rs:242-245).  Like the other file it rests on the
formulas only (the reference cannot be built where these tests run) and adds the two things the
model family's config keys ask for: the attention scale `query_pre_attn_scalar ** -0.5`
(reference: 1/sqrt(head_dim), :503) and a window of `sliding_window` keys on even layers
(reference: all keys, :508).

Nothing here imports the library under test or the other plain file.
"""
from __future__ import annotations

import math
from typing import Dict, List

import numpy as np

F = np.float32


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """src/forward.rs:166-174 with add_one: ss = sum x^2 / n; y = x * (1/sqrt(ss + eps)) * (1 + w)."""
    ss = F(0.0)
    for v in x:
        ss = F(ss + v * v)
    ss = F(ss / F(len(x)))
    r = F(1.0) / np.sqrt(F(ss + F(eps)))
    return (x * r * (F(1.0) + w)).astype(F)


def gelu(g: np.ndarray) -> np.ndarray:
    """src/forward.rs:186-189."""
    c = F(math.sqrt(2.0 / math.pi))
    return (F(0.5) * g * (F(1.0) + np.tanh(c * (g + F(0.044715) * g * g * g)))).astype(F)


def softcap(v, c: float):
    """src/forward.rs:191-199."""
    return F(c) * np.tanh(v / F(c)) if c > 0.0 else v


def rope(v: np.ndarray, head_dim: int, pos: int, theta: float) -> None:
    """In place, every head of v.  src/forward.rs:203-222 with neox pairing (i, i + hd/2)."""
    half = head_dim // 2
    for h in range(len(v) // head_dim):
        for i in range(half):
            freq = F(1.0) / np.power(F(theta), F(2 * i) / F(head_dim), dtype=F)
            a = F(F(pos) * freq)
            s, c = F(np.sin(a)), F(np.cos(a))
            x0, x1 = v[h * head_dim + i], v[h * head_dim + i + half]
            v[h * head_dim + i] = F(x0 * c - x1 * s)
            v[h * head_dim + i + half] = F(x0 * s + x1 * c)


def softmax(s: np.ndarray) -> np.ndarray:
    """src/forward.rs:224-234."""
    e = np.exp(s - s.max()).astype(F)
    return (e / e.sum(dtype=F)).astype(F)


class Stepper:
    """State{k_cache, v_cache, pos} (src/forward.rs:146-162) and forward(token, pos) (:443-616)."""

    def __init__(self, weights: Dict[str, np.ndarray], cfg: dict, ctx: int):
        self.w = {k: np.asarray(v, dtype=F) for k, v in weights.items()}
        self.L = int(cfg["num_hidden_layers"])
        self.dim = int(cfg["hidden_size"])
        self.nh = int(cfg["num_attention_heads"])
        self.nkv = int(cfg.get("num_key_value_heads", self.nh))
        self.hd = int(cfg.get("head_dim", self.dim // self.nh))
        self.eps = float(cfg.get("rms_norm_eps", 1e-5))
        self.theta = float(cfg.get("rope_theta", 10000.0))
        self.window = int(cfg.get("sliding_window", 4096))
        self.scale = F(float(cfg.get("query_pre_attn_scalar", self.hd)) ** -0.5)
        self.attn_cap = float(cfg.get("attn_logit_softcapping") or 0.0)
        self.final_cap = float(cfg.get("final_logit_softcapping") or 0.0)
        kvd = self.nkv * self.hd
        self.k_cache = [np.zeros((ctx, kvd), dtype=F) for _ in range(self.L)]
        self.v_cache = [np.zeros((ctx, kvd), dtype=F) for _ in range(self.L)]
        self.pos = 0

    def forward(self, token: int) -> np.ndarray:
        w, hd, pos = self.w, self.hd, self.pos
        kv_mul = self.nh // self.nkv
        x = (w["model.embed_tokens.weight"][token] * np.sqrt(F(self.dim))).astype(F)          # :458-463
        for l in range(self.L):
            p = f"model.layers.{l}."
            xb = rmsnorm(x, w[p + "input_layernorm.weight"], self.eps)                        # :473
            q = (w[p + "self_attn.q_proj.weight"] @ xb).astype(F)                             # :475-477
            k = (w[p + "self_attn.k_proj.weight"] @ xb).astype(F)
            v = (w[p + "self_attn.v_proj.weight"] @ xb).astype(F)
            rope(q, hd, pos, self.theta)                                                      # :494-495
            rope(k, hd, pos, self.theta)
            self.k_cache[l][pos] = k                                                          # :498-501
            self.v_cache[l][pos] = v
            lo = max(0, pos + 1 - self.window) if l % 2 == 0 else 0      # even layers: the last `window` keys
            att = np.zeros(self.nh * hd, dtype=F)
            for h in range(self.nh):                                                          # :504-526
                kvh = h // kv_mul
                qh = q[h * hd:(h + 1) * hd]
                scores = np.empty(pos + 1 - lo, dtype=F)
                for t in range(lo, pos + 1):
                    kh = self.k_cache[l][t, kvh * hd:(kvh + 1) * hd]
                    dot = F(0.0)
                    for i in range(hd):
                        dot = F(dot + qh[i] * kh[i])
                    scores[t - lo] = softcap(F(dot * self.scale), self.attn_cap)
                pr = softmax(scores)
                oh = np.zeros(hd, dtype=F)
                for t in range(lo, pos + 1):
                    oh += pr[t - lo] * self.v_cache[l][t, kvh * hd:(kvh + 1) * hd]
                att[h * hd:(h + 1) * hd] = oh
            a = (w[p + "self_attn.o_proj.weight"] @ att).astype(F)                            # :528
            x = (x + rmsnorm(a, w[p + "post_attention_layernorm.weight"], self.eps)).astype(F)   # :530-536
            xb = rmsnorm(x, w[p + "pre_feedforward_layernorm.weight"], self.eps)              # :539
            gate = (w[p + "mlp.gate_proj.weight"] @ xb).astype(F)                             # :574-588
            up = (w[p + "mlp.up_proj.weight"] @ xb).astype(F)
            f = (w[p + "mlp.down_proj.weight"] @ (gelu(gate) * up).astype(F)).astype(F)
            x = (x + rmsnorm(f, w[p + "post_feedforward_layernorm.weight"], self.eps)).astype(F)  # :590-596
        xb = rmsnorm(x, w["model.norm.weight"], self.eps)                                     # :601
        head = w.get("lm_head.weight", w["model.embed_tokens.weight"])                        # src/model.rs:879-883
        logits = (head @ xb).astype(F)                                                        # :607-608
        if self.final_cap > 0.0:                                                              # :609-613
            logits = softcap(logits, self.final_cap).astype(F)
        self.pos = pos + 1                                                                    # :614
        return logits


def logits_token_by_token(weights: Dict[str, np.ndarray], cfg: dict, tokens: List[int]) -> np.ndarray:
    """[len(tokens), vocab]: the logits after each token, the sequence fed one token at a time."""
    st = Stepper(weights, cfg, len(tokens))
    return np.stack([st.forward(t) for t in tokens])
