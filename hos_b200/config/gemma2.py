"""Typed configuration of Gemma-2 (`Gemma2ForCausalLM`), read from its own
config.json keys.

Required keys and defaults follow the reference's reader (src/hf.rs:173-181:
hidden_size, num_hidden_layers, num_attention_heads, intermediate_size are
required; num_key_value_heads defaults to the head count,
max_position_embeddings to 2048, rms_norm_eps to 1e-5, rope_theta to 10000;
head_dim defaults to hidden/heads, src/model.rs:753-757; soft-caps are off when
absent, src/hf.rs:206-211).  `query_pre_attn_scalar` (default head_dim, which
reproduces the reference's 1/sqrt(head_dim), src/forward.rs:287) and
`sliding_window` (default 4096) are keys of the model family that the reference
does not read.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Mapping, Tuple

from ..errors import MissingMetaError
from .base import ConfigReader, ModelConfig


@dataclass(frozen=True)
class Gemma2Config(ModelConfig):
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    sliding_window: int = 4096
    query_pre_attn_scalar: float = 0.0      # 0 stands for "head_dim" until resolved in from_dict
    attn_logit_softcapping: float = 0.0     # 0 = off
    final_logit_softcapping: float = 0.0    # 0 = off
    tie_word_embeddings: bool = True
    bos_token_id: Tuple[int, ...] = ()
    eos_token_id: Tuple[int, ...] = ()

    architecture = "Gemma2ForCausalLM"
    model_type = "gemma2"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Gemma2Config":
        r = ConfigReader(raw)
        hidden = r.need_int("hidden_size")
        layers = r.need_int("num_hidden_layers")
        heads = r.need_int("num_attention_heads")
        inter = r.need_int("intermediate_size")
        vocab = r.need_int("vocab_size")
        kv_heads = r.opt_int("num_key_value_heads", heads)
        if heads <= 0:
            raise MissingMetaError("model metadata num_attention_heads must be positive")
        head_dim = r.opt_int("head_dim", hidden // heads)
        qpas = r.opt_float("query_pre_attn_scalar", float(head_dim))
        cfg = cls(
            num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
            vocab_size=vocab,
            max_position_embeddings=r.opt_int("max_position_embeddings", 2048),
            rms_norm_eps=r.opt_float("rms_norm_eps", 1e-5),
            rope_theta=r.opt_float("rope_theta", 10000.0),
            sliding_window=r.opt_int("sliding_window", 4096),
            query_pre_attn_scalar=qpas,
            attn_logit_softcapping=r.opt_float("attn_logit_softcapping", 0.0),
            final_logit_softcapping=r.opt_float("final_logit_softcapping", 0.0),
            tie_word_embeddings=r.opt_bool("tie_word_embeddings", True),
            bos_token_id=r.token_ids("bos_token_id"),
            eos_token_id=r.token_ids("eos_token_id"),
        )
        cfg.check()
        return cfg

    def check(self) -> None:
        def bad(msg: str):
            raise MissingMetaError("model metadata invalid: " + msg)
        for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings",
                    "sliding_window"):
            if getattr(self, key) <= 0:
                bad(f"{key} must be positive, found {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            bad(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            bad(f"head_dim ({self.head_dim}) must be even for the rotary encoding")
        if not self.rms_norm_eps > 0.0:
            bad("rms_norm_eps must be positive")
        if not self.rope_theta > 0.0:
            bad("rope_theta must be positive")
        if not self.query_pre_attn_scalar > 0.0:
            bad("query_pre_attn_scalar must be positive")
        if self.attn_logit_softcapping < 0.0 or self.final_logit_softcapping < 0.0:
            bad("soft-capping values must not be negative")

    def layer_is_sliding(self, layer: int) -> bool:
        """Even layers look at a window of keys, odd layers at all of them."""
        return layer % 2 == 0

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = self.model_type
        for key in ("bos_token_id", "eos_token_id"):
            ids = d[key]
            if len(ids) == 0:
                del d[key]
            elif len(ids) == 1:
                d[key] = ids[0]
            else:
                d[key] = list(ids)
        if self.attn_logit_softcapping == 0.0:
            d["attn_logit_softcapping"] = None
        if self.final_logit_softcapping == 0.0:
            d["final_logit_softcapping"] = None
        d["hidden_activation"] = "gelu_pytorch_tanh"
        d["torch_dtype"] = "bfloat16"
        return d
