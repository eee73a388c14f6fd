"""Shared by the tests: the two tiny configurations, model folders in temporary
directories, the plain implementation's view of a checkpoint, tolerances."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List

import torch

# Two tiny Gemma-2 configurations that differ in every size and option.
TINY_A = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=256, rope_theta=10000.0, sliding_window=8,
    max_position_embeddings=64, query_pre_attn_scalar=16, attn_logit_softcapping=50.0,
    final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True, eos_token_id=1)
TINY_B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
    intermediate_size=160, vocab_size=512, rope_theta=1000000.0, sliding_window=16,
    max_position_embeddings=128, query_pre_attn_scalar=24, attn_logit_softcapping=20.0,
    final_logit_softcapping=15.0, rms_norm_eps=1e-5, tie_word_embeddings=True, eos_token_id=[1, 7])
# A third one for long sequences: the window's ring (64 positions) wraps several times.
TINY_C = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
    intermediate_size=136, vocab_size=331, rope_theta=5000.0, sliding_window=40,
    max_position_embeddings=512, query_pre_attn_scalar=40, attn_logit_softcapping=30.0,
    final_logit_softcapping=0.0, rms_norm_eps=1e-6, tie_word_embeddings=True)

TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}

# Tolerances on logits against the plain float32 implementation.  Fixed up front:
# float32 differs by summation order only; bfloat16 rounds every activation that a
# matrix product reads (8 bits of mantissa) through a few layers.
TOL = {"float32": dict(atol=2e-4, rtol=2e-4), "bfloat16": dict(atol=4e-2, rtol=4e-2)}


def make_folder(tmp_path, name: str) -> str:
    """Write tiny config `name` with its seed's random weights; returns the folder."""
    from hos_b200.registry import config_from_dict
    from hos_b200 import models  # noqa: F401
    from hos_b200.weights import write_model_folder
    raw, seed = TINY[name]
    d = os.path.join(str(tmp_path), f"tiny_{name}")
    write_model_folder(config_from_dict(raw), seed, d)
    return d


def plain_model(folder: str):
    """(weights as float32 CPU tensors, PlainConfig), read with the safetensors package
    (not with the library under test)."""
    import safetensors.torch as st
    from plain.gemma2_plain import PlainConfig
    with open(os.path.join(folder, "config.json")) as f:
        cfg = PlainConfig.from_json(json.load(f))
    w = {k: v.to(torch.float32) for k, v in st.load_file(os.path.join(folder, "model.safetensors")).items()}
    return w, cfg


def random_tokens(rng: random.Random, n: int, vocab: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = ""):
    tol = TOL[dtype]
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    err = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    bad = err > bound
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} values differ; first at {idx}: "
                             f"got {got[tuple(idx)].item():.6f} want {want[tuple(idx)].item():.6f}; "
                             f"max abs err {err.max().item():.3e}")
