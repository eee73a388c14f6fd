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

# A fourth one with a head size of 64: the cache's permuted layout, the tcgen05 prompt attention and
# the tensor-core decode attention inside the engine (the sizes above use the other kernels).
TINY_D = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=2, hidden_size=136, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
    intermediate_size=264, vocab_size=1000, rope_theta=20000.0, sliding_window=70,
    max_position_embeddings=1024, query_pre_attn_scalar=50, attn_logit_softcapping=40.0,
    final_logit_softcapping=25.0, rms_norm_eps=1e-6, tie_word_embeddings=True)

# Head sizes 128 and 256 (what the 27B and the 2B/9B checkpoints have), small everywhere else.
TINY_E = dict(TINY_D, num_attention_heads=3, num_key_value_heads=1, head_dim=128, hidden_size=72,
              intermediate_size=200, query_pre_attn_scalar=144, sliding_window=100, vocab_size=777)
TINY_F = dict(TINY_D, num_attention_heads=2, num_key_value_heads=2, head_dim=256, hidden_size=104,
              intermediate_size=168, query_pre_attn_scalar=256, sliding_window=130, vocab_size=600,
              attn_logit_softcapping=50.0, final_logit_softcapping=30.0)

# Two query heads per kv head at head size 128: the prompt attention on pairs of SMs.
TINY_G = dict(TINY_D, num_attention_heads=4, num_key_value_heads=2, head_dim=128, hidden_size=88,
              intermediate_size=184, query_pre_attn_scalar=100, sliding_window=150, vocab_size=900,
              attn_logit_softcapping=30.0, final_logit_softcapping=0.0, rms_norm_eps=1e-5)

TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4), "F": (TINY_F, 5),
        "G": (TINY_G, 6)}

# Tolerances on logits against the plain float32 implementation.  Fixed up front:
# float32 differs by summation order only; bfloat16 rounds every activation that a
# matrix product reads (8 bits of mantissa) through a few layers.
TOL = {"float32": dict(atol=1e-5, rtol=1e-5), "bfloat16": dict(atol=2.5e-2, rtol=2.5e-2)}


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


# ---- building traces for bin/trace_run and checking what it wrote ---------------------------

class Trace:
    """Steps for the replay program, with a record of which (request, position) each
    written row is, and the largest number of tokens (each request rounded up to 64)
    that live requests hold at any time."""

    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[tuple]] = {}       # step -> [(request key, position)]
        self.live: Dict[str, int] = {}
        self.max_tokens = 0

    def step(self, entries, end=()):
        """entries: [(id, request key, tokens, first position, wanted places)]"""
        n = len(self.steps)
        self.steps.append({"step": n, "end": list(end), "entries": [
            {"id": i, "tokens": list(t), "want": list(w)} for i, _, t, _, w in entries]})
        rows = []
        for i, key, toks, start, want in entries:
            self.live[i] = start + len(toks)
            rows += [(key, start + j) for j in want]
        if rows:
            self.rows[n] = rows
        self.max_tokens = max(self.max_tokens, sum((v + 63) // 64 * 64 for v in self.live.values()))
        for i in end:
            del self.live[i]

    def whole(self, rid, key, tokens):
        self.step([(rid, key, tokens, 0, range(len(tokens)))], end=[rid])

    def tail_one_by_one(self, rid, key, tokens, tail=32):
        head = max(1, len(tokens) - tail)
        self.step([(rid, key, tokens[:head], 0, range(head))])
        for p in range(head, len(tokens)):
            self.step([(rid, key, tokens[p:p + 1], p, [0])], end=[rid] if p == len(tokens) - 1 else [])
        if head == len(tokens):
            self.step([], end=[rid])

    def batch(self, members, prompt_lens):
        """members: [(id, key, tokens)]; each starts with prompt_lens[i] tokens in one
        step, then all go on one token per step; a request leaves when its tokens end."""
        live = list(range(len(members)))
        ends = [members[m][0] for m in live if prompt_lens[m] == len(members[m][2])]
        self.step([(members[m][0], members[m][1], members[m][2][:prompt_lens[m]], 0,
                    range(prompt_lens[m])) for m in live], end=ends)
        pos = list(prompt_lens)
        live = [m for m in live if pos[m] < len(members[m][2])]
        while live:
            ends = [members[m][0] for m in live if pos[m] + 1 == len(members[m][2])]
            self.step([(members[m][0], members[m][1], members[m][2][pos[m]:pos[m] + 1], pos[m], [0])
                       for m in live], end=ends)
            for m in live:
                pos[m] += 1
            live = [m for m in live if pos[m] < len(members[m][2])]

    def chunked(self, rid, key, tokens, sizes):
        """One request fed in pieces of the given sizes (used round and round), every place wanted."""
        at, i = 0, 0
        while at < len(tokens):
            k = min(sizes[i % len(sizes)], len(tokens) - at)
            self.step([(rid, key, tokens[at:at + k], at, range(k))], end=[rid] if at + k == len(tokens) else [])
            at, i = at + k, i + 1

    def mixed(self, members, joins, sizes):
        """members: [(id, key, tokens)]; member m joins at step joins[m] of this run and from then
        on brings sizes[m][j] tokens in its j-th step (the list used round and round) until its
        tokens end: requests that start, requests that go on by many tokens and requests that
        go on by one share steps.  Every place is wanted."""
        at = [0] * len(members)
        turn = [0] * len(members)
        t = 0
        while any(at[m] < len(members[m][2]) for m in range(len(members))):
            entries, ends = [], []
            for m, (rid, key, toks) in enumerate(members):
                if joins[m] > t or at[m] >= len(toks):
                    continue
                k = min(sizes[m][turn[m] % len(sizes[m])], len(toks) - at[m])
                entries.append((rid, key, toks[at[m]:at[m] + k], at[m], range(k)))
                at[m] += k
                turn[m] += 1
                if at[m] == len(toks):
                    ends.append(rid)
            if entries:
                self.step(entries, end=ends)
            t += 1

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def run_trace(folder: str, dtype: str, trace: Trace, out_dir: str, timeout: int = 600,
              extra_args=()) -> Dict[int, torch.Tensor]:
    """Run bin/trace_run as a user would; returns {step: logits [wanted, vocab]}."""
    import subprocess
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(trace.max_tokens)] + [str(a) for a in extra_args]
    p = subprocess.run(cmd, input=trace.text().encode(), stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                       timeout=timeout)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stderr.decode()[-3000:]}"
    done = [l for l in p.stdout.decode().splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(trace.steps))], "a 'done <step>' line per step is expected"
    with open(os.path.join(folder, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for step, rows in trace.rows.items():
        arr = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
        assert arr.size == len(rows) * vocab, f"step {step}: {arr.size} floats for {len(rows)} rows"
        out[step] = torch.from_numpy(arr.reshape(len(rows), vocab).copy())
    written = {int(f[:-4]) for f in os.listdir(out_dir) if f.endswith(".f32")}
    assert written == set(trace.rows), "a file for exactly the steps that want something"
    return out


def check_trace(trace: Trace, got: Dict[int, torch.Tensor], expected: Dict[object, torch.Tensor], dtype: str):
    """expected[key]: plain logits [len, vocab] of the whole request `key`."""
    for step, rows in trace.rows.items():
        want = torch.stack([expected[key][pos] for key, pos in rows])
        try:
            assert_close(got[step], want, dtype, f"step {step}")
        except AssertionError as e:
            tol = TOL[dtype]
            err = (got[step] - want).abs() - (tol["atol"] + tol["rtol"] * want.abs())
            r = int((err.max(dim=1).values > 0).nonzero()[0])
            raise AssertionError(f"{e}\nfirst wrong row of step {step}: request {rows[r][0]!r} "
                                 f"position {rows[r][1]}; entries of the step: "
                                 f"{[(x['id'], len(x['tokens'])) for x in trace.steps[step]['entries']]}") from None
