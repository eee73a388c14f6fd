"""The assembled model at the layer widths of real checkpoints against the plain implementation.

The tiny configurations never reach the kernels that only run at real widths inside the
engine: the product on pairs of SMs with K = 9,216 or 36,864 and its rotary epilogue at heads
of 256 and 128 columns, K-split partial sums added by the norm kernel, prompt attention on
pairs of SMs, decode attention whose shares merge as a cluster, the chunk attention at these
head sizes.  Here a few layers of Gemma-2 2B widths and of 27B widths (small vocabulary, a
window of 300 so that it is crossed) run a ragged batch of prompts, then 40 single-token steps,
then a piece of 70 tokens per sequence, in 32-bit and in bfloat16, and every logit row asked for
is compared with the plain implementation on the whole sequence.

Weights are made on the GPU by the test and handed to the engine through a tensor source of its
own, and to the plain implementation as float32 copies: no files.

Tolerances, fixed before the first run.  32-bit: sums of K terms in another order differ by
about sqrt(K) roundings; the tiny models (K up to 264) are held to 1e-5, so K = 36,864 gets
sqrt(36864 / 264) = 12 times that, rounded up: 2e-4.  bfloat16: every operand of a product is
rounded to 8 bits (relative 2^-9); with random signs the relative error of a product does not
grow with K, but it adds up over the products of a layer and over layers, and a logit is a sum
over the width of rounded terms: observed once at these widths against the engine's own 32-bit
path, rms 0.006 to 0.009 and at most 0.054 on logits of size up to 29.  Held to atol 8e-2,
rtol 2.5e-2, and to an rms of 2e-2.
"""
import random

import pytest
import torch

from plain import gemma2_plain as P

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", vocab_size=2000, rope_theta=10000.0,
            sliding_window=300, max_position_embeddings=2048, attn_logit_softcapping=50.0,
            final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True)
WIDTHS = {
    "2b": dict(BASE, num_hidden_layers=4, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4,
               head_dim=256, intermediate_size=9216, query_pre_attn_scalar=256),
    "27b": dict(BASE, num_hidden_layers=2, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
                head_dim=128, intermediate_size=36864, query_pre_attn_scalar=144),
}
TOL = {"float32": dict(atol=2e-4, rtol=2e-4, rms=2e-5), "bfloat16": dict(atol=8e-2, rtol=2.5e-2, rms=2e-2)}


class TensorSource:
    """A tensor source (names / info / read / close, as a safetensors folder is one) over tensors
    that already exist."""

    def __init__(self, tensors):
        self.t = tensors

    def names(self):
        return list(self.t)

    def info(self, name):
        return self.t[name].dtype, tuple(self.t[name].shape)

    def read(self, name):
        return self.t[name]

    def close(self):
        pass


def make_weights(config, seed):
    from hos_b200.model import weight_specs_for
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = {}
    for s in weight_specs_for(config):
        if s.fallback is not None:
            continue                                  # the tied head: the embedding table is used
        t = torch.randn(tuple(s.shape), generator=g, device="cuda", dtype=torch.float32) * s.init_std
        out[s.name] = t.to(torch.bfloat16)
    return out


def check(got, want, dtype, what):
    tol = TOL[dtype]
    got, want = got.float().cpu(), want.float()
    err = (got - want).abs()
    bound = tol["atol"] + tol["rtol"] * want.abs()
    assert bool((err <= bound).all()), (f"{what}: {int((err > bound).sum())} of {err.numel()} logits differ, "
                                        f"largest error {float(err.max()):.4f} on logits up to {float(want.abs().max()):.1f}")
    rms = float((err ** 2).mean().sqrt())
    assert rms <= tol["rms"], f"{what}: rms error {rms:.5f}"
    return float(err.max()), rms


@pytest.mark.parametrize("name", ["2b", "27b"])
def test_real_widths_against_the_plain_implementation(name):
    from hos_b200.engine import Runner
    from hos_b200.registry import config_from_dict
    from hos_b200 import models  # noqa: F401
    raw = WIDTHS[name]
    config = config_from_dict(raw)
    weights = make_weights(config, 11)
    pcfg = P.PlainConfig.from_json(raw)
    pw = {k: v.float().cpu() for k, v in weights.items()}
    rng = random.Random(17)
    lens = [700, 333, 65]                                   # 1,098 rows: products on pairs of SMs
    n_decode, n_piece = 40, 70
    seqs = [[rng.randrange(raw["vocab_size"]) for _ in range(n + n_decode + n_piece)] for n in lens]
    with torch.no_grad():
        plain = [P.forward_logits(pw, pcfg, s) for s in seqs]
    assert max(float(p.abs().max()) for p in plain) > 5.0   # logits of ordinary size, not a degenerate model
    results = {}
    for dtype in ("float32", "bfloat16"):
        r = Runner(config, TensorSource(weights), dtype=dtype, max_tokens=3 * 1024, chunk_tokens=128)
        slots = r.admit(3)
        rows = []
        # the prompts, one ragged step; logits at the first place, in the middle, at the window's edge, at the end
        want = [sorted({0, n // 2, min(n - 1, 299), min(n - 1, 300), n - 1}) for n in lens]
        got = r.step(slots, [s[:n] for s, n in zip(seqs, lens)], want)
        exp = torch.cat([plain[i][want[i]] for i in range(3)])
        worst = [check(got, exp, dtype, f"{name} {dtype} prompts")]
        rows.append(got.float().cpu())
        # single-token steps (the shortest sequence leaves half-way: the batch shrinks)
        for t in range(n_decode):
            live = [i for i in range(3) if not (i == 2 and t >= n_decode // 2)]
            got = r.step([slots[i] for i in live], [[seqs[i][lens[i] + t]] for i in live])
            exp = torch.stack([plain[i][lens[i] + t] for i in live])
            worst.append(check(got, exp, dtype, f"{name} {dtype} decode step {t}"))
            rows.append(got.float().cpu())
        # a piece of 70 tokens on top of the two that are left, beside a new sequence that starts
        r.release(slots[2])
        slots[2] = r.admit(1)[0]
        starts = [lens[0] + n_decode, lens[1] + n_decode, 0]
        feeds = [seqs[0][starts[0]:starts[0] + n_piece], seqs[1][starts[1]:starts[1] + n_piece], seqs[2][:50]]
        want = [[0, 35, 69], [0, 69], [0, 49]]
        got = r.step(slots, feeds, want)
        exp = torch.cat([plain[i][[starts[i] + j for j in want[i]]] for i in range(3)])
        worst.append(check(got, exp, dtype, f"{name} {dtype} piece of 70 beside a new prompt"))
        rows.append(got.float().cpu())
        r.wait()
        r.cache.check()
        results[dtype] = torch.cat(rows)
        print(f"[real widths {name} {dtype}] largest error {max(w[0] for w in worst):.5f}, "
              f"largest rms {max(w[1] for w in worst):.6f}")
        del r
        torch.cuda.empty_cache()
    # the two paths of the engine against each other, on the same weights
    diff = (results["bfloat16"] - results["float32"]).abs()
    assert float(diff.max()) < 0.1 and float((diff ** 2).mean().sqrt()) < 2e-2
