"""Long sequences at a real head size, window and ring: what the tiny configurations cannot reach.

Two layers (one with a window of 4,096 keys, one that keeps all keys), heads of 256 columns, everything else
small, so that the plain implementation can run 9,300 tokens on the CPU.  One sequence is fed as a prompt of 5,000
tokens, a piece of 2,048, a piece of 2,052 (more than the window layer's ring has room for in one pass: the step
function cuts it), then 200 single tokens; a second sequence joins as a prompt of 4,000 tokens beside the first
one's piece, goes on by a piece of 100 and then by single tokens across position 4,096, where its window begins to
slide.  The ring of the window layer (96 pages) wraps for the first sequence.  In bfloat16 this runs the tcgen05
prompt kernel, the tcgen05 chunk kernel over thousands of keys, and the decode kernel with its keys split over
clusters; in 32-bit the plain kernels.  Every logit row asked for is compared with the plain implementation on
the whole sequence.  A page that was dropped, read twice or read from the wrong place would move a logit by a
hundredth or more, far above the 32-bit tolerance.
"""
import random

import pytest
import torch

from plain import gemma2_plain as P
from test_real_widths_gpu import TensorSource, make_weights

pytestmark = pytest.mark.gpu

RAW = dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", vocab_size=500, rope_theta=10000.0,
           sliding_window=4096, max_position_embeddings=16384, attn_logit_softcapping=50.0,
           final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True, num_hidden_layers=2,
           hidden_size=128, num_attention_heads=2, num_key_value_heads=1, head_dim=256, intermediate_size=256,
           query_pre_attn_scalar=256)
TOL = {"float32": dict(atol=1e-4, rtol=1e-4), "bfloat16": dict(atol=2.5e-2, rtol=2.5e-2)}


def close(got, want, dtype, what):
    got, want = got.float().cpu(), want.float()
    err = (got - want).abs()
    bound = TOL[dtype]["atol"] + TOL[dtype]["rtol"] * want.abs()
    assert bool((err <= bound).all()), f"{what}: largest error {float(err.max()):.5f} on logits up to {float(want.abs().max()):.2f}"
    return float(err.max())


# head sizes and groups: 256 and 128 with two query heads per kv head (the prompt kernel on pairs of SMs), 64 with
# three (the one-SM kernel); the 32-bit path once
@pytest.mark.parametrize("dtype,heads", [("float32", (2, 1, 256)), ("bfloat16", (2, 1, 256)), ("bfloat16", (4, 2, 128)),
                                         ("bfloat16", (3, 1, 64))])
def test_long_sequences_through_the_window_ring_and_in_pieces(dtype, heads):
    from hos_b200.engine import Runner
    from hos_b200.registry import config_from_dict
    from hos_b200 import models  # noqa: F401
    raw = dict(RAW, num_attention_heads=heads[0], num_key_value_heads=heads[1], head_dim=heads[2],
               query_pre_attn_scalar=heads[2])
    config = config_from_dict(raw)
    weights = make_weights(config, 3)
    # attention that is not diffuse: larger q and k projections, so that single keys matter
    for name in list(weights):
        if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
            weights[name] = (weights[name].float() * 6.0).to(torch.bfloat16)
    pcfg = P.PlainConfig.from_json(raw)
    pw = {k: v.float().cpu() for k, v in weights.items()}
    rng = random.Random(9)
    seq_a = [rng.randrange(500) for _ in range(9300)]
    seq_b = [rng.randrange(500) for _ in range(4300)]
    with torch.no_grad():
        plain_a, plain_b = P.forward_logits(pw, pcfg, seq_a), P.forward_logits(pw, pcfg, seq_b)
    r = Runner(config, TensorSource(weights), dtype=dtype, max_tokens=9344 + 4352, max_seq_len=16384)
    assert r.cache.chunk_room() == 2049
    worst = 0.0
    a, = r.admit(1)
    got = r.step([a], [seq_a[:5000]], [[0, 2500, 4095, 4096, 4999]])
    worst = max(worst, close(got, plain_a[[0, 2500, 4095, 4096, 4999]], dtype, "prompt of 5,000"))
    b, = r.admit(1)
    got = r.step([a, b], [seq_a[5000:7048], seq_b[:4000]], [[0, 1000, 2047], [0, 3999]])
    want = torch.cat([plain_a[[5000, 6000, 7047]], plain_b[[0, 3999]]])
    worst = max(worst, close(got, want, dtype, "a piece of 2,048 beside a prompt of 4,000"))
    got = r.step([a, b], [seq_a[7048:9100], seq_b[4000:4100]], [[0, 2048, 2049, 2051], [0, 99]])
    want = torch.cat([plain_a[[7048, 9096, 9097, 9099]], plain_b[[4000, 4099]]])
    worst = max(worst, close(got, want, dtype, "a piece of 2,052 (two passes) beside a piece of 100"))
    for t in range(200):
        got = r.step([a, b], [[seq_a[9100 + t]], [seq_b[4100 + t]]])
        want = torch.stack([plain_a[9100 + t], plain_b[4100 + t]])
        worst = max(worst, close(got, want, dtype, f"single tokens, step {t}"))
    r.wait()
    assert r.length(a) == 9300 and r.length(b) == 4300
    r.cache.check()
    print(f"[long context {dtype} heads {heads}] largest error {worst:.6f}")
