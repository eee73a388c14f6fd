"""The plain implementation against closed forms and against its own invariants (no GPU)."""
import math
import random

import pytest
import torch

from plain import gemma2_plain as P
from helpers import TINY, make_folder, plain_model, random_tokens


def test_rmsnorm_closed_form():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([0.5, -1.0])
    y = P.rmsnorm(x, w, 0.0)                       # rms = sqrt(12.5)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3 / r * 1.5, 0.0]]), atol=1e-6)
    assert torch.allclose(P.rmsnorm(torch.zeros(1, 4), torch.zeros(4), 1e-6), torch.zeros(1, 4))


def test_gelu_softcap_softmax_closed_forms():
    assert P.gelu_tanh(torch.tensor(0.0)) == 0
    assert abs(float(P.gelu_tanh(torch.tensor(1.0))) - 0.841192) < 1e-5
    assert abs(float(P.gelu_tanh(torch.tensor(-3.0))) + 0.0036374) < 1e-5
    v = torch.tensor([100.0, -100.0, 0.1])
    c = P.softcap(v, 5.0)
    assert c[0] <= 5.0 and c[0] > 4.99 and c[1] >= -5.0 and abs(float(c[2]) - 5 * math.tanh(0.02)) < 1e-6
    assert torch.equal(P.softcap(v, 0.0), v)
    s = P.softmax_rows(torch.tensor([[0.0, math.log(3.0)]]))
    assert torch.allclose(s, torch.tensor([[0.25, 0.75]]), atol=1e-6)


def test_rope_rotates_pairs_by_position_times_frequency():
    hd, theta = 8, 100.0
    v = torch.zeros(3, 1, hd)
    v[:, 0, 1] = 1.0                                # pair (1, 5)
    out = P.rope_rotate_half(v, torch.tensor([0, 1, 7]), hd, theta)
    assert torch.allclose(out[0], v[0])            # position 0: untouched
    f = 1.0 / theta ** (2 * 1 / hd)
    for row, pos in ((1, 1), (2, 7)):
        assert abs(float(out[row, 0, 1]) - math.cos(pos * f)) < 1e-6
        assert abs(float(out[row, 0, 5]) - math.sin(pos * f)) < 1e-6
    # a rotation keeps norms, and q.k depends on the distance only
    q = torch.randn(1, 1, hd).repeat(6, 1, 1)
    k = torch.randn(1, 1, hd).repeat(6, 1, 1)
    qr = P.rope_rotate_half(q, torch.arange(6), hd, theta)
    kr = P.rope_rotate_half(k, torch.arange(6), hd, theta)
    assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    assert abs(float((qr[5] * kr[3]).sum() - (qr[2] * kr[0]).sum())) < 1e-4


def test_attention_masks_and_groups():
    torch.manual_seed(0)
    T, nh, nkv, hd = 12, 4, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, nkv, hd), torch.randn(T, nkv, hd)
    full = P.attention(q, k, v, 0.3, 0.0, None)
    assert torch.allclose(full[0, 0], v[0, 0], atol=1e-6)          # the first token sees itself only
    assert torch.allclose(full[0, 3], v[0, 1], atol=1e-6)          # head 3 reads kv head 1
    assert torch.allclose(P.attention(q, k, v, 0.3, 0.0, T), full)  # a window >= T changes nothing
    win = P.attention(q, k, v, 0.3, 0.0, 1)                         # window 1: each token sees itself
    assert torch.allclose(win[:, 0], v[:, 0], atol=1e-6)
    w3 = P.attention(q, k, v, 0.3, 0.0, 3)
    k2, v2 = k.clone(), v.clone()
    k2[:7], v2[:7] = 9.0, -9.0                                      # keys 0..6 are outside token 9's window
    assert torch.allclose(P.attention(q, k2, v2, 0.3, 0.0, 3)[9], w3[9], atol=1e-6)
    k2[7] = 5.0                                                     # key 7 is inside it
    assert not torch.allclose(P.attention(q, k2, v2, 0.3, 0.0, 3)[9], w3[9], atol=1e-4)


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_prefix_does_not_depend_on_what_follows(tmp_path, name):
    """Causality: the logits of the first n tokens are the same whether or not more
    tokens follow (the reference's 'prefill == token loop' invariant, src/forward.rs:242-245)."""
    w, cfg = plain_model(make_folder(tmp_path, name))
    vocab = TINY[name][0]["vocab_size"]
    toks = random_tokens(random.Random(1), 30, vocab)
    whole = P.forward_logits(w, cfg, toks)
    for n in (1, 9, 17, 25):
        assert torch.allclose(P.forward_logits(w, cfg, toks[:n]), whole[:n], atol=2e-6)


def test_window_larger_than_the_sequence_equals_no_window(tmp_path):
    w, cfg = plain_model(make_folder(tmp_path, "B"))
    toks = random_tokens(random.Random(2), 40, 512)
    a = P.forward_logits(w, cfg, toks)
    cfg.sliding_window = 4096
    b = P.forward_logits(w, cfg, toks)
    assert torch.allclose(a[:16], b[:16], atol=1e-6)        # the window (16) is not yet in force
    assert not torch.allclose(a[39], b[39], atol=1e-5)      # here it is


def test_scale_default_is_the_references(tmp_path):
    """query_pre_attn_scalar = head_dim gives the reference's 1/sqrt(head_dim) (src/forward.rs:287)."""
    cfg = P.PlainConfig.from_json(dict(num_hidden_layers=1, hidden_size=32, num_attention_heads=2,
                                       intermediate_size=8))
    assert cfg.query_pre_attn_scalar == 16 and cfg.head_dim == 16 and cfg.num_key_value_heads == 2
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0


def test_logits_are_capped(tmp_path):
    w, cfg = plain_model(make_folder(tmp_path, "B"))
    w = dict(w)
    w["model.embed_tokens.weight"] = w["model.embed_tokens.weight"] * 200.0     # huge logits
    out = P.forward_logits(w, cfg, [1, 2, 3])
    assert float(out.abs().max()) <= cfg.final_logit_softcapping + 1e-5
    assert float(out.abs().max()) > cfg.final_logit_softcapping * 0.9


def test_sampler_rules():
    logits = torch.tensor([1.0, 3.0, 3.0, 2.0, -1.0])
    assert P.sample(logits, 0.0, 0, 1.0, 1.0, [], 42)[0] == 1                 # first maximum wins
    assert P.sample(logits, 0.0, 0, 1.0, 2.0, [1], 42)[0] == 2                # penalty moves it
    assert P.sample(torch.tensor([-1.0, -3.0]), 0.0, 0, 1.0, 2.0, [0], 42)[0] == 0   # negative: times p
    assert P.sample(torch.tensor([-1.0, -1.5]), 0.0, 0, 1.0, 2.0, [0], 42)[0] == 1
    seen = set()
    rng = 42
    for _ in range(200):
        t, rng = P.sample(logits, 1.0, 2, 1.0, 1.0, [], rng)
        seen.add(t)
    assert seen == {1, 2}                                                      # top-2 only
    seen = set()
    for _ in range(200):
        t, rng = P.sample(logits, 1.0, 0, 0.5, 1.0, [], rng)                   # p(1)=p(2)~0.39: both needed
        seen.add(t)
    assert seen == {1, 2}
    seeds = [(s * 0x9E3779B97F4A7C15) & ((1 << 64) - 1) for s in range(1, 50)]   # small seeds draw ~0 first
    a = [P.sample(logits, 0.8, 0, 1.0, 1.0, [], s)[0] for s in seeds]
    b = [P.sample(logits, 0.8, 0, 1.0, 1.0, [], s)[0] for s in seeds]
    assert a == b and len(set(a)) > 2


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_two_restatements_agree(tmp_path, name):
    """The prompt driver restated with matrices on whole sequences (gemma2_plain.py, from
    src/forward.rs:247-438) and the one-token driver restated with loops on top of a cache
    (gemma2_steps.py, from src/forward.rs:443-616): two shapes of the same arithmetic, written
    apart, must give the same logits at every position (the reference's own invariant,
    src/forward.rs:242-245).  Lengths cross the windows (8 and 16 keys)."""
    import json
    import os
    from plain import gemma2_steps as S
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    with open(os.path.join(folder, "config.json")) as f:
        raw = json.load(f)
    vocab = raw["vocab_size"]
    tokens = random_tokens(random.Random(31), 27, vocab)
    whole = P.forward_logits(w, cfg, tokens)
    steps = S.logits_token_by_token({k: v.numpy() for k, v in w.items()}, raw, tokens)
    assert steps.shape == tuple(whole.shape)
    err = (torch.from_numpy(steps) - whole).abs().max()
    assert float(err) < 2e-5, f"the two restatements differ by {float(err):.2e}"
    assert float(whole.abs().max()) > 0.3            # and they are not trivially small
