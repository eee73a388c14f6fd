"""Trace replay on the GPU, through bin/trace_run as a user runs it, compared with
the plain implementation: each request alone and whole; with its last 32 tokens one
by one; in batches of unequal lengths whose shorter requests end earlier, one batch
after another so that slots and pages are used again; and fed in pieces of unequal
sizes, alone and in steps that other requests share (some starting, some going on by
one token, some by many).  In 32-bit and in bfloat16."""
import random

import pytest

from plain import gemma2_plain as P
from helpers import TINY, Trace, check_trace, make_folder, plain_model, random_tokens, run_trace

pytestmark = pytest.mark.gpu

# lengths chosen around what is special: 1 token, the window's size and one more, a page (64)
# and one more, and long enough that the window's ring of 64 positions wraps
LENGTHS = {"A": [1, 5, 8, 9, 33, 64, 65, 97], "B": [1, 9, 16, 17, 23, 40, 80, 128],
           "C": [2, 40, 41, 63, 129, 200, 333, 150],
           # head size 64 (permuted cache tiles, tcgen05 prompt attention): a window of 70 in a ring of two pages
           "D": [1, 64, 70, 71, 128, 129, 260, 400]}


def build(name):
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(100 + ord(name))
    reqs = [random_tokens(rng, n, vocab) for n in LENGTHS[name]]
    t = Trace()
    for i, r in enumerate(reqs):
        t.whole(f"w{i}", i, r)
    for i, r in enumerate(reqs):
        t.tail_one_by_one(f"t{i}", i, r)
    # batches: prompts are a part of each request, the rest is decoded; unequal all the way
    order = list(range(len(reqs)))
    rng.shuffle(order)
    for b, group in enumerate((order[:3], order[3:6], order[6:], order[1:5])):
        members = [(f"b{b}_{i}", i, reqs[i]) for i in group]
        plens = [max(1, len(reqs[i]) - rng.choice([0, 3, 32, 70])) for i in group]
        t.batch(members, plens)
    return reqs, t


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_matches_the_plain_implementation(tmp_path, name, dtype):
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    reqs, trace = build(name)
    expected = {i: P.forward_logits(w, cfg, r) for i, r in enumerate(reqs)}
    # a ring made for one more token per step: the shortest ring, which wraps soonest
    got = run_trace(folder, dtype, trace, str(tmp_path / "out"), extra_args=["--chunk-tokens", 1])
    check_trace(trace, got, expected, dtype)


PIECES = [1, 7, 64, 100, 3, 33]


def build_pieces(name):
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(200 + ord(name))
    reqs = [random_tokens(rng, n, vocab) for n in LENGTHS[name]]
    t = Trace()
    for i, r in enumerate(reqs):                      # each request alone, in pieces
        t.chunked(f"c{i}", i, r, PIECES[i % len(PIECES):] + PIECES[:i % len(PIECES)])
    # requests that share steps: one is still fed in pieces while others go on by one token, and
    # others join on the way (a step with sequences that start and sequences that go on)
    order = sorted(range(len(reqs)), key=lambda i: -len(reqs[i]))
    a = order[:4]
    t.mixed([(f"m{i}", i, reqs[i]) for i in a], joins=[0, 0, 2, 3],
            sizes=[[5, 40, 1, 1, 70], [len(reqs[a[1]]) // 2, 1], [9, 1, 1, 30], [1000]])
    b = order[2:]
    t.mixed([(f"n{i}", i, reqs[i]) for i in b], joins=[0, 1, 1, 2, 4, 5][:len(b)],
            sizes=[[3, 1], [1], [64, 1, 1], [1000], [2, 65], [17]][:len(b)])
    return reqs, t


@pytest.mark.parametrize("chunk_tokens", [24, 2048])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_in_pieces_matches_the_plain_implementation(tmp_path, name, dtype, chunk_tokens):
    """With --chunk-tokens 24 the rings of the window layers hold one or two pages, wrap all the
    time, and pieces of 64 and 100 tokens are more than they have room for (the step function
    feeds them in several passes); with 2048 (the default) every piece runs in one pass."""
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    reqs, trace = build_pieces(name)
    expected = {i: P.forward_logits(w, cfg, r) for i, r in enumerate(reqs)}
    got = run_trace(folder, dtype, trace, str(tmp_path / "out"), extra_args=["--chunk-tokens", chunk_tokens])
    check_trace(trace, got, expected, dtype)


SPECIAL_LENGTHS = [1, 2, 63, 64, 65, 127, 128, 129, 191, 192, 193, 256, 257]


def build_random(name, seed):
    """A schedule drawn from a seed: batches, requests fed in pieces, steps that starting and continuing requests
    share, and tails decoded one by one, over requests whose lengths lie on and around the pages' borders."""
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(seed * 1000 + ord(name))
    n_req = rng.randint(6, 12)
    lens = [rng.choice(SPECIAL_LENGTHS) if rng.random() < 0.4 else rng.randint(1, 420) for _ in range(n_req)]
    reqs = [random_tokens(rng, n, vocab) for n in lens]
    t = Trace()
    made = [0]

    def rid(prefix):
        made[0] += 1
        return f"{prefix}{made[0]}"

    for _ in range(rng.randint(5, 8)):
        kind = rng.choice(["batch", "batch", "mixed", "mixed", "chunked", "tail"])
        if kind == "batch":
            group = rng.sample(range(n_req), rng.randint(1, min(8, n_req)))
            plens = [max(1, len(reqs[i]) - rng.choice([0, 1, 3, 32, 70, 130])) for i in group]
            t.batch([(rid("b"), i, reqs[i]) for i in group], plens)
        elif kind == "mixed":
            group = rng.sample(range(n_req), rng.randint(2, min(6, n_req)))
            joins = [0] + [rng.randint(0, 5) for _ in group[1:]]
            sizes = [[rng.choice([1, 1, 1, 2, 5, 17, 40, 64, 65, 100, 1000]) for _ in range(rng.randint(1, 5))]
                     for _ in group]
            t.mixed([(rid("m"), i, reqs[i]) for i in group], joins, sizes)
        elif kind == "chunked":
            i = rng.randrange(n_req)
            t.chunked(rid("c"), i, reqs[i], [rng.choice([1, 3, 7, 33, 64, 100]) for _ in range(rng.randint(1, 4))])
        else:
            i = rng.randrange(n_req)
            t.tail_one_by_one(rid("t"), i, reqs[i], tail=rng.choice([1, 5, 32, 80]))
    return reqs, t, rng.choice([1, 24, 100, 2048])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
# these seeds draw rings made for 1, 100, 24 and 2,048 more tokens a step
@pytest.mark.parametrize("name,seed", [("A", 6), ("B", 4), ("C", 13), ("D", 9)])
def test_replay_of_a_drawn_schedule_matches_the_plain_implementation(tmp_path, name, seed, dtype):
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    reqs, trace, chunk_tokens = build_random(name, seed)
    expected = {i: P.forward_logits(w, cfg, r) for i, r in enumerate(reqs)}
    got = run_trace(folder, dtype, trace, str(tmp_path / "out"), extra_args=["--chunk-tokens", chunk_tokens])
    check_trace(trace, got, expected, dtype)
