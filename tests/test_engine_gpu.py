"""The step function and the Python entry point on the GPU against the plain implementation."""
import random

import pytest
import torch

from plain import gemma2_plain as P
from helpers import TINY, TOL, assert_close, make_folder, plain_model, random_tokens

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def runner_for(folder, dtype, max_tokens=4096, chunk_tokens=1):
    """chunk_tokens = 1: the window layers keep the shortest ring of pages, which wraps soonest (the library's
    default makes rings long enough for pieces of 2,048 tokens, which these short sequences would never fill)."""
    from hos_b200.engine import Runner
    return Runner.from_folder(folder, dtype=dtype, max_tokens=max_tokens, chunk_tokens=chunk_tokens)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(tmp_path, name, dtype):
    """Positions 0, 1, 2: a one-token prompt beside a two-token prompt, then single tokens."""
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(3)
    seqs = [random_tokens(rng, 4, vocab), random_tokens(rng, 5, vocab)]
    r = runner_for(folder, dtype)
    slots = r.admit(2)
    got = [r.step(slots, [seqs[0][:1], seqs[1][:2]], [[0], [0, 1]])]
    for t in range(3):
        got.append(r.step(slots, [[seqs[0][1 + t]], [seqs[1][2 + t]]]))
    want0, want1 = P.forward_logits(w, cfg, seqs[0]), P.forward_logits(w, cfg, seqs[1])
    assert_close(got[0], torch.stack([want0[0], want1[0], want1[1]]), dtype, "prompt step")
    for t in range(3):
        assert_close(got[1 + t], torch.stack([want0[1 + t], want1[2 + t]]), dtype, f"decode step {t}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_wraps_the_window_ring(tmp_path, dtype):
    """Config C keeps a window of 40 keys in a ring of 64 positions: decoding 300 tokens
    one by one goes round it more than four times, beside a sequence that is much shorter."""
    folder = make_folder(tmp_path, "C")
    w, cfg = plain_model(folder)
    rng = random.Random(4)
    long_seq, short_seq = random_tokens(rng, 310, 331), random_tokens(rng, 40, 331)
    r = runner_for(folder, dtype)
    a, b = r.admit(2)
    r.step([a, b], [long_seq[:7], short_seq[:3]])
    want_long, want_short = P.forward_logits(w, cfg, long_seq), P.forward_logits(w, cfg, short_seq)
    for t in range(7, 310):
        k = t - 7 + 3
        if k < 40:
            got = r.step([a, b], [[long_seq[t]], [short_seq[k]]])
            assert_close(got, torch.stack([want_long[t], want_short[k]]), dtype, f"position {t}/{k}")
        else:
            if k == 40:
                r.release(b)
            got = r.step([a], [[long_seq[t]]])
            assert_close(got, want_long[t][None], dtype, f"position {t}")
    r.release(a)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_rows_change_nothing(tmp_path, dtype):
    """The same batch with padding rows appended gives the same logits: bit for bit while the
    padded batch runs the same kernels (5 rows more), and within the engine's tolerance when
    padding takes a decode step from the few-rows kernels to the many-rows ones (64 more)."""
    from hos_b200.engine.batch import build_step
    folder = make_folder(tmp_path, "B")
    rng = random.Random(5)
    prompts = [random_tokens(rng, n, 512) for n in (3, 20, 19)]       # 42 rows: past the few-rows kernels
    outs = []
    for pad in (0, 5, 64):
        r = runner_for(folder, dtype)
        slots = r.admit(3)
        for s, p in zip(slots, prompts):
            r.cache.extend(s, len(p))
        r.cache.flush()
        n = sum(len(p) for p in prompts)
        info = build_step(prompts, [0, 0, 0], slots, r.device, 512, pad_to=n + pad if pad else 0)
        x = r.model.hidden(info, r.cache)
        rows = torch.arange(n, dtype=torch.int32, device=r.device)
        outs.append(r.model.logits(x, rows).cpu())
        # and a decode step on top, padded the same way
        info = build_step([[5], [6], [7]], [len(p) for p in prompts], slots, r.device, 512,
                          pad_to=3 + pad if pad else 0)
        for s, p in zip(slots, prompts):
            r.cache.extend(s, len(p) + 1)
        r.cache.flush()
        x = r.model.hidden(info, r.cache)
        outs.append(r.model.logits(x, torch.arange(3, dtype=torch.int32, device=r.device)).cpu())
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
    assert torch.equal(outs[0], outs[4])
    if dtype == "float32":
        assert torch.equal(outs[1], outs[5])
    else:
        assert_close(outs[5], outs[1], dtype, "decode step padded past the few-rows kernels")


def test_step_refuses_what_it_cannot_run(tmp_path):
    from hos_b200.errors import CacheError, HosError
    folder = make_folder(tmp_path, "A")
    r = runner_for(folder, "float32", max_tokens=128)
    a, b = r.admit(2)
    r.step([a], [[1, 2, 3]])
    with pytest.raises(HosError, match="outside the vocabulary"):
        r.step([a], [[256]])
    with pytest.raises(HosError, match="appears twice"):
        r.step([a, a], [[1], [2]])
    with pytest.raises(HosError, match="outside the 1 tokens"):
        r.step([a], [[1]], [[1]])
    with pytest.raises(CacheError):
        r.step([b], [list(range(65))])          # config A's context holds 64 positions
    assert r.length(a) == 3 and r.length(b) == 0      # refused steps left the cache as it was
    # all or nothing across the sequences of a step: the second one cannot be run, the first keeps its length
    # (the same for a sequence that finds no free page: tests/test_cache.py)
    pages_a = [len(g._slot_pages[a]) for g in r.cache.groups]
    with pytest.raises(CacheError, match="longer than the cache holds"):
        r.step([a, b], [[4], list(range(65))])
    assert r.length(a) == 3 and r.length(b) == 0
    assert [len(g._slot_pages[a]) for g in r.cache.groups] == pages_a
    r.cache.check()
    # a sequence that goes on by several tokens beside one that starts: one step
    out = r.step([a, b], [[4, 5], [6, 7, 8]], [[0, 1], [2]])
    assert out.shape == (3, 256) and r.length(a) == 5 and r.length(b) == 3


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    from hos_b200 import Engine
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(6)
    prompts = [random_tokens(rng, n, vocab) for n in (4, 1, 13, 7, 2)]
    eng = Engine(folder, dtype=dtype, max_batch=3)             # five requests: two batches
    outs = eng.generate_ids(prompts, 10, stop_ids=[])
    assert [len(o) for o in outs] == [10] * 5
    tol = TOL[dtype]
    for p, o in zip(prompts, outs):
        if dtype == "float32":
            assert o == P.greedy_generate(w, cfg, p, 10)
        else:
            # bfloat16 may pick another token only where the plain logits nearly tie
            seq = list(p)
            for t in o:
                l = P.forward_logits(w, cfg, seq)[-1]
                assert float(l.max() - l[t]) <= 2 * (tol["atol"] + tol["rtol"] * float(l.abs().max()))
                seq.append(t)
    # one request alone gives what it gave in the batch
    assert eng.generate_ids(prompts[2], 10, stop_ids=[]) == outs[2]
    # a stop token ends the sequence and is not returned
    stop = outs[0][4]
    cut = outs[0].index(stop)
    assert eng.generate_ids(prompts[0], 10, stop_ids=[stop]) == outs[0][:cut]
    eng.runner.cache.check()
    assert eng.runner.cache.slots.n_held == 0


def test_sampling_through_the_entry_point_follows_the_reference_rule(tmp_path):
    """temp, top-k, top-p and the repetition penalty together, in 32-bit, against the plain
    sampler fed with the plain logits and the same xorshift stream."""
    from hos_b200 import Engine
    folder = make_folder(tmp_path, "A")
    w, cfg = plain_model(folder)
    eng = Engine(folder, dtype="float32")
    prompts = [[5, 6, 7], [100, 3]]
    kw = dict(temp=0.9, top_k=12, top_p=0.9, rep_penalty=1.3, repeat_last_n=4, seed=0x1234567890ABCDEF)
    outs = eng.generate(prompts, 12, stop_ids=[], **kw)
    from hos_b200.sampling import stream_seed
    for i, (p, o) in enumerate(zip(prompts, outs)):
        rng = stream_seed(kw["seed"], i)
        seq, recent = list(p), []
        for t in o:
            l = P.forward_logits(w, cfg, seq)[-1]
            want, rng = P.sample(l, kw["temp"], kw["top_k"], kw["top_p"], kw["rep_penalty"],
                                 recent[-kw["repeat_last_n"]:], rng)
            assert t == want
            seq.append(t)
            recent.append(t)
    assert len({tuple(o) for o in outs}) == 2


def test_single_token_steps_take_their_position_from_the_device_record(tmp_path):
    """The host's count of a sequence's tokens hands out pages; the position a single-token step
    runs at is the one in the slot's record on the device.  Set the record back by five tokens
    behind the host's back: the next step's logits are those of the shorter sequence."""
    from hos_b200 import ops
    folder = make_folder(tmp_path, "B")
    w, cfg = plain_model(folder)
    r = runner_for(folder, "float32")
    ids = random_tokens(random.Random(3), 30, 512)
    a, b = r.admit(2)
    r.step([a, b], [ids[:24], ids[:9]])
    dev = r.device
    vals = torch.zeros((1, ops.SLOT_WORDS), dtype=torch.int32, device=dev)
    vals[0, ops.SLOT_POS] = 19
    ops.slot_write(r.cache.record, torch.tensor([a], dtype=torch.int32, device=dev), vals, 1 << ops.SLOT_POS)
    assert r.length(a) == 24                                    # the host still counts 24
    got = r.step([a, b], [[ids[25]], [ids[9]]])
    want_a = P.forward_logits(w, cfg, ids[:19] + [ids[25]])[-1]
    want_b = P.forward_logits(w, cfg, ids[:10])[-1]
    assert_close(got, torch.stack([want_a, want_b]), "float32", "record-driven step")
    rec = r.cache.record.cpu()
    assert int(rec[a, ops.SLOT_POS]) == 20 and int(rec[b, ops.SLOT_POS]) == 10


@pytest.mark.parametrize("dtype", DTYPES)
def test_conversations_continue_where_they_ended(tmp_path, dtype):
    """Turns on sequences that keep their slots (Engine.generate_from_ids): a turn that ends with
    all its tokens, a turn that ends at a stop token (one step had run for nothing by then), a long
    second prompt that the step function feeds in pieces; against the plain implementation run on
    the whole history each time."""
    from hos_b200 import Engine
    folder = make_folder(tmp_path, "D")
    w, cfg = plain_model(folder)
    eng = Engine(folder, dtype=dtype, max_batch=4)
    rng = random.Random(8)
    c1, c2 = eng.open(2)
    hist = [random_tokens(rng, 20, 1000), random_tokens(rng, 3, 1000)]
    first = eng.generate_from_ids([c1, c2], hist, max_tokens=6, temp=0.0, rep_penalty=1.0, stop_ids=[])
    want = [P.greedy_generate(w, cfg, h, 6) for h in hist]
    if dtype == "float32":
        assert first == want
    hist = [h + o for h, o in zip(hist, first)]
    assert c1.pending == first[0][-1] and c1.position == 20 + 5
    # second turn: a long prompt for one (more than a ring of the window layers has room for in one
    # pass: 70 keys of window in 2 + 8 pages... the step function decides), a short one for the other;
    # the second conversation stops at a token it would sample third
    turn = [random_tokens(rng, 700, 1000), random_tokens(rng, 2, 1000)]
    probe = P.greedy_generate(w, cfg, hist[1] + turn[1], 5)
    stop = probe[2]
    second = eng.generate_from_ids([c1, c2], turn, max_tokens=5, temp=0.0, rep_penalty=1.0, stop_ids=[stop])
    want = [P.greedy_generate(w, cfg, h + t, 5, stop_ids=[stop]) for h, t in zip(hist, turn)]
    if dtype == "float32":
        assert second == want and len(second[1]) == probe.index(stop)
    hist = [h + t + o for h, t, o in zip(hist, turn, second)]
    # after a stop token the conversation holds its history and nothing else
    if len(second[1]) < 5 and dtype == "float32":
        assert c2.pending is None and c2.position == len(hist[1])
    # third turn on the second conversation alone; the first is reset and starts afresh
    third = eng.generate_from_ids([c2], [[7, 8, 9]], max_tokens=4, temp=0.0, rep_penalty=1.0, stop_ids=[])
    if dtype == "float32":
        assert third == [P.greedy_generate(w, cfg, hist[1] + [7, 8, 9], 4)]
    else:
        seq = hist[1] + [7, 8, 9]
        for t in third[0]:                                       # bfloat16: each choice is (almost) the best one
            l = P.forward_logits(w, cfg, seq)[-1]
            assert float(l.max() - l[t]) < 0.1
            seq.append(t)
    c1.reset()
    again = eng.generate_from_ids([c1], [hist[0][:20]], max_tokens=6, temp=0.0, rep_penalty=1.0, stop_ids=[])
    assert again == [first[0]]
    c1.close()
    c2.close()
    eng.runner.cache.check()
    assert eng.runner.cache.slots.n_held == 0


def test_the_per_layer_tap_follows_the_plain_residual_stream(tmp_path):
    """`Runner.hidden_states`: the residual stream after the embedding and after every layer, against
    the plain implementation cut off after as many layers."""
    import dataclasses
    folder = make_folder(tmp_path, "B")
    w, cfg = plain_model(folder)
    r = runner_for(folder, "float32")
    ids = random_tokens(random.Random(12), 21, 512)
    slot = r.admit(1)[0]
    taps = r.hidden_states([slot], [ids])
    assert len(taps) == cfg.num_hidden_layers + 1
    for n, got in enumerate(taps):
        want = P.forward_hidden(w, dataclasses.replace(cfg, num_hidden_layers=n), ids)
        assert_close(got, want, "float32", f"residual stream after {n} layers")
    assert r.length(slot) == 21


def test_perplexity_and_bench(tmp_path):
    from hos_b200 import Engine
    folder = make_folder(tmp_path, "B")
    w, cfg = plain_model(folder)
    eng = Engine(folder, dtype="float32")
    ids = random_tokens(random.Random(7), 50, 512)
    n, mean, ppl = eng.perplexity(ids)
    logits = P.forward_logits(w, cfg, ids[:-1]).double()
    want = float(-(torch.log_softmax(logits, -1).gather(1, torch.tensor(ids[1:])[:, None])).mean())
    assert n == 49 and abs(mean - want) < 1e-5 and abs(ppl - torch.tensor(want).exp().item()) < 1e-2
    b = eng.bench(ids[:20], 5)
    assert b[0] == 20 and b[3] <= 5 and b[2] > 0 and (b[3] == 0 or b[5] > 0)
    b = eng.bench([ids[:20], ids[5:12], ids[30:31]], 4)           # a batch: tokens counted over it
    assert b[0] == 28 and b[3] <= 12 and b[2] > 0
    eng.runner.cache.check()
    assert not eng.runner.cache.lengths                            # every slot was given back


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_short_prompts_replayed_as_graphs_match_whole_prompts(tmp_path, name, dtype):
    """Prompt steps of up to 256 tokens run from static buffers as a replayed graph, one graph per
    capacity: batches of other lengths and other numbers of sequences reuse it (the rows beyond the
    real tokens are padding, the sequences beyond the real ones empty).  Every batch gives the plain
    implementation's logits, the decode steps on top find what the prompt step stored, and slots
    are reused from batch to batch."""
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(8)
    r = runner_for(folder, dtype)
    longest = TINY[name][0]["max_position_embeddings"] - 2
    batches = [[5], [16], [17, 3], [1, 1, 1], [30, 31, 2, 1], [9, 100, 40], [60] * 4, [33] * 7, [2, 250]]
    from hos_b200.engine.decode import prompt_bucket
    buckets = set()
    for lens in batches:
        lens = [min(n, longest) for n in lens]
        buckets.add(prompt_bucket(sum(lens), len(lens)))
        seqs = [random_tokens(rng, n + 2, vocab) for n in lens]
        want = [P.forward_logits(w, cfg, s) for s in seqs]
        slots = r.admit(len(seqs))
        got = r.step(slots, [s[:n] for s, n in zip(seqs, lens)])
        assert_close(got, torch.stack([wl[n - 1] for wl, n in zip(want, lens)]), dtype, f"prompt step {lens}")
        for t in range(2):
            got = r.step(slots, [[s[n + t]] for s, n in zip(seqs, lens)])
            assert_close(got, torch.stack([wl[n + t] for wl, n in zip(want, lens)]), dtype, f"decode {t} after {lens}")
        for s in slots:
            r.release(s)
        r.cache.check()
    used = {k[1:] for k in r._sessions if isinstance(k, tuple) and k[0] == "prompt"}
    assert used == buckets and len(used) >= 5           # nine batches, fewer graphs
    # the same steps launched kernel by kernel agree (other kernels for other row counts: within tolerance)
    r2 = runner_for(folder, dtype)
    r2.prompt_sessions = False
    seqs = [random_tokens(rng, n, vocab) for n in (30, 31, 2, 1)]
    s1, s2 = r.admit(4), r2.admit(4)
    assert_close(r.step(s1, seqs), r2.step(s2, seqs), dtype, "graph against kernel by kernel")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["D", "E", "F", "G"])
def test_head_sizes_64_128_256_whole_prompts_then_decoding(tmp_path, name, dtype):
    """Configs D to G (head sizes 64, 128, 256; one, two or three query heads per kv head; a window in a
    ring of two or three pages): prompts of 644 tokens in all that span several blocks of 128 queries
    in one batch (in bfloat16 the products on pairs of SMs with rotation and cache write in the q/k/v
    product's epilogue, the tcgen05 prompt attention, on pairs of SMs for G), then 150 single-token
    steps that wrap the ring, all positions against the plain implementation."""
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    rng = random.Random(12)
    lens, extra = [300, 129, 5, 210], 150
    seqs = [random_tokens(rng, n + extra, TINY[name][0]["vocab_size"]) for n in lens]
    want = [P.forward_logits(w, cfg, s) for s in seqs]
    r = runner_for(folder, dtype)
    slots = r.admit(len(lens))
    got = r.step(slots, [s[:n] for s, n in zip(seqs, lens)], [list(range(n)) for n in lens])
    assert_close(got, torch.cat([wl[:n] for wl, n in zip(want, lens)]), dtype, "whole prompts")
    for t in range(extra):
        got = r.step(slots, [[s[n + t]] for s, n in zip(seqs, lens)])
        assert_close(got, torch.stack([wl[n + t] for wl, n in zip(want, lens)]), dtype, f"decode step {t}")
    for s in slots:
        r.release(s)
    r.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_seqs", [20, 40, 70])
def test_many_sequences_decode_together(tmp_path, n_seqs, dtype):
    """20, 40 and 70 sequences in one batch (the row counts at which the products change
    kernels: up to 32 rows, up to 64, more), prompts of unequal lengths in one step, then
    single-token steps during which sequences leave the batch one by one."""
    folder = make_folder(tmp_path, "D")
    w, cfg = plain_model(folder)
    rng = random.Random(n_seqs)
    lens = [rng.randrange(1, 12) for _ in range(n_seqs)]
    total = [n + rng.randrange(2, 7) for n in lens]
    seqs = [random_tokens(rng, t, 1000) for t in total]
    want = [P.forward_logits(w, cfg, s) for s in seqs]
    r = runner_for(folder, dtype, max_tokens=64 * 128)          # a page, and so a slot, for each of them
    slots = r.admit(n_seqs)
    got = r.step(slots, [s[:n] for s, n in zip(seqs, lens)])
    assert_close(got, torch.stack([wl[n - 1] for wl, n in zip(want, lens)]), dtype, "prompt step")
    pos = list(lens)
    live = list(range(n_seqs))
    while live:
        got = r.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live])
        assert_close(got, torch.stack([want[i][pos[i]] for i in live]), dtype, f"decode with {len(live)} live")
        for i in live:
            pos[i] += 1
        for i in [i for i in live if pos[i] == total[i]]:
            r.release(slots[i])
        live = [i for i in live if pos[i] < total[i]]
    r.cache.check()


@pytest.mark.parametrize("name", ["C", "D", "F"])
def test_decoding_with_even_shares_of_the_keys(tmp_path, name, monkeypatch):
    """The other way to cut the decode attention's work: every CTA the same number of pages, wherever the borders
    of the (token, kv head) fall, merged by the last arrival.  Forced here for every launch (the planner asks for
    it only from dozens of sequences on): 23 sequences of 1 to 7 pages, whose window rings have wrapped (C, D),
    in a session of 24 rows (one padding row), decoded until the shortest have left.  Every logit against the
    plain implementation."""
    from hos_b200.parts import attention_fast as af
    calls = []
    monkeypatch.setattr(af, "decode_splits", lambda *a, **k: (calls.append(1), 0)[1])
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(11)
    lens = [rng.randrange(1, 440) for _ in range(23)]
    lens[0], lens[1], lens[2] = 1, 64, 65                       # a page's borders
    total = [n + rng.randrange(2, 9) for n in lens]
    seqs = [random_tokens(rng, t, vocab) for t in total]
    want = [P.forward_logits(w, cfg, s) for s in seqs]
    r = runner_for(folder, "bfloat16", max_tokens=64 * 256)
    slots = r.admit(len(seqs))
    r.step(slots, [s[:n] for s, n in zip(seqs, lens)])
    pos, live = list(lens), list(range(len(seqs)))
    while live:
        got = r.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live])
        assert_close(got, torch.stack([want[i][pos[i]] for i in live]), "bfloat16", f"decode with {len(live)} live")
        for i in live:
            pos[i] += 1
        for i in [i for i in live if pos[i] == total[i]]:
            r.release(slots[i])
        live = [i for i in live if pos[i] < total[i]]
    r.wait()
    assert calls, "the decode kernel was never asked how to cut its work"
    assert not af.decode_gave_up(TINY[name][0]["head_dim"])
    r.cache.check()


def test_sequences_of_unequal_lengths_get_even_shares_by_the_planner(tmp_path, monkeypatch):
    """40 sequences of 2 kv heads, most of them short and five of some 3,000 tokens: the session tells the
    attention how full of keys the sequences are, and the planner itself asks for even shares (nothing is forced
    here).  Every logit against the plain implementation."""
    from hos_b200.engine import Runner
    from hos_b200.parts import attention_fast as af
    from hos_b200.registry import config_from_dict
    from hos_b200.weights import write_model_folder
    chosen = []
    real = af.decode_splits
    monkeypatch.setattr(af, "decode_splits", lambda *a, **k: (chosen.append(real(*a, **k)), chosen[-1])[1])
    folder = str(tmp_path / "tiny_D_long")
    write_model_folder(config_from_dict(dict(TINY["D"][0], max_position_embeddings=4096)), 3, folder)
    w, cfg = plain_model(folder)
    rng = random.Random(12)
    lens = [rng.choice((3000, 2600)) if i % 8 == 0 else rng.randrange(5, 120) for i in range(40)]
    total = [n + 3 for n in lens]
    seqs = [random_tokens(rng, t, 1000) for t in total]
    with torch.no_grad():
        want = [P.forward_logits(w, cfg, s) for s in seqs]
    r = Runner.from_folder(folder, dtype="bfloat16", max_tokens=64 * 400, chunk_tokens=1)
    slots = r.admit(len(seqs))
    for lo in range(0, 40, 8):                                  # the prompts, eight sequences a step
        r.step(slots[lo:lo + 8], [s[:n] for s, n in zip(seqs[lo:lo + 8], lens[lo:lo + 8])])
    chosen.clear()
    for t in range(3):
        got = r.step(slots, [[s[n + t]] for s, n in zip(seqs, lens)])
        assert_close(got, torch.stack([wl[n + t] for wl, n in zip(want, lens)]), "bfloat16", f"decode step {t}")
    r.wait()
    assert chosen and 0 in chosen, f"the planner never asked for even shares: {sorted(set(chosen))}"
    r.cache.check()


@pytest.mark.parametrize("sizes", [dict(num_hidden_layers=4),
                                   dict(num_hidden_layers=2, hidden_size=4608, num_attention_heads=32,
                                        num_key_value_heads=16, head_dim=128, intermediate_size=36864,
                                        query_pre_attn_scalar=144)])
def test_real_layer_sizes_whole_prompt_against_prompt_and_decode(sizes):
    """Four layers of Gemma-2 2B's sizes, two of 27B's (random weights; too large for the plain implementation): the
    logits after a prompt of 5,000 tokens, which is longer than the window of 4,096, run whole must
    agree with the same tokens run as a prompt of 4,999 and one single-token step, and so must 40
    more steps on both sequences: the prompt path and the decode path (other kernels, the window's
    ring filled by a prompt or wrapped token by token) see the same keys.  Both sides are bfloat16
    results, each allowed the tolerance against exact logits, so their difference is allowed twice it."""
    from hos_b200 import Engine
    from hos_b200.registry import config_from_dict
    cfg = config_from_dict(dict(
        architectures=["Gemma2ForCausalLM"], model_type="gemma2", **{**dict(hidden_size=2304,
        num_attention_heads=8, num_key_value_heads=4, head_dim=256, intermediate_size=9216,
        query_pre_attn_scalar=256), **sizes},
        vocab_size=256000, rope_theta=10000.0, sliding_window=4096, max_position_embeddings=8192,
        attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
        rms_norm_eps=1e-6, tie_word_embeddings=True))
    eng = Engine.from_config(cfg, seed=1, dtype="bfloat16", max_batch=2, max_tokens=2 * 8192, max_seq_len=8192)
    r = eng.runner
    rng = random.Random(0)
    toks = random_tokens(rng, 5000, 256000)
    a, b = r.admit(2)
    whole = r.step([a], [toks])
    r.step([b], [toks[:-1]])
    cut = r.step([b], [[toks[-1]]])
    assert float(whole.abs().max()) > 5.0                      # logits of ordinary size, not a degenerate model

    def both_rounded(x, y, what):
        err = (x.float() - y.float()).abs()
        bound = 2.0 * (TOL["bfloat16"]["atol"] + TOL["bfloat16"]["rtol"] * y.float().abs())
        assert bool((err <= bound).all()), f"{what}: largest difference {float(err.max()):.4f}"

    both_rounded(cut, whole, "prompt of 4,999 and one step against the whole prompt")
    for t in random_tokens(rng, 40, 256000):
        out = r.step([a, b], [[t], [t]])
        both_rounded(out[1:2], out[0:1], "later steps of the two sequences")
    r.release(a)
    r.release(b)
    r.cache.check()


def test_a_step_that_fails_leaves_its_sequences_as_long_as_they_were(tmp_path, monkeypatch):
    """A kernel that refuses in the middle of a step (here: made to, on the host side): the step raises, and the
    sequences are as long as before on the host and in their records; the same step then runs."""
    from hos_b200 import ops
    from hos_b200.errors import KernelError
    folder = make_folder(tmp_path, "A")
    w, cfg = plain_model(folder)
    r = runner_for(folder, "float32")
    a, b = r.admit(2)
    r.step([a, b], [[1, 2, 3], [4, 5]])
    real = ops.norm_add_norm
    calls = {"n": 0}

    def failing(*args, **kw):
        calls["n"] += 1
        if calls["n"] == 3:
            raise KernelError("made to fail")
        return real(*args, **kw)
    monkeypatch.setattr(ops, "norm_add_norm", failing)
    r.use_sessions = False                                  # kernel by kernel, so that the failure falls inside the step
    with pytest.raises(KernelError, match="made to fail"):
        r.step([a, b], [[6, 7, 8, 9], [10]])
    monkeypatch.setattr(ops, "norm_add_norm", real)
    assert r.length(a) == 3 and r.length(b) == 2
    rec = r.cache.record.cpu()
    assert int(rec[a, ops.SLOT_POS]) == 3 and int(rec[b, ops.SLOT_POS]) == 2
    got = r.step([a, b], [[6, 7, 8, 9], [10]])
    want = torch.stack([P.forward_logits(w, cfg, [1, 2, 3, 6, 7, 8, 9])[-1], P.forward_logits(w, cfg, [4, 5, 10])[-1]])
    assert_close(got, want, "float32", "the step after the failed one")
    r.cache.check()


def test_stop_ids_beyond_the_ones_the_device_knows(tmp_path):
    """The device marks a sequence finished for the first 16 stop ids; the host checks all of them.  A stop id that
    is the 20th of the list ends its sequence all the same, the token after it is dropped, and a sequence beside it
    goes on; so does a stop id among the first 16."""
    from hos_b200 import Engine
    folder = make_folder(tmp_path, "B")
    w, cfg = plain_model(folder)
    eng = Engine(folder, dtype="float32", max_batch=4)
    prompts = [[9, 8, 7, 6], [100, 200, 300]]
    free = [P.greedy_generate(w, cfg, p, 12) for p in prompts]
    k = next(i for i in range(2, 12) if free[0][i] not in free[0][:i])      # a token the first sequence samples then for the first time
    stop = free[0][k]
    others = [t for t in range(400, 440) if t not in free[0] and t not in free[1]]
    for stops in (others[:19] + [stop], [stop] + others[:5]):
        outs = eng.generate_ids(prompts, 12, stop_ids=stops)
        assert outs == [P.greedy_generate(w, cfg, p, 12, stop_ids=stops) for p in prompts]
        assert outs[0] == free[0][:k]
    eng.runner.cache.check()
    assert eng.runner.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["C", "D"])
def test_short_turns_on_live_sequences_are_replayed_and_match_whole_prompts(tmp_path, name, dtype):
    """Sequences that go on by a few dozen tokens (a second turn) in a step that wants their last logits: the step
    is captured once per capacity and replayed with other sequences, lengths and slots; against the plain
    implementation on the whole history, and against the same step launched kernel by kernel."""
    folder = make_folder(tmp_path, name)
    w, cfg = plain_model(folder)
    vocab = TINY[name][0]["vocab_size"]
    rng = random.Random(21)
    r = runner_for(folder, dtype, chunk_tokens=300)
    eager = runner_for(folder, dtype, chunk_tokens=300)
    eager.prompt_sessions = False
    hist = [random_tokens(rng, n, vocab) for n in (30, 77, 5)]
    turns = [[random_tokens(rng, n, vocab) for n in ns] for ns in ((17, 5, 40), (3, 50, 2), (33, 2, 9))]
    slots, slots_e = r.admit(3), eager.admit(3)
    r.step(slots, hist)
    eager.step(slots_e, hist)
    for turn in turns:
        got = r.step(slots, turn)
        same = eager.step(slots_e, turn)
        hist = [h + t for h, t in zip(hist, turn)]
        want = torch.stack([P.forward_logits(w, cfg, h)[-1] for h in hist])
        assert_close(got, want, dtype, "a replayed turn")
        assert_close(same, want, dtype, "the same turn kernel by kernel")
        # and single tokens in between, as generation would bring them
        nxt = [[rng.randrange(vocab)] for _ in hist]
        got = r.step(slots, nxt)
        hist = [h + t for h, t in zip(hist, nxt)]
        eager.step(slots_e, nxt)
        assert_close(got, torch.stack([P.forward_logits(w, cfg, h)[-1] for h in hist]), dtype, "a token after the turn")
    assert any(k[0] == "turn" for k in r._sessions if isinstance(k, tuple))       # the turns did run as replayed steps
    assert not any(isinstance(k, tuple) and k[0] == "turn" for k in eager._sessions)
    # fewer sequences than the capture's capacity, in another order of slots
    got = r.step([slots[2], slots[0]], [[1, 2, 3], [4, 5]])
    want = torch.stack([P.forward_logits(w, cfg, hist[2] + [1, 2, 3])[-1], P.forward_logits(w, cfg, hist[0] + [4, 5])[-1]])
    assert_close(got, want, dtype, "two of the three")
    r.cache.check()


def test_single_token_steps_of_many_sequences_keep_the_decode_kernel(tmp_path, monkeypatch):
    """A replayed single-token step of 40 sequences must not be taken for a step of many tokens per sequence: the
    kernel that takes 64 or 128 queries per key tile would give the right logits and take twice the time."""
    from hos_b200.parts import attention_fast as af
    folder = make_folder(tmp_path, "D")
    r = runner_for(folder, "bfloat16", max_tokens=64 * 64)
    slots = r.admit(40)
    rng = random.Random(2)
    r.step(slots, [random_tokens(rng, 3 + i % 5, 1000) for i in range(40)])
    calls = []
    real = af.attend_chunks
    monkeypatch.setattr(af, "attend_chunks", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    r.step(slots, [[rng.randrange(1000)] for _ in slots])
    r.step(slots, [[rng.randrange(1000)] for _ in slots])
    assert not calls
    r.step(slots[:2], [random_tokens(rng, 40, 1000), random_tokens(rng, 9, 1000)])     # a turn of 49 tokens does take it
    assert calls


@pytest.mark.parametrize("dtype", DTYPES)
def test_embeddings_are_the_pooled_final_hidden_state(tmp_path, dtype):
    """Engine.embed: the hidden state after the last norm, mean over the tokens or the last token's
    (py/src/lib.rs:50-63), against the plain implementation; sequences under way are not disturbed."""
    from hos_b200 import Engine
    folder = make_folder(tmp_path, "B")
    w, cfg = plain_model(folder)
    eng = Engine(folder, dtype=dtype, max_batch=2)
    ids = random_tokens(random.Random(6), 37, 512)
    h = P.rmsnorm(P.forward_hidden(w, cfg, ids), w["model.norm.weight"], cfg.rms_norm_eps)
    conv, = eng.open(1)
    eng.generate_from_ids([conv], [[5, 6, 7]], max_tokens=2, temp=0.0, rep_penalty=1.0, stop_ids=[])
    held = eng.runner.length(conv.slot)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == "float32" else dict(atol=6e-2, rtol=6e-2)
    torch.testing.assert_close(eng.embed(ids, "mean").cpu(), h.mean(0), **tol)
    torch.testing.assert_close(eng.embed(ids, "last").cpu(), h[-1], **tol)
    with pytest.raises(ValueError, match="pooling"):
        eng.embed(ids, "max")
    assert eng.runner.length(conv.slot) == held and eng.runner.cache.slots.n_held == 1
    conv.close()
