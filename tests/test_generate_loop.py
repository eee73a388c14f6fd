"""The generation loop's decisions, driven with a fake step function (no GPU)."""
import pytest

from hos_b200.engine import generate as gen
from hos_b200.errors import HosError
from hos_b200.sampling import SamplingParams, next_rand, stream_seed


class FakeBackend:
    """The loop's backend without a GPU.  The next token of a sequence is (sum of the tokens it has
    been fed) % 50.  Like the device backend, it samples at once but hands the tokens over only
    when asked (`fetch`), so the loop must decide who goes on before it knows them."""

    def __init__(self, n_slots=8, max_seq_len=1000):
        self.free = list(range(n_slots))
        self.seen = {}
        self.last = {}
        self.max_seq_len = max_seq_len
        self.steps = []                    # (slots, token lists) of every step
        self.taken_log = []
        self.queue = []
        self.settled = {}

    def admit(self, n):
        assert n <= len(self.free)
        out = [self.free.pop(0) for _ in range(n)]
        for s in out:
            self.seen[s] = []
        self.taken_log.append(list(out))
        return out

    def length(self, slot):
        return len(self.seen[slot])

    def _step(self, slots, token_lists):
        self.steps.append((list(slots), [list(t) for t in token_lists]))
        toks = []
        for s, t in zip(slots, token_lists):
            assert len(self.seen[s]) + len(t) <= self.max_seq_len, "a step past the context's end"
            self.seen[s].extend(t)
            self.last[s] = sum(self.seen[s]) % 50
            toks.append(self.last[s])
        self.queue.append(toks)

    def begin(self, slots, token_lists, indices, max_new, stop_ids):
        assert len(slots) == len(token_lists) == len(indices)
        self._step(slots, token_lists)

    def advance(self, slots):
        assert self.queue, "a step is launched one sampling ahead at most... but never with nothing pending"
        assert len(self.queue) <= 1, "at most one sampling may be waiting when the next step is launched"
        self._step(slots, [[self.last[s]] for s in slots])

    def fetch(self):
        return self.queue.pop(0)

    def settle(self, slots, lengths):
        self.settled.update(zip(slots, lengths))

    def release(self, slot):
        assert slot in self.seen, "released twice"
        del self.seen[slot]
        self.free.append(slot)
        self.free.sort()


def reference(prompt, max_new, stop, max_len=1000):
    seq, out = list(prompt), []
    for _ in range(max_new):
        t = sum(seq) % 50
        if t in stop:
            break
        out.append(t)
        if len(seq) >= max_len:
            break
        seq.append(t)
    return out


def test_plan_batches_respects_count_and_capacity():
    assert gen.plan_batches([5, 5, 5, 5, 5], 10, 10_000, 2, 4096) == [[0, 1], [2, 3], [4]]
    # each request needs round64(100 + 30) = 192 tokens; 400 hold two
    assert gen.plan_batches([100, 100, 100], 30, 400, 8, 4096) == [[0, 1], [2]]
    # the context caps what a request can ever hold
    assert gen.plan_batches([60, 60], 1000, 128, 8, 64) == [[0, 1]]
    with pytest.raises(HosError, match="empty prompt"):
        gen.plan_batches([3, 0], 4, 1000, 8, 4096)
    with pytest.raises(HosError, match="more than the context"):
        gen.plan_batches([5000], 4, 100000, 8, 4096)
    with pytest.raises(HosError, match="cache holds"):
        gen.plan_batches([500], 4, 256, 8, 4096)


def test_unequal_prompts_end_at_different_times_and_match_single_runs():
    prompts = [[3, 4, 5], [1], [9, 9, 9, 9, 9, 9, 2], [11, 13]]
    stop = set(range(0, 50, 4))
    b = FakeBackend()
    outs = gen.generate(b, prompts, 12, stop, 10_000, 8)
    assert outs == [reference(p, 12, stop) for p in prompts]
    assert len({len(o) for o in outs}) > 1                 # they did end at different times
    assert b.seen == {} and b.free == list(range(8))       # every slot came back
    first_slots, first_tokens = b.steps[0]
    assert first_tokens == prompts                          # all prompts in ONE step
    sizes = [len(s) for s, _ in b.steps]
    assert sizes == sorted(sizes, reverse=True)             # the batch only shrinks


def test_stop_token_is_not_returned_and_first_token_can_stop():
    b = FakeBackend()
    outs = gen.generate(b, [[7]], 5, {7}, 1000, 8)      # first sampled token is 7
    # the step launched before the stop token was seen ran for nothing; no other follows
    assert outs == [[]] and len(b.steps) == 2 and b.seen == {}


def test_max_new_bounds_the_output_and_no_step_follows_the_last_token():
    b = FakeBackend()
    outs = gen.generate(b, [[2, 3]], 4, set(), 1000, 8)
    assert len(outs[0]) == 4
    assert len(b.steps) == 4                 # prompt + 3 single tokens; the 4th token is not fed
    assert gen.generate(FakeBackend(), [[2, 3]], 0, set(), 1000, 8) == [[]]


def test_context_limit_ends_a_sequence():
    b = FakeBackend(max_seq_len=6)
    outs = gen.generate(b, [[1, 2, 3, 4]], 50, set(), 1000, 8)
    assert outs == [reference([1, 2, 3, 4], 50, set(), max_len=6)]
    assert len(outs[0]) == 3                 # positions 4 and 5 are fed, a third token is sampled
    assert max(len(t) for _, toks in b.steps for t in toks) == 4


def test_batches_follow_one_another_and_reuse_slots():
    prompts = [[i + 1] * (i + 1) for i in range(7)]
    b = FakeBackend(n_slots=3)
    outs = gen.generate(b, prompts, 5, {0}, 10_000, 3)
    assert outs == [reference(p, 5, {0}) for p in prompts]
    assert b.taken_log == [[0, 1, 2], [0, 1, 2], [0]]
    assert b.seen == {}


def test_slots_come_back_when_a_step_fails():
    class Boom(FakeBackend):
        def _step(self, slots, token_lists):
            if len(self.steps) == 2:
                raise RuntimeError("boom")
            return super()._step(slots, token_lists)
    b = Boom()
    with pytest.raises(RuntimeError):
        gen.generate(b, [[1, 2], [3]], 9, set(), 1000, 8)
    assert b.seen == {} and b.free == list(range(8))


def test_a_stopped_sequence_runs_one_step_for_nothing_and_no_more():
    # prompt [3]: 3, then (3+3)=6, 12, 24, 48, 96%50=46 ...; stop at 24
    b = FakeBackend()
    outs = gen.generate(b, [[3], [1, 1]], 10, {24}, 1000, 8)
    assert outs[0] == [3, 6, 12] and outs[0] == reference([3], 10, {24})
    assert outs[1] == reference([1, 1], 10, {24})
    fed_to_first = [t for slots, toks in b.steps for s, t in zip(slots, toks) if s == 0]
    # the prompt, the three returned tokens, and the stop token once (a step that was under way)
    assert fed_to_first == [[3], [3], [6], [12], [24]]


def test_sequences_that_keep_their_slots_are_settled_at_their_true_length():
    b = FakeBackend()
    slots = b.admit(2)
    outs = gen.run_batch(b, [[3], [1, 1]], [0, 1], 4, {24}, slots=slots)
    assert outs == [reference([3], 4, {24}), reference([1, 1], 4, {24})]
    assert sorted(b.seen) == slots                       # nothing was released
    # first: prompt + 3 tokens fed, the stop token fed for nothing is not counted;
    # second: prompt + 3 of its 4 tokens fed (the last one was sampled but never run)
    assert b.settled == {slots[0]: 1 + 3, slots[1]: 2 + 3}
    # a second turn continues them
    outs2 = gen.run_batch(b, [[5], [outs[1][-1], 7]], [0, 1], 2, set(), slots=slots)
    assert len(outs2[0]) == 2 and len(outs2[1]) == 2


def test_host_random_stream_matches_the_reference_generator():
    # xorshift64 (13, 7, 17), top 24 bits: src/lib.rs:78-85; first draws for seed 42
    s, u1 = next_rand(42)
    assert s == 45454805674 and u1 == (45454805674 >> 40) / (1 << 24)
    s2, u2 = next_rand(s)
    x = s
    x ^= (x << 13) & ((1 << 64) - 1); x ^= x >> 7; x ^= (x << 17) & ((1 << 64) - 1)
    assert s2 == x and 0.0 <= u2 < 1.0
    assert stream_seed(42, 0) == 42 and stream_seed(42, 3) == 45 and stream_seed(0, 0) != 0


def test_sampling_defaults_are_the_references():
    p = SamplingParams()
    assert (p.temp, p.top_k, p.top_p, p.rep_penalty, p.repeat_last_n, p.seed) == (0.0, 40, 0.95, 1.1, 64, 42)
    q = SamplingParams.pure()
    assert (q.top_k, q.top_p, q.rep_penalty) == (0, 1.0, 1.0)


def test_a_penalty_window_longer_than_the_record_keeps_is_refused():
    # the reference penalises recent[len - repeat_last_n..] whatever its length (src/lib.rs:102-118);
    # here a sequence's record keeps its last 256 sampled tokens, so a longer window is refused, not cut
    SamplingParams(rep_penalty=1.3, repeat_last_n=256)
    SamplingParams(rep_penalty=1.0, repeat_last_n=100000)          # no penalty: the window does not matter
    with pytest.raises(HosError, match="256 recent tokens"):
        SamplingParams(rep_penalty=1.3, repeat_last_n=257)
