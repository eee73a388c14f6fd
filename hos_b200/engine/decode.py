"""Single-token steps with static device buffers, so that a whole step (all layers, the head,
and optionally the token choice) is captured once in a CUDA graph and replayed: decoding is
then bound by the kernels, not by the host.

A session serves every batch of up to `bucket` sequences: which slots take part is data (a
device array), not structure, and unused rows are padding (token_seq = -1), which every
kernel skips.  What the host sends per step is the list of slots (and, for a step whose
tokens the caller brings, the tokens): positions are read from the slots' records on the
device and moved on there (csrc/slot_state.cu).

  upload(slots, tokens) + run_step()      one step on host token ids -> logits (the step function)
  upload(slots) + run_generate(params)    one step whose input is the token sampled last (kept in the
                                          record), followed by sampling on the device; the new token
                                          goes into the record and is fetched asynchronously
                                          (fetch_start / fetch_read): the generation loop and the
                                          measurements

The cache's pages for the positions a step writes must exist before it runs: the caller
extends the sequences first.
"""
from __future__ import annotations

import gc
import os
import weakref
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..parts.base import StepInfo
from ..sampling.sampler import SamplingParams

BUCKETS = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)
META = 2 + ops.MAX_STOPS        # live rows, number of stop ids, the stop ids


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return (n + 63) // 64 * 64


def smaller_bucket(b: int) -> int:
    """The largest bucket below b (0 if there is none): a session of b rows holds more live rows than that."""
    below = [x for x in BUCKETS if x < b]
    return below[-1] if below else max(0, b - 64)


def live_class(n_live: int, bucket: int):
    """(fewest, most) live rows that a replayed step of `bucket` rows is planned for when `n_live` of them are
    live: the rows above the next smaller bucket, cut into up to four classes.  How the attention kernel splits
    the keys depends on how many rows take part (17 rows of 4 kv heads in two shares fill the SMs once; 24 do
    not), so a step is captured per class, as it is per length class."""
    lo = smaller_bucket(bucket) + 1
    if n_live < lo:
        return (1, lo - 1) if n_live > 0 else (lo, bucket)     # fewer rows than the bucket is meant for: one class
    width = max(1, (bucket - lo + 1 + 3) // 4)
    first = lo + (n_live - lo) // width * width
    return first, min(bucket, first + width - 1)


def fill_class(total: Optional[int], n_live: int, planned_len: int) -> float:
    """The fraction of (live rows x planned length) that the sequences' lengths add up to, rounded up to 1, 1/2,
    1/4 or 1/8: sequences of unequal lengths hold fewer keys than as many of the longest length would, and where
    the attention kernel's work is cut by the sum of the pages (even shares) that decides how it is planned."""
    if not total or n_live <= 0 or planned_len <= 0:
        return 1.0
    ratio = total / float(n_live * planned_len)
    for f in (0.125, 0.25, 0.5):
        if ratio <= f:
            return f
    return 1.0


MIN_LENGTH_CLASS = 512


def length_class(longest: Optional[int], max_seq_len: int) -> int:
    """The sequence length a replayed step is planned for: the next of 512, 768, 1024, 1536, 2048, 3072, ... at or
    above the longest live sequence (at most what the cache holds).  How the attention kernel cuts the keys over
    the GPU depends on it, and is part of what is captured: a step is captured once per class, so a batch of short
    sequences is not run with the cut that the longest possible one would want.  (Powers of two alone left the plan
    up to a factor of two beside the truth: sixteen sequences of up to 2,300 keys were planned as for 4,096.)"""
    if longest is None or longest >= max_seq_len:
        return max_seq_len
    c = MIN_LENGTH_CLASS
    while c < longest:
        c = c * 3 // 2 if c & (c - 1) == 0 else c * 4 // 3
    return min(c, max_seq_len)


class DecodeSession:
    def __init__(self, runner, bucket: int, use_graph: Optional[bool] = None):
        self._runner = weakref.ref(runner)      # the runner owns its sessions: no reference cycle
        b = self.b = bucket
        dev = runner.device
        if use_graph is None:
            use_graph = os.environ.get("HOS_NO_GRAPH", "") == ""
        self.use_graph = use_graph
        # What the host sends: meta | slots | tokens.  Two pinned mirrors used in turn, each guarded by
        # an event, so that the host may run a step ahead of the device without overwriting a copy's source.
        n_up = META + 2 * b
        self._hosts = [torch.zeros(n_up, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._hosts_np = [h.numpy() for h in self._hosts]
        self._copied = [None, None]
        self._turn = 0
        self._dev = torch.zeros(n_up + 4 * b + 1, dtype=torch.int32, device=dev)
        o = 0

        def take(n):
            nonlocal o
            v = self._dev[o:o + n]
            o += n
            return v
        self.meta, self.slot, self.tokens = take(META), take(b), take(b)
        self.pos, self.seq, self.after, self.cu = take(b), take(b), take(b), take(b + 1)     # written on the device
        self.sampled = torch.zeros(b, dtype=torch.int32, device=dev)
        self.uniforms = torch.zeros(b, dtype=torch.float32, device=dev)
        self.recent_len = torch.zeros(b, dtype=torch.int32, device=dev)
        self._recent = {}                       # repeat_last_n -> static [b, n] buffer
        # sampled tokens on their way to the host: pinned buffers used in turn
        self._fetch_hosts = [torch.zeros(b, dtype=torch.int32).pin_memory() for _ in range(3)]
        self._fetch_turn = 0
        self.logits: Optional[torch.Tensor] = None
        self._programs = {}                     # key -> (graph or None, logits buffer)
        self._pool = None                       # the programs' buffers share one pool: only one of them runs at a time
        self.launches_per_step = 0
        self._max_len = runner.cache.max_seq_len
        self._planned_len = self._max_len       # the lengths the replayed launches are planned for (see length_class)
        self._planned_live = (smaller_bucket(b) + 1, b)      # and the numbers of live rows (see live_class)
        self._planned_fill = ()                 # and how full of keys the sequences are, per window (see fill_class)
        self._seen_len, self._seen_fill = self._max_len, ()     # what the step at hand really holds: a new capture plans with it
        self._windows = sorted({g.need.window or 0 for g in runner.cache.groups})
        self.n_live = 0

    @property
    def runner(self):
        return self._runner()

    def _info(self) -> StepInfo:
        return StepInfo(n_tokens=self.b, n_seqs=self.b, tokens=self.tokens, token_pos=self.pos,
                        token_seq=self.seq, cu_seqlens=self.cu, seq_slot=self.slot,
                        seq_len_after=self.after, from_zero=False, single_token=True, max_new=1,
                        max_len_after=self._seen_len, slots_host=(), cu_host=tuple(range(self.b + 1)),
                        starts_host=(), token_slot=self.slot,      # row n is sequence n here
                        min_live=self._planned_live[0], max_live=self._planned_live[1], fills=self._seen_fill,
                        replayed=True)

    def upload(self, slots: Sequence[int], tokens: Optional[Sequence[int]] = None,
               stop_ids: Sequence[int] = (), longest: Optional[int] = None,
               lengths: Optional[Sequence[int]] = None) -> None:
        """Which slots the next step runs (rows beyond them are padding), the tokens if the caller
        brings them, and the stop ids that mark a sequence finished on the device (the first
        ops.MAX_STOPS of them; the host checks all of them anyway): one host-to-device copy.
        `longest`: the length of the longest of these sequences after the step, if the caller knows it
        (the attention kernel's split of the keys is planned for the class of lengths above it); `lengths`: all of
        their lengths after the step, if known (see fill_class)."""
        n = len(slots)
        self.n_live = n
        if lengths is not None and longest is None:
            longest = max(lengths)
        planned = self._planned_len = length_class(longest, self._max_len)
        self._planned_live = live_class(n, self.b)
        # Per window of the cache's groups (0: all keys): the keys held, over n x what the longest holds.  The classes
        # name the captured program; a capture itself plans with what the step at hand really holds (the first
        # step of a class decides for the class: the classes are narrow enough for that).
        self._seen_len = min(longest, self._max_len) if longest is not None else self._max_len
        self._planned_fill = self._seen_fill = ()
        if lengths is not None:
            held = [(w, sum(min(x, w) if w else x for x in lengths), min(self._seen_len, w) if w else self._seen_len)
                    for w in self._windows]
            self._seen_fill = tuple((w, min(1.0, total / float(n * most))) for w, total, most in held)
            self._planned_fill = tuple((w, fill_class(total, n, most)) for w, total, most in held)
        turn = self._turn
        self._turn ^= 1
        if self._copied[turn] is not None:
            self._copied[turn].synchronize()       # the copy that last read this mirror is done
        hn, b = self._hosts_np[turn], self.b
        stops = list(stop_ids)[: ops.MAX_STOPS]
        hn[0], hn[1] = n, len(stops)
        hn[2:2 + len(stops)] = stops
        hn[META:META + n] = slots
        hn[META + n:META + b] = 0
        size = META + b
        if tokens is not None:
            hn[META + b:META + b + n] = tokens
            hn[META + b + n:META + 2 * b] = -1
            size = META + 2 * b
        self._dev[:size].copy_(self._hosts[turn][:size], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._copied[turn] = ev

    # ---- what a step launches ---------------------------------------------------------------
    def _begin(self, flags: int, recent=None) -> None:
        c = self.runner.cache
        ops.slot_begin(c.record, c.recent, self.slot, self.meta, self.b, flags, self.tokens, self.pos, self.after,
                       self.seq, self.cu, self.uniforms if flags & ops.BEGIN_UNIFORM else None, recent,
                       self.recent_len if recent is not None else None)

    def _forward_step(self) -> torch.Tensor:
        r = self.runner
        self._begin(ops.BEGIN_ADVANCE)
        return r.model.step_logits(self._info(), r.cache)

    def _forward_generate(self, p: SamplingParams) -> torch.Tensor:
        r = self.runner
        penal = p.rep_penalty != 1.0 and p.repeat_last_n > 0
        recent = None
        if penal:
            recent = self._recent.get(p.repeat_last_n)
            if recent is None:
                recent = self._recent[p.repeat_last_n] = torch.zeros((self.b, p.repeat_last_n), dtype=torch.int32,
                                                                     device=r.device)
        flags = ops.BEGIN_ADVANCE | ops.BEGIN_TOKEN_FROM_RECORD | ops.BEGIN_SKIP_FINISHED
        flags |= ops.BEGIN_UNIFORM if p.temp > 0.0 else 0
        flags |= ops.BEGIN_RECENT if penal else 0
        self._begin(flags, recent)
        logits = r.model.step_logits(self._info(), r.cache)
        sample_into(logits, self.sampled, p, self.uniforms, recent, self.recent_len)
        c = r.cache
        ops.slot_end(c.record, c.recent, self.slot, self.meta, self.b, self.sampled)
        return logits

    def _program(self, key, fn):
        """The launches of `fn` as a replayable program: run once as they are (first-use set-up of
        kernels must not happen inside a capture; what that run changed in the slots' records is
        put back), then captured."""
        prog = self._programs.get(key)
        if prog is not None:
            return prog
        c = self.runner.cache
        keep = (c.record.clone(), c.recent.clone())
        before = ops.launch_count
        out = fn()
        self.launches_per_step = ops.launch_count - before
        c.record.copy_(keep[0])
        c.recent.copy_(keep[1])
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        # nothing but this thread's own launches may touch the capture: no collection of old
        # graphs or tensors (whose release frees device memory) while it is under way
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, pool=self._pool, capture_error_mode="thread_local"):
                out = fn()
        finally:
            if gc_was_on:
                gc.enable()
        if self._pool is None:
            # Every class of lengths, of live rows and of fill has its own program, and each would keep its own
            # logits [rows, vocab] and activations; what a program leaves is used before the next one runs, so
            # they may all live in the same memory.
            self._pool = g.pool()
        prog = self._programs[key] = (g, out)
        return prog

    def _run(self, key, fn) -> torch.Tensor:
        self.runner.cache.flush()
        if not self.use_graph:
            before = ops.launch_count
            self.logits = fn()
            self.launches_per_step = ops.launch_count - before
            return self.logits
        g, self.logits = self._program(key + (self._planned_len, self._planned_live, self._planned_fill), fn)
        g.replay()
        return self.logits

    def run_step(self) -> torch.Tensor:
        """One step on the tokens that `upload` brought.  Returns float32 logits [live sequences,
        vocab] (a view of a static buffer when graphs are on: use it before the next run)."""
        return self._run(("step",), self._forward_step)[: self.n_live]

    def run_generate(self, params: SamplingParams) -> None:
        """One step whose input tokens are the ones sampled last; the new ones are sampled on the
        device (`self.sampled`) and go into the slots' records."""
        key = ("generate", params.temp, params.top_k, params.top_p, params.rep_penalty, params.repeat_last_n)
        self._run(key, lambda: self._forward_generate(params))

    def sample_logits(self, logits: torch.Tensor, params: SamplingParams) -> None:
        """Sample from logits [live rows, vocab] of a step that ran elsewhere (the sequences' first
        step), with the records' generators and recent tokens, as run_generate does after its own step."""
        n = logits.shape[0]
        penal = params.rep_penalty != 1.0 and params.repeat_last_n > 0
        recent = None
        if penal:
            recent = torch.empty((self.b, params.repeat_last_n), dtype=torch.int32, device=logits.device)
        flags = (ops.BEGIN_UNIFORM if params.temp > 0.0 else 0) | (ops.BEGIN_RECENT if penal else 0)
        c = self.runner.cache
        if flags:
            ops.slot_begin(c.record, c.recent, self.slot, self.meta, self.b, flags, self.tokens, self.pos, self.after,
                           self.seq, self.cu, self.uniforms if flags & ops.BEGIN_UNIFORM else None, recent,
                           self.recent_len if recent is not None else None)
        sample_into(logits, self.sampled[:n], params, self.uniforms[:n], recent[:n] if penal else None,
                    self.recent_len[:n])
        ops.slot_end(c.record, c.recent, self.slot, self.meta, self.b, self.sampled)

    # ---- sampled tokens to the host, without waiting --------------------------------------------
    def fetch_start(self):
        """Start copying the tokens just sampled to the host; hand the result to fetch_read later."""
        turn = self._fetch_turn
        self._fetch_turn = (turn + 1) % len(self._fetch_hosts)
        host = self._fetch_hosts[turn]
        host[: self.b].copy_(self.sampled, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return host, ev, self.n_live

    @staticmethod
    def fetch_read(handle) -> List[int]:
        host, ev, n = handle
        ev.synchronize()
        ops.check_errors()            # a kernel that gave up a wait: these tokens are not to be trusted
        return host[:n].tolist()


def sample_into(logits: torch.Tensor, out: torch.Tensor, p: SamplingParams, uniforms, recent, recent_len) -> None:
    """The sampler's rule (src/lib.rs:91-172) on device data: arg max when temp <= 0, else
    temperature, top-k, top-p and the draw `uniforms`; the repetition penalty over `recent` if given."""
    pen = p.rep_penalty if recent is not None else 1.0
    if p.temp <= 0.0:
        ops.argmax(logits, out, pen, recent, recent_len if recent is not None else None)
    else:
        ops.sample(logits, uniforms, out, p.temp, p.top_k, p.top_p, pen, recent,
                   recent_len if recent is not None else None)


# ---- short prompts ---------------------------------------------------------------------------
# A prompt of a few dozen tokens is bound by the host when its kernels are launched one by one
# (about 16 us per launch).  Prompt steps of up to PROMPT_TOKENS tokens in all, of sequences that
# start at position 0 and want the logits of their last token, are therefore captured too: one
# graph per (token capacity, sequence capacity), the real token count, lengths and slots being
# data.  Rows beyond the real tokens are padding; sequences beyond the real ones have length 0.
PROMPT_TOKENS = 512
PROMPT_TOKEN_BUCKETS = (16, 32, 64, 128, 256, 384, 512)
PROMPT_SEQ_BUCKETS = (1, 2, 4, 8)


def prompt_bucket(n_tokens: int, n_seqs: int):
    """(token capacity, sequence capacity) of the session that takes such a prompt step, or None."""
    if n_tokens > PROMPT_TOKENS or n_seqs > PROMPT_SEQ_BUCKETS[-1]:
        return None
    return (next(t for t in PROMPT_TOKEN_BUCKETS if n_tokens <= t),
            next(q for q in PROMPT_SEQ_BUCKETS if n_seqs <= q))


class PromptSession:
    """`continuing`: the sequences do not start at position 0 but go on from where the cache left them (a
    second turn of a few dozen tokens): the same capture, with positions that begin at each sequence's length and
    attention over the cache, planned for sequences of up to `planned_len` tokens."""

    def __init__(self, runner, tokens_cap: int, seqs_cap: int, use_graph: Optional[bool] = None,
                 continuing: bool = False, planned_len: int = 0):
        self._runner = weakref.ref(runner)
        self.t, self.q = tokens_cap, seqs_cap
        self.continuing, self.planned_len = continuing, planned_len
        if use_graph is None:
            use_graph = os.environ.get("HOS_NO_GRAPH", "") == ""
        self.use_graph = use_graph
        t, q = tokens_cap, seqs_cap
        n = 3 * t + (q + 1) + 3 * q
        self._hosts = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._hosts_np = [h.numpy() for h in self._hosts]
        self._copied = [None, None]
        self._turn = 0
        self._dev = torch.zeros(n, dtype=torch.int32, device=runner.device)
        d, o = self._dev, 3 * t
        self.tokens, self.pos, self.seq = d[0:t], d[t:2 * t], d[2 * t:3 * t]
        self.cu, self.slot, self.after, self.rows = d[o:o + q + 1], d[o + q + 1:o + 2 * q + 1], \
            d[o + 2 * q + 1:o + 3 * q + 1], d[o + 3 * q + 1:o + 4 * q + 1]
        self.logits: Optional[torch.Tensor] = None
        self._graph = None
        self._ready = False
        self.n_live = 0

    @property
    def runner(self):
        return self._runner()

    def _info(self) -> StepInfo:
        return StepInfo(n_tokens=self.t, n_seqs=self.q, tokens=self.tokens, token_pos=self.pos,
                        token_seq=self.seq, cu_seqlens=self.cu, seq_slot=self.slot, seq_len_after=self.after,
                        from_zero=not self.continuing, single_token=False, max_new=self.t,
                        max_len_after=self.planned_len if self.continuing else self.t,
                        slots_host=(), cu_host=(), starts_host=(), replayed=True, min_live=1)

    def feed(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
             starts: Optional[Sequence[int]] = None) -> None:
        live = len(slots)
        self.n_live = live
        turn = self._turn
        self._turn ^= 1
        if self._copied[turn] is not None:
            self._copied[turn].synchronize()
        hn, t, q = self._hosts_np[turn], self.t, self.q
        o = 3 * t
        at = 0
        cu = hn[o:o + q + 1]
        for i, toks in enumerate(token_lists):
            k = len(toks)
            hn[at:at + k] = toks
            hn[t + at:t + at + k] = np.arange(k, dtype=np.int32) + (starts[i] if starts is not None else 0)
            hn[2 * t + at:2 * t + at + k] = i
            cu[i] = at
            at += k
        hn[at:t] = -1                      # padding rows
        hn[t + at:2 * t] = 0
        hn[2 * t + at:3 * t] = -1
        cu[live:] = at                     # sequences beyond the real ones are empty
        hn[o + q + 1:o + q + 1 + live] = slots
        hn[o + q + 1 + live:o + 2 * q + 1] = 0
        lens = np.diff(cu)
        hn[o + 2 * q + 1:o + 3 * q + 1] = lens
        if starts is not None:
            hn[o + 2 * q + 1:o + 2 * q + 1 + live] += np.asarray(starts, dtype=np.int32)
        hn[o + 3 * q + 1:o + 4 * q + 1] = np.maximum(cu[1:] - 1, 0)     # the last row of each sequence
        self._dev.copy_(self._hosts[turn], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._copied[turn] = ev

    def _forward(self) -> torch.Tensor:
        r = self.runner
        # the kernels of a prompt step, short ones too, are launched ahead of one another's end: their set-up
        # (barriers, tensor memory, the first look-ups) runs under the kernel before (40 tokens 2.15 -> 2.11 ms, 256
        # tokens 2.90 -> 2.81, 512 tokens 3.66 -> 3.48 at Gemma-2 2B sizes)
        # (up to 32 rows the few-rows products run, which choose for themselves which of them go ahead: all of them
        # ahead is what they measured as their worst case, 16 tokens 2.63 ms instead of 2.0)
        ops.set_launch_ahead(self.t > 32)
        try:
            x = r.model.hidden(self._info(), r.cache)
            ops.slot_set_pos(r.cache.record, self.slot, self.after, self.cu, self.q)    # the records learn the new lengths
            return r.model.logits(x, self.rows)
        finally:
            ops.set_launch_ahead(False)

    def run(self) -> torch.Tensor:
        """The step on what `feed` put in: float32 logits [real sequences, vocab] at each one's last
        token (a view of a static buffer when graphs are on: use it before the next run)."""
        self.runner.cache.flush()
        if not self.use_graph:
            self.logits = self._forward()
            return self.logits[: self.n_live]
        if not self._ready:
            self.logits = self._forward()       # first-use set-up of kernels must not happen inside a capture
            torch.cuda.synchronize()
            self._graph = torch.cuda.CUDAGraph()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(self._graph, capture_error_mode="thread_local"):
                    self.logits = self._forward()
            finally:
                if gc_was_on:
                    gc.enable()
            self._ready = True
        self._graph.replay()
        return self.logits[: self.n_live]
