"""Single-token steps with static device buffers, so that a whole step (all layers, the head,
and optionally the token choice and the move to the next position) is captured once in a
CUDA graph and replayed: decoding is then bound by the kernels, not by the host.

A session serves every batch of up to `bucket` sequences: which slots take part is data (a
device array), not structure, and unused rows are padding (token_seq = -1), which every
kernel skips.  `feed(...)` + `run()` is one step with host token ids (what the step function
and the generation loop use); `run_greedy_on_device()` is one step whose arg max stays on
the device and becomes the next input (what measurements of the device time use).  The
cache's pages for the positions a step writes must exist before it runs: `Runner` extends
the sequences first.
"""
from __future__ import annotations

import gc
import os
import weakref
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..parts.base import StepInfo

BUCKETS = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)


def bucket_for(n: int) -> int:
    for b in BUCKETS:
        if n <= b:
            return b
    return (n + 63) // 64 * 64


def smaller_bucket(b: int) -> int:
    """The largest bucket below b (0 if there is none): a session of b rows holds more live rows than that."""
    below = [x for x in BUCKETS if x < b]
    return below[-1] if below else max(0, b - 64)


class DecodeSession:
    def __init__(self, runner, bucket: int, use_graph: Optional[bool] = None):
        self._runner = weakref.ref(runner)      # the runner owns its sessions: no reference cycle
        b = self.b = bucket
        dev = runner.device
        if use_graph is None:
            use_graph = os.environ.get("HOS_NO_GRAPH", "") == ""
        self.use_graph = use_graph
        # one int32 device buffer; two pinned host mirrors used in turn, each guarded by an event,
        # so that the host may run a step ahead of the device without overwriting a copy's source
        self._hosts = [torch.zeros(6 * b + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._hosts_np = [h.numpy() for h in self._hosts]
        self._laid_out = [-1, -1]               # live rows each mirror's constant fields were written for
        self._copied = [None, None]
        self._turn = 0
        self._dev = torch.zeros(6 * b + 1, dtype=torch.int32, device=dev)
        o = 0

        def take(n):
            nonlocal o
            v = self._dev[o:o + n]
            o += n
            return v
        self.tokens, self.pos, self.seq, self.cu = take(b), take(b), take(b), take(b + 1)
        self.slot, self.after = take(b), take(b)
        self.rows = torch.arange(b, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros(b, dtype=torch.int32, device=dev)
        self.logits: Optional[torch.Tensor] = None
        self._graph = None
        self._graph_greedy = None
        self._ready = False
        self._greedy_ready = False
        self.launches_per_step = 0
        self._max_len = runner.cache.max_seq_len
        self.n_live = 0

    @property
    def runner(self):
        return self._runner()

    def _info(self) -> StepInfo:
        return StepInfo(n_tokens=self.b, n_seqs=self.b, tokens=self.tokens, token_pos=self.pos,
                        token_seq=self.seq, cu_seqlens=self.cu, seq_slot=self.slot,
                        seq_len_after=self.after, from_zero=False, single_token=True, max_new=1,
                        max_len_after=self._max_len, slots_host=(), cu_host=tuple(range(self.b + 1)),
                        starts_host=(), token_slot=self.slot,      # row n is sequence n here
                        min_live=smaller_bucket(self.b) + 1, replayed=True)

    def feed(self, slots: Sequence[int], tokens: Sequence[int], lengths_before: Sequence[int]) -> None:
        """Host token ids, slots and each sequence's length before the step -> the static
        buffers (one host-to-device copy).  Rows beyond len(slots) are padding."""
        n = len(slots)
        self.n_live = n
        pad = self.b - n
        turn = self._turn
        self._turn ^= 1
        if self._copied[turn] is not None:
            self._copied[turn].synchronize()       # the copy that last read this mirror is done
        h = self._hosts[turn]
        hn = self._hosts_np[turn]              # the same memory as a numpy array: no tensor per field
        b = self.b
        hn[0:n] = tokens
        hn[b:b + n] = lengths_before
        hn[4 * b + 1:4 * b + 1 + n] = slots
        np.add(hn[b:b + n], 1, out=hn[5 * b + 1:5 * b + 1 + n])
        if self._laid_out[turn] != n:          # what depends on the number of live rows only
            hn[n:b] = -1
            hn[b + n:2 * b] = 0
            hn[2 * b:2 * b + n] = np.arange(n, dtype=np.int32)
            hn[2 * b + n:3 * b] = -1
            hn[3 * b:4 * b + 1] = np.minimum(np.arange(b + 1, dtype=np.int32), n)
            hn[4 * b + 1 + n:5 * b + 1] = 0
            hn[5 * b + 1 + n:6 * b + 1] = 1
            self._laid_out[turn] = n
        self._dev.copy_(h, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._copied[turn] = ev

    def _forward(self) -> torch.Tensor:
        r = self.runner
        x = r.model.hidden(self._info(), r.cache)
        return r.model.logits(x, self.rows)

    def _forward_greedy(self) -> torch.Tensor:
        logits = self._forward()
        ops.argmax(logits, self.sampled)
        ops.decode_advance(self.tokens, self.pos, self.after, self.seq, self.sampled)
        return logits

    def _capture(self, fn):
        # run once eagerly (first-use set-up of kernels must not happen inside a capture)
        before = ops.launch_count
        out = fn()
        self.launches_per_step = ops.launch_count - before
        if not self.use_graph:
            return None, out
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        # nothing but this thread's own launches may touch the capture: no collection of old
        # graphs or tensors (whose release frees device memory) while it is under way
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                out = fn()
        finally:
            if gc_was_on:
                gc.enable()
        return g, out

    def run(self) -> torch.Tensor:
        """One step on what `feed` put in.  Returns float32 logits [live sequences, vocab] (a
        view of a static buffer when graphs are on: use it before the next run)."""
        self.runner.cache.flush()
        if not self._ready:
            self._graph, self.logits = self._capture(self._forward)
            self._ready = True
            if self._graph is None:
                return self.logits[: self.n_live]
        if self._graph is not None:
            self._graph.replay()
        else:
            self.logits = self._forward()
        return self.logits[: self.n_live]

    def run_greedy_on_device(self) -> None:
        """One step; the arg max becomes the next input and positions move on, all on the device."""
        self.runner.cache.flush()
        if not self._greedy_ready:
            keep = self._dev.clone()
            self._graph_greedy, _ = self._capture(self._forward_greedy)
            self._dev.copy_(keep)            # undo the warm-up run's move to the next position
            self._greedy_ready = True
        if self._graph_greedy is not None:
            self._graph_greedy.replay()
        else:
            self._forward_greedy()


# ---- short prompts ---------------------------------------------------------------------------
# A prompt of a few dozen tokens is bound by the host when its kernels are launched one by one
# (about 16 us per launch).  Prompt steps of up to PROMPT_TOKENS tokens in all, of sequences that
# start at position 0 and want the logits of their last token, are therefore captured too: one
# graph per (token capacity, sequence capacity), the real token count, lengths and slots being
# data.  Rows beyond the real tokens are padding; sequences beyond the real ones have length 0.
PROMPT_TOKENS = 256
PROMPT_TOKEN_BUCKETS = (16, 32, 64, 128, 256)
PROMPT_SEQ_BUCKETS = (1, 2, 4, 8)


def prompt_bucket(n_tokens: int, n_seqs: int):
    """(token capacity, sequence capacity) of the session that takes such a prompt step, or None."""
    if n_tokens > PROMPT_TOKENS or n_seqs > PROMPT_SEQ_BUCKETS[-1]:
        return None
    return (next(t for t in PROMPT_TOKEN_BUCKETS if n_tokens <= t),
            next(q for q in PROMPT_SEQ_BUCKETS if n_seqs <= q))


class PromptSession:
    def __init__(self, runner, tokens_cap: int, seqs_cap: int, use_graph: Optional[bool] = None):
        self._runner = weakref.ref(runner)
        self.t, self.q = tokens_cap, seqs_cap
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
                        from_zero=True, single_token=False, max_new=self.t, max_len_after=self.t,
                        slots_host=(), cu_host=(), starts_host=(), replayed=True)

    def feed(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]]) -> None:
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
            hn[t + at:t + at + k] = np.arange(k, dtype=np.int32)
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
        hn[o + 3 * q + 1:o + 4 * q + 1] = np.maximum(cu[1:] - 1, 0)     # the last row of each sequence
        self._dev.copy_(self._hosts[turn], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._copied[turn] = ev

    def _forward(self) -> torch.Tensor:
        r = self.runner
        x = r.model.hidden(self._info(), r.cache)
        return r.model.logits(x, self.rows)

    def run(self) -> torch.Tensor:
        """The step on what `feed` put in: float32 logits [real sequences, vocab] at each one's last
        token (a view of a static buffer when graphs are on: use it before the next run)."""
        self.runner.cache.flush()
        if not self._ready:
            self._graph, self.logits = DecodeSession._capture(self, self._forward)
            self._ready = True
            if self._graph is None:
                return self.logits[: self.n_live]
        if self._graph is not None:
            self._graph.replay()
        else:
            self.logits = self._forward()
        return self.logits[: self.n_live]
