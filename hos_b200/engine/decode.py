"""Single-token steps of a fixed set of sequences, with static device buffers so that the
whole step (all layers, head, and optionally the token choice and the move to the next
position) is captured once in a CUDA graph and replayed: decoding is bound by kernel launch
and memory latency, not by the host.

A session is made for a list of slots.  `feed(tokens)` + `run()` is one step with host token
ids (what the generation loop uses); `run_greedy_on_device()` is one step whose arg max stays
on the device and becomes the next input (what measurements of the device time use).  The
cache's pages for the positions a step writes must exist before it runs: `Runner` extends
the sequences first.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from .. import ops
from ..parts.base import StepInfo


class DecodeSession:
    def __init__(self, runner, slots: Sequence[int], use_graph: Optional[bool] = None):
        self.runner = runner
        self.slots = list(slots)
        b = self.b = len(self.slots)
        dev = runner.device
        if use_graph is None:
            use_graph = os.environ.get("HOS_NO_GRAPH", "") == ""
        self.use_graph = use_graph
        # one int32 buffer, one host mirror (pinned), one copy per step
        self._host = torch.zeros(6 * b + 1, dtype=torch.int32).pin_memory()
        self._dev = torch.zeros(6 * b + 1, dtype=torch.int32, device=dev)
        o = 0

        def take(n):
            nonlocal o
            v = (self._host[o:o + n], self._dev[o:o + n])
            o += n
            return v
        (self.h_tokens, self.tokens), (self.h_pos, self.pos) = take(b), take(b)
        (self.h_seq, self.seq), (self.h_cu, self.cu) = take(b), take(b + 1)
        (self.h_slot, self.slot), (self.h_after, self.after) = take(b), take(b)
        self.h_seq.copy_(torch.arange(b, dtype=torch.int32))
        self.h_cu.copy_(torch.arange(b + 1, dtype=torch.int32))
        self.h_slot.copy_(torch.tensor(self.slots, dtype=torch.int32))
        self.rows = torch.arange(b, dtype=torch.int32, device=dev)
        self.sampled = torch.zeros(b, dtype=torch.int32, device=dev)
        self.logits: Optional[torch.Tensor] = None
        self._graph = None
        self._graph_greedy = None
        self.launches_per_step = 0
        self._max_len = runner.cache.max_seq_len

    def _info(self) -> StepInfo:
        return StepInfo(n_tokens=self.b, n_seqs=self.b, tokens=self.tokens, token_pos=self.pos,
                        token_seq=self.seq, cu_seqlens=self.cu, seq_slot=self.slot,
                        seq_len_after=self.after, from_zero=False, single_token=True, max_new=1,
                        max_len_after=self._max_len, slots_host=tuple(self.slots),
                        cu_host=tuple(range(self.b + 1)), starts_host=())

    def feed(self, tokens: Sequence[int], lengths_before: Sequence[int]) -> None:
        """Host token ids and each sequence's length before the step -> the static buffers."""
        self.h_tokens.copy_(torch.tensor(list(tokens), dtype=torch.int32))
        lb = torch.tensor(list(lengths_before), dtype=torch.int32)
        self.h_pos.copy_(lb)
        self.h_after.copy_(lb + 1)
        self._dev.copy_(self._host, non_blocking=True)

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
        with torch.cuda.graph(g):
            out = fn()
        return g, out

    def run(self) -> torch.Tensor:
        """One step on what `feed` put in.  Returns float32 logits [B, vocab] (a static buffer
        when graphs are on: read it before the next run)."""
        self.runner.cache.flush()
        if self._graph is None and self.logits is None:
            self._graph, self.logits = self._capture(self._forward)
            if self._graph is None:
                return self.logits
            # the capture itself ran nothing: replay below
        if self._graph is not None:
            self._graph.replay()
            return self.logits
        self.logits = self._forward()
        return self.logits

    def run_greedy_on_device(self, first: bool = False) -> None:
        """One step; the arg max becomes the next input and positions move on, all on the
        device.  The eager first call repeats nothing: state is restored after the warm-up."""
        self.runner.cache.flush()
        if self._graph_greedy is None and not getattr(self, "_greedy_ready", False):
            keep = self._dev.clone()
            self._graph_greedy, _ = self._capture(self._forward_greedy)
            self._dev.copy_(keep)            # undo the eager warm-up's advance
            self._greedy_ready = True
        if self._graph_greedy is not None:
            self._graph_greedy.replay()
        else:
            self._forward_greedy()
