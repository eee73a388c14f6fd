"""Choosing the next token of each sequence.

The rule is the reference's `sample` (src/lib.rs:91-172), computed by the kernel in
csrc/sampling.cu: repetition penalty over the last `repeat_last_n` generated
tokens, arg max when temp <= 0 (first maximum wins), else temperature softmax,
top-k, top-p, and a draw with the reference's xorshift64 generator
(src/lib.rs:78-85), one stream per sequence.  The host side here only keeps each
sequence's generator state and recent tokens and hands them to the kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Sequence

import torch

from .. import ops
from ..errors import HosError

_MASK64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    """Names and defaults of the reference's options (src/main.rs:3463-3468)."""
    temp: float = 0.0             # <= 0: greedy
    top_k: int = 40               # 0: off
    top_p: float = 0.95           # >= 1: off
    rep_penalty: float = 1.1      # 1: off
    repeat_last_n: int = 64
    seed: int = 42

    def __post_init__(self):
        # the penalty looks at the last repeat_last_n sampled tokens; a sequence's record keeps 256 of them
        if self.rep_penalty != 1.0 and self.repeat_last_n > ops.RECENT_MAX:
            raise HosError(f"repeat_last_n = {self.repeat_last_n} is more than the {ops.RECENT_MAX} recent tokens "
                           f"that are kept per sequence; use at most {ops.RECENT_MAX} (or rep_penalty = 1)")

    @staticmethod
    def pure(temp: float = 0.0, seed: int = 42) -> "SamplingParams":
        """No top-k, top-p or penalty: the choice is a function of the logits alone
        (what the reference's `generate_ids` uses, src/lib.rs:471-473)."""
        return SamplingParams(temp=temp, top_k=0, top_p=1.0, rep_penalty=1.0, seed=seed)


def next_rand(state: int):
    """xorshift64 (13, 7, 17); the top 24 bits give a float in [0, 1).  src/lib.rs:78-85."""
    x = state
    x ^= (x << 13) & _MASK64
    x ^= x >> 7
    x ^= (x << 17) & _MASK64
    return x, float(x >> 40) / float(1 << 24)


def stream_seed(seed: int, index: int) -> int:
    """The generator state of sequence `index` of a call: seed + index, and never 0
    (xorshift stays at 0 for ever)."""
    s = (seed + index) & _MASK64
    return s if s != 0 else 0x9E3779B97F4A7C15


class Sampler:
    """Per-call sampling state for a set of sequences, identified by any hashable key."""

    def __init__(self, params: SamplingParams, device: torch.device):
        self.params = params
        self.device = device
        self._rng: Dict[object, int] = {}
        self._recent: Dict[object, List[int]] = {}

    def open(self, key, index: int) -> None:
        self._rng[key] = stream_seed(self.params.seed, index)
        self._recent[key] = []

    def close(self, key) -> None:
        self._rng.pop(key, None)
        self._recent.pop(key, None)

    def needs_logits_copy(self) -> bool:
        return False

    def sample(self, logits: torch.Tensor, keys: Sequence) -> List[int]:
        """logits: float32 [len(keys), vocab] on the device.  Returns one token per key
        and records it as recent (the stop token too, as the reference does, :433)."""
        p = self.params
        b = logits.shape[0]
        out = torch.empty((b,), dtype=torch.int32, device=logits.device)
        penal = p.rep_penalty != 1.0 and p.repeat_last_n > 0
        recent_t = recent_len = None
        if penal:
            n = p.repeat_last_n
            rows, lens = [], []
            for k in keys:
                r = self._recent[k][-n:]
                lens.append(len(r))
                rows.append(r + [-1] * (n - len(r)))
            both = torch.tensor([row + [ln] for row, ln in zip(rows, lens)], dtype=torch.int32).to(logits.device)
            recent_t, recent_len = both[:, :n].contiguous(), both[:, n].contiguous()
        if p.temp <= 0.0:
            # greedy: the chunked arg max, with the penalty applied on the fly if there is one
            ops.argmax(logits, out, p.rep_penalty if penal else 1.0, recent_t, recent_len)
        else:
            us = []
            for k in keys:
                self._rng[k], u = next_rand(self._rng[k])
                us.append(u)
            uniforms = torch.tensor(us, dtype=torch.float32).to(logits.device)
            ops.sample(logits, uniforms, out, p.temp, p.top_k, p.top_p,
                       p.rep_penalty if penal else 1.0, recent_t, recent_len)
        toks = out.tolist()
        ops.check_errors()            # the copy waited for the step that made the logits
        for k, t in zip(keys, toks):
            self._recent[k].append(int(t))
        return [int(t) for t in toks]
