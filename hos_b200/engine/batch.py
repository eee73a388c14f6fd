"""Turning a step's host-side description into the device tensors the kernels read."""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..errors import HosError
from ..parts.base import FEW_TOKENS, StepInfo


def build_step(token_lists: Sequence[Sequence[int]], starts: Sequence[int], slots: Sequence[int],
               device: torch.device, vocab_size: int, pad_to: int = 0,
               extra: Optional[Sequence[int]] = None):
    """token_lists[i]: the new tokens of sequence i; starts[i]: its length before the step.
    All the small integer arrays of the step travel in one host-to-device copy, from pinned
    memory when the device is a GPU, so that the host does not wait for the device.  With
    `extra` (a list of integers, e.g. the rows whose logits are wanted) the result is
    (StepInfo, extra as an int32 device tensor) and it rides in the same copy."""
    b = len(token_lists)
    n_fresh = 0                       # the sequences that start at position 0 stand first
    while n_fresh < b and starts[n_fresh] == 0:
        n_fresh += 1
    if any(s == 0 for s in starts[n_fresh:]):
        raise HosError("the sequences of a step that start at position 0 must be listed first")
    news = [len(t) for t in token_lists]
    n_tail = 0                        # and the ones that go on by a few tokens only stand last
    while n_tail < b - n_fresh and news[b - 1 - n_tail] <= FEW_TOKENS:
        n_tail += 1
    n = sum(news)
    nn = max(n, pad_to)
    cu = np.zeros(b + 1, dtype=np.int64)
    np.cumsum(news, out=cu[1:])
    n_extra = len(extra) if extra is not None else 0
    flat = np.empty(4 * nn + (b + 1) + 2 * b + n_extra, dtype=np.int32)
    tokens, pos, seq, tslot = flat[:nn], flat[nn:2 * nn], flat[2 * nn:3 * nn], flat[3 * nn:4 * nn]
    tokens[n:], pos[n:], seq[n:], tslot[n:] = -1, 0, -1, 0       # padding rows
    for i, (toks, start) in enumerate(zip(token_lists, starts)):
        lo, hi = int(cu[i]), int(cu[i + 1])
        if hi == lo:
            continue
        ids = np.asarray(toks, dtype=np.int64)
        if ids.ndim != 1:
            raise HosError("a sequence's tokens must be a flat list of integers")
        if int(ids.min()) < 0 or int(ids.max()) >= vocab_size:
            bad = ids[(ids < 0) | (ids >= vocab_size)][0]
            raise HosError(f"token id {int(bad)} is outside the vocabulary (0..{vocab_size - 1})")
        tokens[lo:hi] = ids
        pos[lo:hi] = np.arange(start, start + hi - lo)
        seq[lo:hi] = i
        tslot[lo:hi] = slots[i]
    o = 4 * nn
    flat[o:o + b + 1] = cu
    flat[o + b + 1:o + 2 * b + 1] = np.asarray(slots, dtype=np.int64)
    lens_after = [s + k for s, k in zip(starts, news)]
    flat[o + 2 * b + 1:o + 3 * b + 1] = lens_after
    if n_extra:
        flat[o + 3 * b + 1:] = np.asarray(extra, dtype=np.int64)
    host = torch.from_numpy(flat)
    if torch.device(device).type == "cuda":
        staged = torch.empty(flat.shape[0], dtype=torch.int32, pin_memory=True)
        staged.copy_(host)
        dev = staged.to(device, non_blocking=True)
    else:
        dev = host.to(device)
    info = StepInfo(
        n_tokens=nn, n_seqs=b, tokens=dev[:nn], token_pos=dev[nn:2 * nn], token_seq=dev[2 * nn:3 * nn],
        token_slot=dev[3 * nn:4 * nn], cu_seqlens=dev[o:o + b + 1], seq_slot=dev[o + b + 1:o + 2 * b + 1],
        seq_len_after=dev[o + 2 * b + 1:o + 3 * b + 1],
        from_zero=all(s == 0 for s in starts),
        single_token=all(k == 1 for k in news),
        max_new=max(news) if news else 0,
        max_len_after=max(lens_after) if lens_after else 0,
        slots_host=tuple(slots), cu_host=tuple(int(c) for c in cu), starts_host=tuple(starts),
        fresh_seqs=n_fresh, fresh_tokens=int(cu[n_fresh]), tail_seqs=n_tail, tail_tokens=int(cu[b] - cu[b - n_tail]))
    if extra is not None:
        return info, dev[o + 3 * b + 1:]
    return info
