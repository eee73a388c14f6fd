"""Turning a step's host-side description into the device tensors the kernels read."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..errors import HosError
from ..parts.base import StepInfo


def build_step(token_lists: Sequence[Sequence[int]], starts: Sequence[int], slots: Sequence[int],
               device: torch.device, vocab_size: int, pad_to: int = 0) -> StepInfo:
    """token_lists[i]: the new tokens of sequence i; starts[i]: its length before the step."""
    tokens: List[int] = []
    pos: List[int] = []
    seq: List[int] = []
    cu = [0]
    for i, (toks, start) in enumerate(zip(token_lists, starts)):
        for j, t in enumerate(toks):
            if not (0 <= int(t) < vocab_size):
                raise HosError(f"token id {t} is outside the vocabulary (0..{vocab_size - 1})")
            tokens.append(int(t))
            pos.append(start + j)
            seq.append(i)
        cu.append(len(tokens))
    n = len(tokens)
    if pad_to > n:
        tokens += [-1] * (pad_to - n)
        pos += [0] * (pad_to - n)
        seq += [-1] * (pad_to - n)
    lens_after = [s + len(t) for s, t in zip(starts, token_lists)]
    # one host-to-device copy for all the small integer arrays
    b = len(token_lists)
    flat = torch.tensor(tokens + pos + seq + cu + list(slots) + lens_after, dtype=torch.int32)
    dev = flat.to(device)
    nn = len(tokens)
    o = 0
    def take(k):
        nonlocal o
        t = dev[o:o + k]
        o += k
        return t
    t_tokens, t_pos, t_seq = take(nn), take(nn), take(nn)
    t_cu, t_slot, t_after = take(b + 1), take(b), take(b)
    news = [len(t) for t in token_lists]
    return StepInfo(
        n_tokens=nn, n_seqs=b, tokens=t_tokens, token_pos=t_pos, token_seq=t_seq,
        cu_seqlens=t_cu, seq_slot=t_slot, seq_len_after=t_after,
        from_zero=all(s == 0 for s in starts),
        single_token=all(k == 1 for k in news),
        max_new=max(news) if news else 0,
        max_len_after=max(lens_after) if lens_after else 0,
        slots_host=tuple(slots), cu_host=tuple(cu), starts_host=tuple(starts))
