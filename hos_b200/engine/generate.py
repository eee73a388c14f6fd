"""The generation loop above the step function.

Requests (prompts as token ids) are cut into batches that fit the cache; each
batch runs to its end before the next starts: one step with all its prompts, of
unequal lengths, then one token per live sequence and step.  A sequence ends when
it samples a stop token (which is not returned: src/lib.rs:456-457, :558-560),
when it has `max_new` tokens, or when the context is full (src/lib.rs:440-442);
it then leaves the batch, and its slot goes back to the cache, where a later
batch uses it again.  Unlike the reference's loop (src/lib.rs:443-445) no forward
pass is run for a token after which nothing is sampled.

The loop talks to a `backend` with four methods, so that its decisions can be
tested without a GPU:
    admit(n) -> slots;  step(slots, token_lists) -> logits handle;
    release(slot);      max_seq_len (attribute)
and to a sampler with open(key, index), sample(logits, keys) -> tokens, close(key).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from ..errors import HosError

PAGE = 64


def rounded(n: int, page: int = PAGE) -> int:
    return (n + page - 1) // page * page


def plan_batches(prompt_lens: Sequence[int], max_new: int, capacity_tokens: int,
                 max_batch: int, max_seq_len: int, page: int = PAGE) -> List[List[int]]:
    """Cut requests, in order, into batches.  A batch takes requests while it has
    fewer than max_batch and the cache can hold every one of them at its longest
    (prompt + max_new, capped by the context, rounded up to whole pages)."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n <= 0:
            raise HosError(f"request {i} has an empty prompt")
        if n > max_seq_len:
            raise HosError(f"request {i} has {n} tokens, more than the context holds ({max_seq_len})")
        need = rounded(min(n + max_new, max_seq_len), page)
        if need > capacity_tokens:
            raise HosError(f"request {i} needs room for {need} tokens, the cache holds {capacity_tokens}")
        if cur and (len(cur) >= max_batch or used + need > capacity_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def run_batch(backend, sampler, prompts: Sequence[Sequence[int]], indices: Sequence[int],
              max_new: int, stop_ids: Sequence[int],
              on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """Generate for one batch.  Returns the new tokens of each request of `indices`."""
    stop = set(int(s) for s in stop_ids)
    n = len(indices)
    out: List[List[int]] = [[] for _ in range(n)]
    if max_new <= 0:
        return out
    slots = backend.admit(n)
    live = list(range(n))                      # positions in `indices` still generating
    lengths = [len(prompts[i]) for i in indices]
    for j, i in enumerate(indices):
        sampler.open(slots[j], i)
    try:
        logits = backend.step([slots[j] for j in live], [list(prompts[indices[j]]) for j in live])
        while live:
            toks = sampler.sample(logits, [slots[j] for j in live])
            still, feed = [], []
            for j, t in zip(live, toks):
                if t in stop:
                    continue                               # ends; the stop token is not returned
                out[j].append(t)
                if on_token is not None:
                    on_token(indices[j], t)
                if len(out[j]) >= max_new:
                    continue                               # has all it may have
                if lengths[j] >= backend.max_seq_len:
                    continue                               # the context is full
                still.append(j)
                feed.append([t])
            for j in live:
                if j not in still:
                    sampler.close(slots[j])
                    backend.release(slots[j])
                    slots[j] = -1
            live = still
            if not live:
                break
            logits = backend.step([slots[j] for j in live], feed)
            for j in live:
                lengths[j] += 1
    finally:
        for j in range(n):
            if slots[j] >= 0:
                sampler.close(slots[j])
                backend.release(slots[j])
    return out


def generate(backend, make_sampler: Callable[[], object], prompts: Sequence[Sequence[int]],
             max_new: int, stop_ids: Sequence[int], capacity_tokens: int, max_batch: int,
             on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
    """As many batches one after another as the requests need."""
    batches = plan_batches([len(p) for p in prompts], max_new, capacity_tokens, max_batch,
                           backend.max_seq_len)
    results: List[List[int]] = [[] for _ in prompts]
    sampler = make_sampler()
    for batch in batches:
        outs = run_batch(backend, sampler, prompts, batch, max_new, stop_ids, on_token)
        for i, o in zip(batch, outs):
            results[i] = o
    return results
