"""The generation loop above the step function.

Requests (prompts as token ids) are cut into batches that fit the cache; each
batch runs to its end before the next starts: one step with all its prompts, of
unequal lengths, then one token per live sequence and step.  A sequence ends when
it samples a stop token (which is not returned: src/lib.rs:456-457, :558-560),
when it has `max_new` tokens, or when the context is full (src/lib.rs:440-442);
it then leaves the batch, and its slot goes back to the cache, where a later
batch uses it again.  Unlike the reference's loop (src/lib.rs:443-445) no forward
pass is run for a token after which nothing is sampled.

The loop never waits for a token before it launches the next step: sampled tokens
stay on the device (the next step reads them from the slots' records) and reach
the host one step late.  So a sequence that samples a stop token takes part in
one more step, whose token is dropped, as the reference drops its last forward.
What the host can tell without the tokens (a sequence has all the tokens it may
have, its context is full) it tells at once.

The loop talks to a `backend`, so that its decisions can be tested without a GPU:
    admit(n) -> slots;  release(slot);  length(slot);  max_seq_len (attribute)
    begin(slots, token_lists, indices, max_new, stop_ids)   the first step of each sequence (its prompt,
                       on top of whatever the slot holds) and the first sampling, not waited for
    advance(slots)     one more step, fed with the tokens sampled last, and its sampling
    fetch() -> tokens  of the oldest sampling not yet fetched, in the order of its slots
    settle(slots, ns)  the sequences hold ns tokens (a step that ran for nothing is forgotten)
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

from ..errors import HosError

PAGE = 64          # the unit a sequence takes room in unless the caller says otherwise (the cache's page)


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


def run_batch(backend, prompts: Sequence[Sequence[int]], indices: Sequence[int],
              max_new: int, stop_ids: Sequence[int],
              on_token: Optional[Callable[[int, int], None]] = None,
              slots: Optional[Sequence[int]] = None) -> List[List[int]]:
    """Generate for one batch.  Returns the new tokens of each request of `indices`.  With `slots`
    the sequences live in those slots already (their prompts continue what the slots hold) and
    keep them afterwards; otherwise slots are taken and given back here."""
    stop = set(int(s) for s in stop_ids)
    n = len(indices)
    out: List[List[int]] = [[] for _ in range(n)]
    if max_new <= 0:
        return out
    own = slots is None
    slots = list(backend.admit(n)) if own else list(slots)
    held = [True] * n

    def finish(j: int) -> None:
        if own and held[j]:
            backend.release(slots[j])
        held[j] = False

    try:
        lengths = [backend.length(slots[j]) + len(prompts[indices[j]]) for j in range(n)]
        backend.begin(slots, [list(prompts[i]) for i in indices], list(indices), max_new, sorted(stop))
        launched = list(range(n))          # the sequences of the sampling that is fetched next
        alive = set(launched)
        k = 0                              # how many samplings have been fetched
        while launched:
            # who goes on, as far as that can be told without the tokens of sampling k
            cand = [j for j in launched if j in alive and k + 1 < max_new and lengths[j] < backend.max_seq_len]
            if cand:
                backend.advance([slots[j] for j in cand])
                for j in cand:
                    lengths[j] += 1
            going = set(cand)
            toks = backend.fetch()
            for j, t in zip(launched, toks):
                if j not in alive:
                    continue                               # it had ended: this token came from a step run for nothing
                if t in stop:
                    alive.discard(j)                       # ends; the stop token is not returned
                    if j in going:
                        lengths[j] -= 1                    # the step that is under way feeds it for nothing
                    finish(j)
                    continue
                out[j].append(t)
                if on_token is not None:
                    on_token(indices[j], t)
                if j not in going:                         # has all it may have, or the context is full
                    alive.discard(j)
                    finish(j)
            launched = cand
            k += 1
        if not own:
            backend.settle(slots, lengths)
    finally:
        if own:
            for j in range(n):
                if held[j]:
                    backend.release(slots[j])
    return out


def generate(backend, prompts: Sequence[Sequence[int]],
             max_new: int, stop_ids: Sequence[int], capacity_tokens: int, max_batch: int,
             on_token: Optional[Callable[[int, int], None]] = None, page: int = PAGE) -> List[List[int]]:
    """As many batches one after another as the requests need.  `capacity_tokens`, `page`: what the cache
    holds and the unit in which a sequence takes room there."""
    batches = plan_batches([len(p) for p in prompts], max_new, capacity_tokens, max_batch,
                           backend.max_seq_len, page)
    results: List[List[int]] = [[] for _ in prompts]
    for batch in batches:
        outs = run_batch(backend, prompts, batch, max_new, stop_ids, on_token)
        for i, o in zip(batch, outs):
            results[i] = o
    return results
