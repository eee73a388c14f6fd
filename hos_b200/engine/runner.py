"""The step function: a model, its cache, and `step()`.

A step runs exactly the tokens it is given, as one batch, on top of what earlier
steps left in the cache, and returns float32 logits at the wanted places.  Each
sequence of a step brings its next tokens, one or many, whether it starts at its
first token or goes on from where the cache left it (src/forward.rs:247-253: a
prompt is run from any `start`; src/lib.rs:352-366: in chunks).  Two shapes have
fast paths: prompts that all start at position 0 (short ones replayed as a CUDA
graph), and sequences that all go on by one token (always replayed).  Everything
else is the general case: the sequences that start at position 0 attend over their
own rows, the others over the cache; a sequence that brings more tokens than the
window rings have room for is fed in several passes.  Sequences that have ended
are simply absent from later steps; their slots go back with `release`.
"""
from __future__ import annotations

import contextlib
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..config.base import ModelConfig, read_config_json
from .. import ops
from ..errors import ExtensionMissingError, HosError
from ..model import Model
from ..parts.base import FEW_TOKENS, Runtime
from ..registry import config_from_dict, plan_for
from ..weights import RandomSource, SafetensorsFolder, load_tensors
from .batch import build_step

LAUNCH_AHEAD_MIN_TOKENS = 256       # steps of at least this many tokens launch their kernels ahead
DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise ExtensionMissingError("no CUDA device is visible: this library runs on the GPU only")
    return torch.device("cuda", torch.cuda.current_device())


class Runner:
    def __init__(self, config: ModelConfig, source, dtype: str = "bfloat16", max_tokens: int = 8192,
                 max_seq_len: Optional[int] = None, max_slots: Optional[int] = None,
                 device: Optional[torch.device] = None, chunk_tokens: int = 2048):
        """`chunk_tokens`: the most tokens a step adds in one pass to a sequence that is under way
        (layers that keep a window of keys make their ring of pages that much longer; a step
        that brings more is run as several passes)."""
        if dtype not in DTYPES:
            raise HosError(f"dtype must be one of {sorted(DTYPES)}, found {dtype!r}")
        self.config = config
        self.device = device or _device()
        self.rt = Runtime(self.device, DTYPES[dtype])
        self.plan = plan_for(config)
        self.model = Model(self.plan, self.rt)
        tensors = load_tensors(self.model.weight_specs(), source, self.device)
        self.model.bind(tensors)
        del tensors
        self.cache: CacheManager = self.model.new_cache(max_tokens, max_seq_len, max_slots, chunk_tokens)
        self.vocab_size = self.plan.vocab_size
        self._sessions = {}
        self.use_sessions = self.model.graph_safe     # single-token steps run through DecodeSession
        self.prompt_sessions = True                   # and short prompt steps through PromptSession

    @classmethod
    def from_folder(cls, model_dir: str, **kw) -> "Runner":
        raw = read_config_json(model_dir)
        config = config_from_dict(raw)
        src = SafetensorsFolder(model_dir)
        try:
            return cls(config, src, **kw)
        finally:
            src.close()

    @classmethod
    def from_random(cls, config: ModelConfig, seed: int, **kw) -> "Runner":
        """Random weights made on the device (no file): for measurements."""
        from ..model import weight_specs_for
        dev = kw.get("device") or _device()
        src = RandomSource(weight_specs_for(config), seed, device=str(dev))
        return cls(config, src, **kw)

    # ---- sequences ------------------------------------------------------------------
    def admit(self, n: int) -> List[int]:
        """Slots for n new sequences (pages come with their first step)."""
        return self.cache.admit([0] * n)

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    # ---- the step -------------------------------------------------------------------
    def step(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None, copy: bool = True) -> torch.Tensor:
        """Run `token_lists[i]` as the next tokens of the sequence in `slots[i]`.
        `want[i]` lists the places among sequence i's new tokens whose logits are
        returned (default: the last one); the result is float32
        [sum of len(want[i]), vocab], in the order of the sequences and of `want`.
        With copy=False the result of a single-token step is a view of a buffer that the
        next step overwrites (the generation loop reads it at once)."""
        if len(slots) != len(token_lists):
            raise HosError("step: one token list per slot is needed")
        if len(set(slots)) != len(slots):
            raise HosError("step: a slot appears twice in one step")
        if not slots:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        starts = []
        for s, toks in zip(slots, token_lists):
            if len(toks) == 0:
                raise HosError("step: a sequence brings no token")
            starts.append(self.cache.lengths[s] if s in self.cache.lengths else self._no_slot(s))
        from_zero = all(st == 0 for st in starts)
        single = all(len(t) == 1 for t in token_lists)
        if want is None:
            want = [[len(t) - 1] for t in token_lists]
        for toks, w in zip(token_lists, want):
            for j in w:
                if not (0 <= j < len(toks)):
                    raise HosError(f"step: wanted place {j} is outside the {len(toks)} tokens brought")
        last_only = all(len(w) == 1 and w[0] == len(t) - 1 for w, t in zip(want, token_lists))
        if single and not from_zero and last_only and self.use_sessions:
            # decoding: static buffers and a captured graph, one per batch-size bucket
            self._check_ids(token_lists)
            self.cache.extend_all(slots, [st + 1 for st in starts])
            with self._lengths_back_on_error(slots, starts):
                sess = self.decode_session(len(slots))
                sess.upload(slots, [t[0] for t in token_lists], lengths=[st + 1 for st in starts])
                out = sess.run_step()
            return out.clone() if copy else out
        if from_zero and last_only and self.use_sessions and self.prompt_sessions:
            # a short prompt step: static buffers and a captured graph per capacity, as for decoding
            from .decode import PromptSession, prompt_bucket
            bucket = prompt_bucket(sum(len(t) for t in token_lists), len(slots))
            if bucket is not None:
                self._check_ids(token_lists)
                self.cache.extend_all(slots, [len(t) for t in token_lists])
                with self._lengths_back_on_error(slots, starts):
                    sess = self._sessions.get(("prompt",) + bucket)
                    if sess is None:
                        sess = self._sessions[("prompt",) + bucket] = PromptSession(self, *bucket)
                    sess.feed(slots, token_lists)
                    out = sess.run()
                return out.clone() if copy else out
        if not single and last_only and self.use_sessions and self.prompt_sessions and all(st > 0 for st in starts):
            # a short step of sequences that go on by several tokens (a second turn): replayed too
            from .decode import PromptSession, length_class, prompt_bucket
            bucket = prompt_bucket(sum(len(t) for t in token_lists), len(slots))
            room = self.cache.chunk_room()
            if bucket is not None and (room is None or bucket[0] <= room):
                self._check_ids(token_lists)
                self.cache.extend_all(slots, [st + len(t) for st, t in zip(starts, token_lists)])
                with self._lengths_back_on_error(slots, starts):
                    planned = length_class(max(st + len(t) for st, t in zip(starts, token_lists)), self.cache.max_seq_len)
                    key = ("turn",) + bucket + (planned,)
                    sess = self._sessions.get(key)
                    if sess is None:
                        sess = self._sessions[key] = PromptSession(self, *bucket, continuing=True, planned_len=planned)
                    sess.feed(slots, token_lists, starts)
                    out = sess.run()
                return out.clone() if copy else out
        return self._general(slots, starts, token_lists, want)

    @contextlib.contextmanager
    def _lengths_back_on_error(self, slots, starts):
        """A step that fails after its sequences were given their pages leaves them as long as they were (the
        pages stay theirs; what the failed step may have stored lies beyond their lengths and is never read)."""
        try:
            yield
        except Exception:
            for s, st in zip(slots, starts):
                if s in self.cache.lengths:
                    self.cache.lengths[s] = st
            try:                     # the records on the device too, if the device still takes work
                live = [(s, st) for s, st in zip(slots, starts) if s in self.cache.lengths]
                self.write_records([s for s, _ in live], pos=[st for _, st in live])
            except Exception:
                pass
            raise

    def decode_session(self, n: int):
        """The session that runs single-token steps of n sequences (one per batch-size bucket)."""
        from .decode import DecodeSession, bucket_for
        bucket = bucket_for(n)
        sess = self._sessions.get(bucket)
        if sess is None:
            sess = self._sessions[bucket] = DecodeSession(self, bucket)
        return sess

    def write_records(self, slots: Sequence[int], pos=None, last=None, rng=None, limit=None,
                      restart: bool = False) -> None:
        """Words of the slots' device records (csrc/slot_state.cu) set from the host: `pos` (with it the
        host's own count of the sequence's tokens; pages are the caller's business), `last` (the token a
        record-driven step feeds next), `rng` (generator states, 64-bit), `limit` (most tokens to sample);
        `restart` clears the finished flag and the count of sampled tokens, and with it the recent tokens."""
        n = len(slots)
        vals = np.zeros((n, ops.SLOT_WORDS), dtype=np.int64)
        mask = 0
        if pos is not None:
            vals[:, ops.SLOT_POS] = pos
            mask |= 1 << ops.SLOT_POS
            for s, p in zip(slots, pos):
                if s not in self.cache.lengths:
                    self._no_slot(s)
                self.cache.lengths[s] = int(p)
        if last is not None:
            vals[:, ops.SLOT_LAST] = last
            mask |= 1 << ops.SLOT_LAST
        if rng is not None:
            r = np.asarray([int(x) & ((1 << 64) - 1) for x in rng], dtype=np.uint64)
            vals[:, ops.SLOT_RNG_LO] = (r & np.uint64(0xffffffff)).astype(np.int64)
            vals[:, ops.SLOT_RNG_HI] = (r >> np.uint64(32)).astype(np.int64)
            mask |= (1 << ops.SLOT_RNG_LO) | (1 << ops.SLOT_RNG_HI)
        if limit is not None:
            vals[:, ops.SLOT_LIMIT] = limit
            mask |= 1 << ops.SLOT_LIMIT
        if restart:
            mask |= (1 << ops.SLOT_FLAGS) | (1 << ops.SLOT_COUNT)
        if not mask or n == 0:
            return
        host = np.concatenate([(vals & 0xffffffff).astype(np.uint32).view(np.int32).reshape(-1),
                               np.asarray(slots, dtype=np.int32)])
        staged = torch.empty(host.shape[0], dtype=torch.int32, pin_memory=True)
        staged.copy_(torch.from_numpy(host))
        dev = staged.to(self.device, non_blocking=True)
        ops.slot_write(self.cache.record, dev[n * ops.SLOT_WORDS:], dev[:n * ops.SLOT_WORDS].view(n, ops.SLOT_WORDS), mask)

    def _check_ids(self, token_lists) -> None:
        for toks in token_lists:
            for t in toks:
                if not (0 <= int(t) < self.vocab_size):
                    raise HosError(f"token id {t} is outside the vocabulary (0..{self.vocab_size - 1})")

    def _general(self, slots, starts, token_lists, want) -> torch.Tensor:
        """Any mix of sequences that start and sequences that go on by any number of tokens.
        The sequences that start at position 0 are listed first (the mixers send them to the
        kernels that attend over a step's own rows).  A sequence that goes on brings at most
        `cache.chunk_room()` tokens per pass, so that in a ring of pages no key is overwritten
        that a token of the same pass still reads; what is left over runs in further passes."""
        self._check_ids(token_lists)
        # all or nothing: every sequence gets its pages for the whole step before anything runs
        self.cache.extend_all(slots, [st + len(t) for st, t in zip(starts, token_lists)])
        with self._lengths_back_on_error(slots, starts):
            return self._passes(slots, starts, token_lists, want)

    def _passes(self, slots, starts, token_lists, want) -> torch.Tensor:
        room = self.cache.chunk_room()
        # stable: the sequences that start come first, the ones that go on by a few tokens last
        order = sorted(range(len(slots)),
                       key=lambda i: 0 if starts[i] == 0 else (1 if len(token_lists[i]) > FEW_TOKENS else 2))
        first_row = [0] * len(slots)          # where each sequence's rows begin in the result
        at = 0
        for i, w in enumerate(want):
            first_row[i] = at
            at += len(w)
        n_out = at
        done = [0] * len(slots)               # tokens of each sequence already run
        out = None
        while True:
            part = []                         # (sequence, first token, tokens) of this pass
            for i in order:
                left = len(token_lists[i]) - done[i]
                if left <= 0:
                    continue
                take = left if (starts[i] == 0 and done[i] == 0) or room is None else min(left, room)
                part.append((i, done[i], take))
            if not part:
                break
            rows, dest = [], []
            base = 0
            for i, lo, k in part:
                for j, place in enumerate(want[i]):
                    if lo <= place < lo + k:
                        rows.append(base + place - lo)
                        dest.append(first_row[i] + j)
                base += k
            x, rows_t = self._hidden([slots[i] for i, _, _ in part], [starts[i] + lo for i, lo, _ in part],
                                     [token_lists[i][lo:lo + k] for i, lo, k in part], rows, extend=False)
            for i, lo, k in part:
                done[i] = lo + k
            if not rows:
                continue
            logits = self.model.logits(x, rows_t)
            if len(dest) == n_out and dest == list(range(n_out)):
                return logits                 # one pass gave every wanted row, in order
            if out is None:
                out = torch.empty((n_out, self.vocab_size), dtype=torch.float32, device=self.device)
            out[torch.tensor(dest, dtype=torch.long, device=self.device)] = logits
        if out is None:
            out = torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        return out

    def hidden_states(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]]) -> List[torch.Tensor]:
        """Run the tokens as `step` does (one pass, kernel by kernel) and return the residual stream
        after the embedding and after every entry of the run order, float32 [tokens, width] each, rows in
        the order of the sequences given (which must list the ones that start at position 0 first).  For
        finding the layer at which two paths (bfloat16 and 32-bit, or this library and another
        implementation) part ways."""
        starts = [self.cache.lengths[s] if s in self.cache.lengths else self._no_slot(s) for s in slots]
        self._check_ids(token_lists)
        tap: List[torch.Tensor] = []
        self._hidden(slots, starts, token_lists, tap=tap)
        return tap

    def _hidden(self, slots, starts, token_lists, rows=(), extend: bool = True, tap=None):
        """The hidden rows of one pass, and `rows` (indices into them) as a device tensor.  The
        sequences that start at position 0 must come first."""
        info, rows_t = build_step(token_lists, starts, slots, self.device, self.vocab_size, extra=rows)
        if extend:
            self.cache.extend_all(slots, [st + len(t) for st, t in zip(starts, token_lists)])
        self.cache.flush()
        # a step of many tokens: its kernels are long enough for the next one's set-up to hide under them
        ops.set_launch_ahead(info.n_tokens >= LAUNCH_AHEAD_MIN_TOKENS)
        try:
            x = self.model.hidden(info, self.cache, tap)
            # the slots' records learn the new lengths (single-token steps take positions from them)
            ops.slot_set_pos(self.cache.record, info.seq_slot, info.seq_len_after, info.cu_seqlens, info.n_seqs)
            return x, rows_t
        finally:
            ops.set_launch_ahead(False)

    def decode_steps_timed(self, slots, first_tokens, warmup: int, steps: int, clocks=None):
        """`warmup` untimed and `steps` timed greedy decode steps, issued back to back with
        the chosen tokens staying on the device (the records); timed with CUDA events.  Returns
        (milliseconds per step, kernel-launching calls in the timed region)."""
        from ..sampling.sampler import SamplingParams
        lengths = [self.cache.lengths[s] for s in slots]
        self.cache.extend_all(slots, [n + warmup + steps for n in lengths])     # pages for every position written
        for s, n in zip(slots, lengths):
            self.cache.lengths[s] = n
        self.write_records(slots, pos=lengths, last=[t[0] for t in first_tokens], limit=[0] * len(slots), restart=True)
        sess = self.decode_session(len(slots))
        sess.upload(slots, lengths=[n + warmup + steps for n in lengths])
        greedy = SamplingParams.pure()
        for _ in range(warmup):
            sess.run_generate(greedy)
        torch.cuda.synchronize()
        if clocks is not None:
            clocks.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sess.run_generate(greedy)
        e1.record()
        torch.cuda.synchronize()
        if clocks is not None:
            clocks.result = clocks.stop()
        for s, n in zip(slots, lengths):
            self.cache.lengths[s] = n + warmup + steps
        return e0.elapsed_time(e1) / steps, sess.launches_per_step * steps

    def wait(self) -> None:
        """Wait for the steps launched so far, and raise KernelError if one of their kernels gave up a
        bounded wait (a caller that reads `step`'s logits by other means calls `ops.check_errors()`
        after its own synchronisation)."""
        torch.cuda.synchronize(self.device)
        ops.check_errors()

    @property
    def max_seq_len(self) -> int:
        return self.cache.max_seq_len

    def _no_slot(self, s: int):
        raise HosError(f"step: slot {s} holds no sequence")
