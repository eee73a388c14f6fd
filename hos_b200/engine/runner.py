"""The step function: a model, its cache, and `step()`.

A step runs exactly the tokens it is given, as one batch, on top of what earlier
steps left in the cache, and returns float32 logits at the wanted places.  The
sequences of a step either all start at their first token (prompts of unequal
lengths, packed into one batch) or all go on by one token.  Sequences that have
ended are simply absent from later steps; their slots go back with `release`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..cache import CacheManager
from ..config.base import ModelConfig, read_config_json
from .. import ops
from ..errors import ExtensionMissingError, HosError
from ..model import Model
from ..parts.base import Runtime
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
                 device: Optional[torch.device] = None):
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
        self.cache: CacheManager = self.model.new_cache(max_tokens, max_seq_len, max_slots)
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
        if not (from_zero or single):
            raise HosError("step: the sequences of a step either all start at their first token or "
                           "all go on by one token")
        if want is None:
            want = [[len(t) - 1] for t in token_lists]
        rows: List[int] = []
        base = 0
        for toks, w in zip(token_lists, want):
            for j in w:
                if not (0 <= j < len(toks)):
                    raise HosError(f"step: wanted place {j} is outside the {len(toks)} tokens brought")
                rows.append(base + j)
            base += len(toks)
        if single and not from_zero and len(rows) == len(slots) and self.use_sessions:
            # decoding: static buffers and a captured graph, one per batch-size bucket
            from .decode import DecodeSession, bucket_for
            for toks in token_lists:
                if not (0 <= int(toks[0]) < self.vocab_size):
                    raise HosError(f"token id {toks[0]} is outside the vocabulary (0..{self.vocab_size - 1})")
            for s, st in zip(slots, starts):
                self.cache.extend(s, st + 1)
            bucket = bucket_for(len(slots))
            sess = self._sessions.get(bucket)
            if sess is None:
                sess = self._sessions[bucket] = DecodeSession(self, bucket)
            sess.feed(slots, [t[0] for t in token_lists], starts)
            out = sess.run()
            return out.clone() if copy else out
        if from_zero and self.use_sessions and self.prompt_sessions and all(len(w) == 1 and w[0] == len(t) - 1
                                                                          for w, t in zip(want, token_lists)):
            # a short prompt step: static buffers and a captured graph per capacity, as for decoding
            from .decode import PromptSession, prompt_bucket
            bucket = prompt_bucket(sum(len(t) for t in token_lists), len(slots))
            if bucket is not None:
                for toks in token_lists:
                    for t in toks:
                        if not (0 <= int(t) < self.vocab_size):
                            raise HosError(f"token id {t} is outside the vocabulary (0..{self.vocab_size - 1})")
                for s, toks in zip(slots, token_lists):
                    self.cache.extend(s, len(toks))
                sess = self._sessions.get(("prompt",) + bucket)
                if sess is None:
                    sess = self._sessions[("prompt",) + bucket] = PromptSession(self, *bucket)
                sess.feed(slots, token_lists)
                out = sess.run()
                return out.clone() if copy else out
        x, rows_t = self._hidden(slots, starts, token_lists, rows)
        return self.model.logits(x, rows_t)

    def _hidden(self, slots, starts, token_lists, rows=()):
        """The hidden rows of a step, and `rows` (indices into them) as a device tensor."""
        info, rows_t = build_step(token_lists, starts, slots, self.device, self.vocab_size, extra=rows)
        for s, st, toks in zip(slots, starts, token_lists):
            self.cache.extend(s, st + len(toks))
        self.cache.flush()
        # a step of many tokens: its kernels are long enough for the next one's set-up to hide under them
        ops.set_launch_ahead(info.n_tokens >= LAUNCH_AHEAD_MIN_TOKENS)
        try:
            return self.model.hidden(info, self.cache), rows_t
        finally:
            ops.set_launch_ahead(False)

    def decode_steps_timed(self, slots, first_tokens, warmup: int, steps: int, clocks=None):
        """`warmup` untimed and `steps` timed greedy decode steps, issued back to back with
        the chosen tokens staying on the device; timed with CUDA events.  Returns
        (milliseconds per step, kernel-launching calls in the timed region)."""
        from .decode import DecodeSession
        lengths = [self.cache.lengths[s] for s in slots]
        for s, n in zip(slots, lengths):
            self.cache.extend(s, n + warmup + steps)        # pages for every position written
        from .decode import bucket_for
        sess = DecodeSession(self, bucket_for(len(slots)))
        sess.feed(slots, [t[0] for t in first_tokens], lengths)
        for _ in range(warmup):
            sess.run_greedy_on_device()
        torch.cuda.synchronize()
        if clocks is not None:
            clocks.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sess.run_greedy_on_device()
        e1.record()
        torch.cuda.synchronize()
        if clocks is not None:
            clocks.result = clocks.stop()
        return e0.elapsed_time(e1) / steps, sess.launches_per_step * steps

    @property
    def max_seq_len(self) -> int:
        return self.cache.max_seq_len

    def _no_slot(self, s: int):
        raise HosError(f"step: slot {s} holds no sequence")
