"""The Python entry point, in the manner of the reference's binding (py/src/lib.rs:12-92):
`Engine(path)`, `generate(prompt, max_tokens=128, temp=0.0, top_k=40, top_p=0.95,
rep_penalty=1.1, repeat_last_n=64, seed=42)`, `perplexity`, `bench`, `vocab_size`.
Prompts and results are token ids (tokenizers are not part of this library): a
prompt is a list of ids, or a list of such lists, which is run as batches.
Bad input raises `ValueError` (every `HosError` is one), as the binding does.
"""
from __future__ import annotations

import math
import time
from typing import List, Optional, Sequence, Tuple, Union

import torch

from ..config.base import ModelConfig
from ..errors import HosError
from ..sampling import SamplingParams, stream_seed
from . import generate as gen
from .runner import Runner

Prompt = Union[Sequence[int], Sequence[Sequence[int]]]


class _DeviceBackend:
    """What the generation loop drives: the runner's step function for each sequence's first
    step, then record-driven single-token steps with sampling on the device.  Tokens come back
    through pinned buffers, fetched in the order in which they were sampled."""

    def __init__(self, runner: Runner, params: SamplingParams):
        self.runner = runner
        self.params = params
        self.admit, self.release, self.length = runner.admit, runner.release, runner.length
        self._queue: List[object] = []
        self._stops: Sequence[int] = ()

    @property
    def max_seq_len(self) -> int:
        return self.runner.max_seq_len

    def begin(self, slots, token_lists, indices, max_new, stop_ids) -> None:
        r, p = self.runner, self.params
        self._stops = tuple(stop_ids)
        logits = r.step(slots, token_lists, copy=False)
        # each sequence's generator starts from seed + index (src/lib.rs:404-407), the recent tokens are none
        r.write_records(slots, rng=[stream_seed(p.seed, i) for i in indices], limit=[max_new] * len(slots),
                        restart=True)
        sess = r.decode_session(len(slots))
        sess.upload(slots, stop_ids=self._stops)
        sess.sample_logits(logits, p)
        self._queue.append(sess.fetch_start())

    def advance(self, slots) -> None:
        r = self.runner
        r.cache.extend_all(slots, [r.cache.lengths[s] + 1 for s in slots])
        sess = r.decode_session(len(slots))
        sess.upload(slots, stop_ids=self._stops, lengths=[r.cache.lengths[s] for s in slots])
        sess.run_generate(self.params)
        self._queue.append(sess.fetch_start())

    def fetch(self) -> List[int]:
        from .decode import DecodeSession
        return DecodeSession.fetch_read(self._queue.pop(0))

    def settle(self, slots, lengths) -> None:
        self.runner.write_records(slots, pos=lengths)


def _is_batch(prompt) -> bool:
    return len(prompt) > 0 and not isinstance(prompt[0], int)


class Engine:
    """A loaded model, its cache and the generation loop.

    path        a folder with config.json and model.safetensors (or shards + index)
    gpu         kept for the reference's signature; this library always runs on the GPU
    dtype       "bfloat16" (the fast kernels) or "float32" (everything in true 32-bit)
    max_batch   most sequences generated side by side
    max_tokens  tokens the cache holds (default: max_batch full contexts, at most 8192 each)
    """

    def __init__(self, path: Optional[str] = None, gpu: bool = True, dtype: str = "bfloat16",
                 max_batch: int = 8, max_tokens: Optional[int] = None,
                 max_seq_len: Optional[int] = None, _runner: Optional[Runner] = None):
        self.max_batch = max_batch
        if _runner is not None:
            self.runner = _runner
        else:
            if path is None:
                raise HosError("Engine needs the path of a model folder")
            from ..config.base import read_config_json
            from ..registry import config_from_dict
            from .. import models  # noqa: F401
            cfg = config_from_dict(read_config_json(path))
            self.runner = Runner.from_folder(path, dtype=dtype, max_seq_len=max_seq_len,
                                             max_tokens=self._default_tokens(cfg, max_batch, max_tokens,
                                                                             max_seq_len))
        self.config = self.runner.config
        self.stop_ids: Tuple[int, ...] = tuple(self.runner.plan.stop_token_ids)

    @staticmethod
    def _default_tokens(cfg, max_batch, max_tokens, max_seq_len) -> int:
        if max_tokens is not None:
            return max_tokens
        ctx = min(getattr(cfg, "max_position_embeddings", 8192), max_seq_len or 8192)
        return max_batch * gen.rounded(ctx)

    @classmethod
    def from_config(cls, config: ModelConfig, seed: int = 0, dtype: str = "bfloat16",
                    max_batch: int = 8, max_tokens: Optional[int] = None,
                    max_seq_len: Optional[int] = None) -> "Engine":
        """A model with random weights made on the device (no files)."""
        runner = Runner.from_random(config, seed, dtype=dtype, max_seq_len=max_seq_len,
                                    max_tokens=cls._default_tokens(config, max_batch, max_tokens,
                                                                   max_seq_len))
        return cls(max_batch=max_batch, _runner=runner)

    # ---- generation -------------------------------------------------------------------
    def generate(self, prompt: Prompt, max_tokens: int = 128, temp: float = 0.0, top_k: int = 40,
                 top_p: float = 0.95, rep_penalty: float = 1.1, repeat_last_n: int = 64,
                 seed: int = 42, stop_ids: Optional[Sequence[int]] = None, on_token=None):
        """New token ids for the prompt (a list) or for each prompt (a list of lists).
        A stop token (the model's eos ids unless `stop_ids` is given) ends a sequence
        and is not returned."""
        params = SamplingParams(temp, top_k, top_p, rep_penalty, repeat_last_n, seed)
        return self._generate(prompt, max_tokens, params, stop_ids, on_token)

    def generate_ids(self, prompt: Prompt, max_tokens: int, temp: float = 0.0, seed: int = 42,
                     stop_ids: Optional[Sequence[int]] = None):
        """As `generate` with top-k, top-p and the penalty off: with temp <= 0 the result
        is a function of the logits alone (src/lib.rs:458-486)."""
        return self._generate(prompt, max_tokens, SamplingParams.pure(temp, seed), stop_ids, None)

    def _generate(self, prompt, max_tokens, params, stop_ids, on_token):
        batch = _is_batch(prompt)
        prompts = [list(p) for p in prompt] if batch else [list(prompt)]
        stops = self.stop_ids if stop_ids is None else tuple(stop_ids)
        outs = gen.generate(_DeviceBackend(self.runner, params), prompts, max_tokens, stops,
                            self.runner.cache.tokens_capacity(), self.max_batch, on_token,
                            page=self.runner.cache.page_tokens)
        return outs if batch else outs[0]

    # ---- sequences that stay: a second turn continues where the first ended --------------------
    def open(self, n: int = 1) -> List["Conversation"]:
        """n sequences that keep their slots between calls (`generate_from_ids` continues them,
        `Conversation.reset` starts one afresh, `Conversation.close` gives its slot back)."""
        return [Conversation(self, s) for s in self.runner.admit(n)]

    def generate_from_ids(self, conversations: Sequence["Conversation"], ids: Sequence[Sequence[int]],
                          max_tokens: int = 128, temp: float = 0.0, top_k: int = 40, top_p: float = 0.95,
                          rep_penalty: float = 1.1, repeat_last_n: int = 64, seed: int = 42,
                          stop_ids: Optional[Sequence[int]] = None, on_token=None) -> List[List[int]]:
        """Feed `ids[i]` to conversation i on top of what it holds and generate, all conversations
        side by side (src/lib.rs:499-503: continues from the current position, does not reset; the
        caller owns the prompt).  Long prompts are fed in pieces by the step function.  A token that
        the last call returned last is fed first (it was sampled but never run)."""
        params = SamplingParams(temp, top_k, top_p, rep_penalty, repeat_last_n, seed)
        stops = self.stop_ids if stop_ids is None else tuple(stop_ids)
        if len(conversations) != len(ids):
            raise HosError("generate_from_ids: one list of ids per conversation is needed")
        prompts = []
        for c, new in zip(conversations, ids):
            c._check_open()
            p = ([c.pending] if c.pending is not None else []) + [int(t) for t in new]
            if not p:
                raise HosError("generate_from_ids: a conversation brings no token")
            if self.runner.length(c.slot) + len(p) > self.runner.max_seq_len:
                raise HosError(f"generate_from_ids: {self.runner.length(c.slot)} tokens held and {len(p)} more are "
                               f"more than the context holds ({self.runner.max_seq_len})")
            prompts.append(p)
        outs = gen.run_batch(_DeviceBackend(self.runner, params), prompts, list(range(len(prompts))), max_tokens,
                             stops, on_token, slots=[c.slot for c in conversations])
        for c, p, o in zip(conversations, prompts, outs):
            # the last returned token has been sampled but not run, unless the context is full
            fed = self.runner.length(c.slot) - c.position - len(p)
            c.position = self.runner.length(c.slot)
            c.pending = o[-1] if o and fed < len(o) else None
        return outs

    # ---- the step function, for callers that drive it themselves ------------------------
    def step(self, slots, token_lists, want=None, copy: bool = True) -> torch.Tensor:
        return self.runner.step(slots, token_lists, want, copy)

    # ---- embeddings ----------------------------------------------------------------------
    def embed(self, ids: Sequence[int], pooling: str = "mean") -> torch.Tensor:
        """The final hidden state (after the last norm, before the head) of a token sequence, pooled: "mean" over
        all its tokens, or "last" (py/src/lib.rs:50-63, src/lib.rs:285-326).  Runs on a slot of its own, so
        sequences that are under way are untouched.  float32 [width], on the device."""
        if pooling not in ("mean", "last"):
            raise HosError("pooling must be 'mean' or 'last'")
        ids = list(ids)
        if not ids:
            raise HosError("embed: no tokens")
        if len(ids) > self.runner.max_seq_len:
            raise HosError(f"embed: {len(ids)} tokens are more than the context holds ({self.runner.max_seq_len})")
        r = self.runner
        slot = r.admit(1)[0]
        try:
            x, _ = r._hidden([slot], [0], [ids])
            if pooling == "last":
                x = x[-1:].contiguous()
            h = r.model.final_norm.forward(x).float()
        finally:
            r.release(slot)
        return h.mean(dim=0) if pooling == "mean" else h[0]

    # ---- measurements -------------------------------------------------------------------
    def perplexity(self, ids: Sequence[int]) -> Tuple[int, float, float]:
        """(scored tokens, mean negative log-likelihood in nats, perplexity) of a token
        sequence, each token scored given the ones before it with an exact log-softmax
        (src/lib.rs:655-679).  One prompt step; the head runs over chunks of rows."""
        ids = list(ids)[: self.runner.max_seq_len]
        if len(ids) < 2:
            return 0, 0.0, 1.0
        r = self.runner
        slot = r.admit(1)[0]
        try:
            feed = ids[:-1]
            x, _ = r._hidden([slot], [0], [feed])
            nll = 0.0
            for lo in range(0, len(feed), 256):
                hi = min(lo + 256, len(feed))
                rows = torch.arange(lo, hi, dtype=torch.int32, device=r.device)
                logits = r.model.logits(x, rows).double()
                target = torch.tensor(ids[lo + 1:hi + 1], device=r.device)
                lse = torch.logsumexp(logits, dim=-1)
                nll += float((lse - logits.gather(1, target[:, None])[:, 0]).sum())
        finally:
            r.release(slot)
        from .. import ops
        ops.check_errors()
        mean = nll / len(feed)
        return len(feed), mean, math.exp(mean)

    def bench(self, prompt: Prompt, decode_tokens: int = 64):
        """Time the prompt step and greedy decoding separately, after a warm-up of one prompt
        step and two decode steps (src/lib.rs:683-727).  `prompt` is one prompt or a batch of them (decoded
        together; a sequence that meets a stop token or the context's end leaves the batch).
        Returns (prefill_tokens, prefill_secs, prefill_tps, decode_tokens, decode_secs,
        decode_tps), tokens counted over the batch."""
        r = self.runner
        prompts = [list(p) for p in prompt] if _is_batch(prompt) else [list(prompt)]
        n_prompt = sum(len(p) for p in prompts)
        backend = _DeviceBackend(r, SamplingParams.pure())
        # the warm-up: the prompt step and two decode steps (kernels built, graphs captured)
        gen.run_batch(backend, prompts, list(range(len(prompts))), 3, ())
        times = {}

        class Timed:                                # the loop's backend, with a clock around the first step
            max_seq_len = r.max_seq_len
            admit, release, length, advance, fetch, settle = (backend.admit, backend.release, backend.length,
                                                              backend.advance, backend.fetch, backend.settle)

            @staticmethod
            def begin(*a):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                backend.begin(*a)
                torch.cuda.synchronize()
                times["prefill"] = time.perf_counter() - t0
                times["t1"] = time.perf_counter()

        # one more token than asked for: the first one belongs to the prompt step
        outs = gen.run_batch(Timed, prompts, list(range(len(prompts))), decode_tokens + 1, self.stop_ids)
        torch.cuda.synchronize()
        decode_secs = time.perf_counter() - times["t1"]
        produced = sum(max(0, len(o) - 1) for o in outs)
        prefill_secs = times["prefill"]
        return (n_prompt, prefill_secs, n_prompt / max(prefill_secs, 1e-9),
                produced, decode_secs, produced / max(decode_secs, 1e-9))

    def vocab_size(self) -> int:
        return self.runner.vocab_size


class Conversation:
    """One sequence that keeps its slot, its keys and values and its position between calls of
    `Engine.generate_from_ids` (the reference's engine is one such sequence: src/lib.rs:175-184,
    `reset` :489-492)."""

    def __init__(self, engine: Engine, slot: int):
        self.engine = engine
        self.slot: Optional[int] = slot
        self.position = 0                       # tokens in the cache
        self.pending: Optional[int] = None      # a returned token that has not been run yet

    def _check_open(self) -> None:
        if self.slot is None:
            raise HosError("this conversation is closed")

    def reset(self) -> None:
        """Forget everything: the next call starts at position 0 (pages go back, the slot stays)."""
        self._check_open()
        r = self.engine.runner
        r.release(self.slot)
        new = r.admit(1)[0]
        self.slot, self.position, self.pending = new, 0, None

    def close(self) -> None:
        if self.slot is not None:
            self.engine.runner.release(self.slot)
            self.slot = None
