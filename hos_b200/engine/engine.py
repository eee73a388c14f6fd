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
from typing import Optional, Sequence, Tuple, Union

import torch

from ..config.base import ModelConfig
from ..errors import HosError
from ..sampling import Sampler, SamplingParams
from . import generate as gen
from .runner import Runner

Prompt = Union[Sequence[int], Sequence[Sequence[int]]]


class _LoopBackend:
    """What the generation loop drives: the runner, with logits handed over without a copy
    (the loop samples from them before the next step overwrites them)."""

    def __init__(self, runner: Runner):
        self.runner = runner
        self.admit, self.release = runner.admit, runner.release

    @property
    def max_seq_len(self) -> int:
        return self.runner.max_seq_len

    def step(self, slots, token_lists):
        return self.runner.step(slots, token_lists, copy=False)


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
        outs = gen.generate(_LoopBackend(self.runner), lambda: Sampler(params, self.runner.device), prompts,
                            max_tokens, stops, self.runner.cache.tokens_capacity(), self.max_batch,
                            on_token)
        return outs if batch else outs[0]

    # ---- the step function, for callers that drive it themselves ------------------------
    def step(self, slots, token_lists, want=None, copy: bool = True) -> torch.Tensor:
        return self.runner.step(slots, token_lists, want, copy)

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
        mean = nll / len(feed)
        return len(feed), mean, math.exp(mean)

    def bench(self, prompt: Prompt, decode_tokens: int = 64):
        """Time the prompt step and greedy decoding separately, after one warm-up prompt
        step (src/lib.rs:683-727).  `prompt` is one prompt or a batch of them (decoded
        together; a sequence that meets a stop token or the context's end leaves the batch).
        Returns (prefill_tokens, prefill_secs, prefill_tps, decode_tokens, decode_secs,
        decode_tps), tokens counted over the batch."""
        r = self.runner
        prompts = [list(p) for p in prompt] if _is_batch(prompt) else [list(prompt)]
        n_prompt = sum(len(p) for p in prompts)
        sampler = Sampler(SamplingParams.pure(), r.device)
        slots = r.admit(len(prompts))
        r.step(slots, prompts)
        for s in slots:
            r.release(s)
        slots = r.admit(len(prompts))
        for i, s in enumerate(slots):
            sampler.open(s, i)
        live = list(slots)
        try:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            logits = r.step(live, prompts)
            torch.cuda.synchronize()
            prefill_secs = time.perf_counter() - t0
            produced = 0
            t1 = time.perf_counter()
            for _ in range(decode_tokens):
                toks = sampler.sample(logits, live)
                keep = [i for i, (s, t) in enumerate(zip(live, toks))
                        if t not in self.stop_ids and r.length(s) < r.max_seq_len]
                if not keep:
                    break
                live, toks = [live[i] for i in keep], [toks[i] for i in keep]
                logits = r.step(live, [[t] for t in toks])
                produced += len(live)
            torch.cuda.synchronize()
            decode_secs = time.perf_counter() - t1
        finally:
            for s in slots:
                sampler.close(s)
                r.release(s)
        return (n_prompt, prefill_secs, n_prompt / max(prefill_secs, 1e-9),
                produced, decode_secs, produced / max(decode_secs, 1e-9))

    def vocab_size(self) -> int:
        return self.runner.vocab_size
