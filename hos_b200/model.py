"""A model built from a plan: the embedding, one arrangement object per layer (each
holding its mixer, feed-forward and norms), the final norm and the head, plus the
run order.  It knows nothing about any architecture: everything comes from the
`ModelPlan` and the part registry."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import ops
from . import parts as _parts  # noqa: F401  (registers the parts)
from . import models as _models  # noqa: F401  (registers the architectures)
from .cache import CacheManager
from .config.base import ModelConfig, ModelPlan
from .parts.base import Runtime, StepInfo, WeightSpec
from .registry import part_impl, plan_for


class Model:
    def __init__(self, plan: ModelPlan, rt: Runtime):
        plan.validate()
        self.plan = plan
        self.rt = rt
        self.embedding = part_impl("embedding", plan.embedding.kind)(plan.embedding, rt)
        self.layers = [part_impl("arrangement", ls.arrangement)(ls, rt) for ls in plan.layers]
        self.final_norm = part_impl("norm", plan.final_norm.kind)(plan.final_norm, rt)
        self.head = part_impl("head", plan.head.kind)(plan.head, rt)
        self.schedule = list(plan.schedule)
        self.graph_safe = all(p.graph_safe for p in self.all_parts())

    def all_parts(self):
        out = [self.embedding]
        for layer in self.layers:
            out.extend(layer.parts())
        out.extend([self.final_norm, self.head])
        return out

    def weight_specs(self) -> List[WeightSpec]:
        specs: List[WeightSpec] = []
        seen = set()
        for p in self.all_parts():
            for s in p.weight_specs():
                if s.name not in seen:
                    seen.add(s.name)
                    specs.append(s)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.all_parts():
            p.bind(tensors)

    def new_cache(self, max_tokens: int, max_seq_len: Optional[int] = None,
                  max_slots: Optional[int] = None, chunk_tokens: int = 1) -> CacheManager:
        kv_needs, cache_from, state_needs = [], [], []
        for call in self.schedule:
            mixer = self.layers[call.layer].mixer
            kv_needs.append(mixer.kv_need())
            cache_from.append(call.cache_from)
            state_needs.append(mixer.state_needs())
        return CacheManager(kv_needs, cache_from, state_needs, max_tokens,
                            max_seq_len or self.plan.max_positions, self.rt.dtype, self.rt.device,
                            max_slots, chunk_tokens)

    def hidden(self, step: StepInfo, cache: CacheManager, tap: Optional[list] = None) -> torch.Tensor:
        """The residual stream after the last entry of the run order, float32 [N, width].  With `tap`
        (a list) a copy of the residual stream is appended after the embedding and after every entry
        of the run order: what tells where two paths begin to differ (the reference keeps such a tap
        per layer, src/forward.rs:45-103)."""
        return self._run_layers(step, cache, tap, None)[0]

    def _run_layers(self, step: StepInfo, cache: CacheManager, tap: Optional[list], last_norm):
        """(x, h): the residual stream after the last entry of the run order and, if `last_norm` is given, that
        norm of it, which comes out of the last layer's last kernel where the arrangement hands norms on."""
        x = self.embedding.forward(step.tokens, step)
        if tap is not None:
            tap.append(x.clone())
        h = None
        for i, call in enumerate(self.schedule):
            layer = self.layers[call.layer]
            if not layer.chains:
                layer.forward(x, step, cache.stores[i])
                h = None
            else:
                nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
                if nxt is None:
                    next_norm = last_norm
                else:
                    next_norm = nxt.entry_norm() if nxt.chains else None
                h = layer.forward(x, step, cache.stores[i], h_in=h, next_norm=next_norm)
            if tap is not None:
                tap.append(x.clone())
        if last_norm is None:
            return x, None
        return x, (h if h is not None else last_norm.forward(x))

    def step_logits(self, step: StepInfo, cache: CacheManager) -> torch.Tensor:
        """float32 [N, vocab]: the logits of every row of the step (what a decoding step wants): no rows are
        picked, and the final norm is the last layer's to hand on."""
        _, h = self._run_layers(step, cache, None, self.final_norm)
        return self.head.forward(h)

    def logits(self, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """float32 [len(rows), vocab] for the given rows of the residual stream."""
        if rows.shape[0] == 0:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=x.device)
        picked = torch.empty((rows.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
        ops.gather_rows(x, rows, picked)
        return self.head.forward(self.final_norm.forward(picked))


def weight_specs_for(config: ModelConfig) -> List[WeightSpec]:
    """The tensors a model of this configuration wants (no GPU needed)."""
    return Model(plan_for(config), Runtime(torch.device("cpu"), torch.bfloat16)).weight_specs()
