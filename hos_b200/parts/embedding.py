"""Token embedding scaled by a constant: x = E[token] * scale, the product taken in
32-bit (src/forward.rs:271-281; Gemma's scale is sqrt(width), src/model.rs:899),
and the head: logits = soft-cap(E_head . h) in float32 (src/forward.rs:429-435),
where E_head is `lm_head.weight` if the checkpoint has it and the embedding table
otherwise (src/model.rs:879-883)."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..registry import register_part
from . import linear
from .base import Part, StepInfo, WeightSpec


class ScaledEmbedding(Part):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["table"], (self.vocab, self.width), "table", 0.02)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = self._matrix(tensors[self.spec.weights["table"]])

    def forward(self, tokens: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        x = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        ops.embed(tokens, self.table, self.scale, x)
        return x


class LinearHead(Part):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.softcap = float(spec.params.get("softcap") or 0.0)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["table"], (self.vocab, self.width), "table", 0.02,
                           fallback=w.get("tied_to"))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = self._matrix(tensors[self.spec.weights["table"]])

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        epi = ops.EPI_SOFTCAP if self.softcap > 0.0 else ops.EPI_NONE
        return linear.matmul(h, self.table, out_dtype=torch.float32, epilogue=epi, cap=self.softcap)


register_part("embedding", "scaled_embedding", ScaledEmbedding)
register_part("head", "linear_head", LinearHead)
