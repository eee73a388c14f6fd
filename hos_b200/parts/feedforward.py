"""Gated feed-forward: down(act(gate(h)) * up(h)) (src/forward.rs:384-398), with the
activation as a parameter ("gelu_tanh" is Gemma's GeGLU, src/forward.rs:186-189;
"silu" is the reference's other branch, :393).  Gate and up are one product whose
epilogue applies the activation and the product, so the 2*inner-wide intermediate
is never written."""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import ops
from ..errors import SpecError
from ..registry import register_part
from . import linear
from .base import FeedForward, StepInfo, WeightSpec


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        act = spec.params.get("activation", "gelu_tanh")
        if act not in ops.ACTIVATIONS:
            raise SpecError(f"arch spec error: unknown activation {act!r}")
        self.act = ops.ACTIVATIONS[act]
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["gate"], (self.inner, self.width), "matrix", 0.02),
                WeightSpec(w["up"], (self.inner, self.width), "matrix", 0.02),
                WeightSpec(w["down"], (self.width, self.inner), "matrix", 0.02)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        g, u = self._matrix(tensors[w["gate"]]), self._matrix(tensors[w["up"]])
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()    # gate rows, then up rows
        self.w_down = self._matrix(tensors[w["down"]])

    def forward(self, h: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        z = linear.matmul(h, self.w_gate_up, epilogue=ops.EPI_GATED, act=self.act)
        return linear.matmul(z, self.w_down)

    def forward_partial(self, h: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        """As forward, but the down projection may come back as float32 partial sums
        [parts, N, width] for a consumer that adds them."""
        z = linear.matmul(h, self.w_gate_up, epilogue=ops.EPI_GATED, act=self.act)
        return linear.matmul_or_partials(z, self.w_down)


register_part("feed_forward", "gated_mlp", GatedMLP)
