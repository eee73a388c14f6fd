"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * (w + add_one)  (src/forward.rs:166-174;
`add_one` is Gemma's (1 + w) convention, src/hf.rs:101-107).  Statistics in 32-bit."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..registry import register_part
from .base import Norm, WeightSpec


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.add_one = bool(spec.params.get("add_one", False))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", 0.1)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = self._vector32(tensors[self.spec.weights["weight"]])

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, self.add_one, out)
        return out

    accepts_partials = True      # y may be [parts, N, width] float32 partial sums

    def add_to(self, y: torch.Tensor, x: torch.Tensor, then: Optional[Norm] = None):
        """x += self(y); with another RMSNorm as `then`, its output comes from the same kernel."""
        if then is None:
            ops.norm_add_norm(y, self.weight, self.eps, self.add_one, x)
            return None
        if isinstance(then, RMSNorm):
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            ops.norm_add_norm(y, self.weight, self.eps, self.add_one, x,
                              then.weight, then.eps, then.add_one, h)
            return h
        ops.norm_add_norm(y, self.weight, self.eps, self.add_one, x)
        return then.forward(x)


register_part("norm", "rmsnorm", RMSNorm)
