"""Arrangements: how one layer wires its norms, its mixer, its feed-forward and the
residual stream.  The residual stream x is float32 and is updated in place; the
sums are 32-bit.

"sandwich" (Gemma-2, src/forward.rs:291-414): norms before AND after each branch,
    x += post_mixer(mixer(pre_mixer(x)));  x += post_ffn(ffn(pre_ffn(x)))
"prenorm" (the reference's other families): a norm before each branch only,
    x += mixer(pre_mixer(x));  x += ffn(pre_ffn(x))
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.base import LayerSpec
from ..errors import SpecError
from ..registry import part_impl, register_part
from .base import CallStore, Runtime, StepInfo


class Layer:
    """Base of the arrangements: builds the layer's parts from the registry."""
    norm_roles = ()

    def __init__(self, spec: LayerSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.mixer = part_impl("mixer", spec.mixer.kind)(spec.mixer, rt)
        self.feed_forward = part_impl("feed_forward", spec.feed_forward.kind)(spec.feed_forward, rt)
        missing = [r for r in self.norm_roles if r not in spec.norms]
        if missing:
            raise SpecError(f"arch spec error: arrangement {spec.arrangement!r} needs norms {missing}")
        self.norms: Dict[str, object] = {
            role: part_impl("norm", ps.kind)(ps, rt) for role, ps in spec.norms.items()}

    def parts(self):
        return [self.mixer, self.feed_forward] + list(self.norms.values())

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore) -> None:
        raise NotImplementedError


class SandwichLayer(Layer):
    norm_roles = ("pre_mixer", "post_mixer", "pre_ffn", "post_ffn")

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore) -> None:
        n = self.norms
        h = n["pre_mixer"].forward(x)
        a = self.mixer.forward(h, step, store)
        h = n["post_mixer"].add_to(a, x, then=n["pre_ffn"])     # x += post(a); h = pre_ffn(x)
        f = self.feed_forward.forward(h, step)
        n["post_ffn"].add_to(f, x)


class PreNormLayer(Layer):
    norm_roles = ("pre_mixer", "pre_ffn")

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore) -> None:
        n = self.norms
        a = self.mixer.forward(n["pre_mixer"].forward(x), step, store)
        ops.residual_add(a, x)
        f = self.feed_forward.forward(n["pre_ffn"].forward(x), step)
        ops.residual_add(f, x)


register_part("arrangement", "sandwich", SandwichLayer)
register_part("arrangement", "prenorm", PreNormLayer)
