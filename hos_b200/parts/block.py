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

    # An arrangement whose first act is a norm of x may say so (`entry_norm`) and set
    # `chains = True`: the model then hands it `h_in`, that norm's output already computed by
    # the layer before, and `next_norm`, the entry norm of the layer after, whose output it
    # returns (computed in the kernel that makes its last residual sum).
    chains = False

    def entry_norm(self):
        return None

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        raise NotImplementedError

    @staticmethod
    def _branch(part, takes_partials: bool, *args):
        """Run a mixer or feed-forward; let it hand back partial sums if it can and its consumer adds them."""
        if takes_partials and hasattr(part, "forward_partial"):
            return part.forward_partial(*args)
        return part.forward(*args)


class SandwichLayer(Layer):
    norm_roles = ("pre_mixer", "post_mixer", "pre_ffn", "post_ffn")

    chains = True

    def entry_norm(self):
        return self.norms["pre_mixer"]

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        n = self.norms
        h = h_in if h_in is not None else n["pre_mixer"].forward(x)
        a = self._branch(self.mixer, getattr(n["post_mixer"], "accepts_partials", False), h, step, store)
        h = n["post_mixer"].add_to(a, x, then=n["pre_ffn"])     # x += post(a); h = pre_ffn(x)
        f = self._branch(self.feed_forward, getattr(n["post_ffn"], "accepts_partials", False), h, step)
        return n["post_ffn"].add_to(f, x, then=next_norm)       # x += post(f); next layer's entry norm


class PreNormLayer(Layer):
    norm_roles = ("pre_mixer", "pre_ffn")

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        n = self.norms
        a = self.mixer.forward(n["pre_mixer"].forward(x), step, store)
        ops.residual_add(a, x)
        f = self.feed_forward.forward(n["pre_ffn"].forward(x), step)
        ops.residual_add(f, x)


register_part("arrangement", "sandwich", SandwichLayer)
register_part("arrangement", "prenorm", PreNormLayer)
