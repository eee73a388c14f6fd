"""Rotary position encoding: for pair i of a head, angle = position / theta^(2i/rotary_dim);
the pair is rotated by it (src/forward.rs:203-222).  `style` chooses the pairing:
"rotate_half" pairs (i, i + rotary_dim/2) (the reference's `neox`, used by Gemma,
src/model.rs:80-82), "interleaved" pairs (2i, 2i+1).  Dimensions beyond
rotary_dim pass unchanged.  The inverse frequencies are computed once, in 32-bit;
the kernel multiplies them by the position and takes sincosf, all in 32-bit.

A position encoding is used by a mixer: the mixer asks it for `kernel_args()` and
hands them to the fused rotate-and-store kernel."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import SpecError
from ..registry import register_part
from .base import Part


_shared = {}


class Rotary(Part):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        style = spec.params.get("style", "rotate_half")
        if style not in ops.ROPE_STYLES:
            raise SpecError(f"arch spec error: unknown rotary pairing {style!r}")
        if self.rotary_dim % 2 != 0 or self.rotary_dim <= 0:
            raise SpecError(f"arch spec error: rotary_dim {self.rotary_dim} must be positive and even")
        self.style = ops.ROPE_STYLES[style]
        key = (str(rt.device), self.theta, self.rotary_dim)
        if key not in _shared:          # layers with the same frequencies share one tensor (and what is derived from it)
            half = self.rotary_dim // 2
            i = torch.arange(half, dtype=torch.float32)
            exponent = 2.0 * i / float(self.rotary_dim)
            _shared[key] = (1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)) \
                .to(rt.device).contiguous()
        self.inv_freq = _shared[key]

    def kernel_args(self):
        """(inverse frequencies [rotary_dim/2] float32 on the device, rotary_dim, style code)."""
        return self.inv_freq, self.rotary_dim, self.style


class NoPosition(Part):
    """No position encoding: q and k are used as projected."""
    graph_safe = True


    def kernel_args(self):
        return None, 0, 0


register_part("position", "rotary", Rotary)
register_part("position", "none", NoPosition)
