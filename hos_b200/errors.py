"""Error types.  Loading and set-up report bad input through these; none of them
aborts the process.  They mirror the reference's `HosError` variants
(src/error.rs:11-27) and all derive from `ValueError`, which is what the
reference's Python binding raises (py/src/lib.rs:23-25)."""
from __future__ import annotations

from typing import List, Sequence, Tuple


class HosError(ValueError):
    """Base class of every error this library raises on bad input."""


class IoError(HosError):
    """A file could not be opened or read."""


class FormatError(HosError):
    """A container is malformed: truncated, bad header, offsets out of bounds,
    unsupported dtype (src/safetensors.rs:31-41, :119-150)."""


class MissingMetaError(HosError):
    """A required config.json key is absent or has the wrong type (src/hf.rs:173-178)."""


class UnsupportedArchError(HosError):
    """config.json names an architecture that is not registered (src/hf.rs:159-163)."""


class MissingTensorError(HosError):
    """A tensor was asked for by a name the container does not hold
    (src/safetensors.rs:193-197)."""


class SpecError(HosError):
    """A model plan is inconsistent: unknown part kind, a schedule entry that
    names a missing layer, a cache reference that points forward."""


class WeightMismatchError(HosError):
    """The checkpoint does not fit the model: one error that lists every missing
    tensor, every unexpected tensor and every tensor of the wrong shape or dtype."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, tuple, tuple]],
                 wrong_dtype: Sequence[Tuple[str, str, str]] = ()):
        self.missing: List[str] = list(missing)
        self.unexpected: List[str] = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {list(want)} found {list(got)}")
        for name, want, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} expected {want} found {got}")
        super().__init__("\n".join(lines))


class CacheError(HosError):
    """The cache cannot hold what was asked (no free slot, no free page, a
    sequence longer than its table) or a slot was misused (freed twice)."""


class KernelError(RuntimeError):
    """A CUDA kernel refused its sizes or reported a launch error.  Not a
    `HosError`: it signals a fault of the set-up, not of a model folder."""


class ExtensionMissingError(RuntimeError):
    """The compiled CUDA library is absent and could not be built.  There is no
    fallback path: nothing runs without it."""
