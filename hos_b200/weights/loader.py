"""From a tensor source to the tensors the model's parts asked for.

The parts' wishes (`WeightSpec`: name, shape, role) are checked against what the
source holds before anything is copied; every problem is gathered into ONE
`WeightMismatchError` that lists the missing tensors, the unexpected ones and the
ones of the wrong shape.  (The reference reports the first missing tensor,
src/safetensors.rs:193-197, and does not check shapes, src/model.rs:210-213.)

Dtypes: a tensor stored as bfloat16 stays bfloat16, one stored as float16 becomes
bfloat16, one stored in 32-bit stays 32-bit, integer tables become int32.  What
the compute path then needs (float32 copies in the 32-bit path, fused matrices) is
made by the parts in `bind`.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ..errors import WeightMismatchError
from ..parts.base import WeightSpec


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    if stored in (torch.bfloat16, torch.float16):
        return torch.bfloat16
    if stored == torch.float32:
        return torch.float32
    if stored in (torch.int32, torch.int64):
        return torch.int32
    raise ValueError(f"no rule for stored dtype {stored}")


def check_against(specs: Sequence[WeightSpec], source) -> Dict[str, str]:
    """Returns {wanted name -> name to read}; raises WeightMismatchError listing everything wrong."""
    have = set(source.names())
    missing: List[str] = []
    wrong_shape = []
    resolve: Dict[str, str] = {}
    used = set()
    for s in specs:
        name = s.name
        if name not in have:
            if s.fallback is not None and s.fallback in have:
                name = s.fallback
            else:
                missing.append(s.name)
                continue
        _, shape = source.info(name)
        if tuple(shape) != tuple(s.shape):
            wrong_shape.append((name, tuple(s.shape), tuple(shape)))
        resolve[s.name] = name
        used.add(name)
    unexpected = sorted(have - used)
    if missing or unexpected or wrong_shape:
        raise WeightMismatchError(sorted(missing), unexpected, wrong_shape)
    return resolve


def load_tensors(specs: Sequence[WeightSpec], source, device: torch.device) -> Dict[str, torch.Tensor]:
    """All wanted tensors on `device`, keyed by the wanted name (a tied tensor is one
    device tensor under both names)."""
    resolve = check_against(specs, source)
    by_read: Dict[str, torch.Tensor] = {}
    out: Dict[str, torch.Tensor] = {}
    for want, read in resolve.items():
        t = by_read.get(read)
        if t is None:
            raw = source.read(read)
            t = raw.to(device=device, dtype=kept_dtype(raw.dtype)).contiguous()
            by_read[read] = t
        out[want] = t
    return out
