"""Random weights from a configuration and a seed.

`RandomSource` is a tensor source (names / info / read, like a safetensors folder)
that makes every tensor the model asks for on the fly: matrices and tables
~ N(0, 0.02), norm vectors ~ N(0, 0.1) (applied as 1 + w by Gemma's norms), stored
as bfloat16.  Each tensor has its own generator seeded from (seed, name), so the
values do not depend on the order of reading.  `write_model_folder` writes such a
model as config.json + model.safetensors.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, List, Sequence, Tuple

import torch

from ..config.base import ModelConfig
from ..errors import MissingTensorError
from ..parts.base import WeightSpec
from .safetensors import SINGLE_FILE, write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


class RandomSource:
    def __init__(self, specs: Sequence[WeightSpec], seed: int, device: str = "cpu",
                 dtype: torch.dtype = torch.bfloat16):
        # a tensor with a fallback (a tied head) is not generated: the fallback is used
        self._specs: Dict[str, WeightSpec] = {s.name: s for s in specs if s.fallback is None}
        self.seed = seed
        self.device = torch.device(device)
        self.dtype = dtype

    def names(self) -> List[str]:
        return list(self._specs)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        s = self._specs.get(name)
        if s is None:
            raise MissingTensorError(f"missing tensor '{name}'")
        return self.dtype, tuple(s.shape)

    def read(self, name: str) -> torch.Tensor:
        s = self._specs.get(name)
        if s is None:
            raise MissingTensorError(f"missing tensor '{name}'")
        g = torch.Generator(device=self.device)
        g.manual_seed(_tensor_seed(self.seed, name))
        t = torch.randn(tuple(s.shape), generator=g, dtype=torch.float32, device=self.device)
        return (t * s.init_std).to(self.dtype)

    def close(self) -> None:
        pass


def write_model_folder(config: ModelConfig, seed: int, model_dir: str) -> None:
    """config.json and model.safetensors of a randomly initialised model."""
    from ..model import weight_specs_for
    os.makedirs(model_dir, exist_ok=True)
    specs = weight_specs_for(config)
    src = RandomSource(specs, seed)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)
    write_safetensors(os.path.join(model_dir, SINGLE_FILE),
                      ((name, src.read(name)) for name in src.names()),
                      metadata={"format": "pt", "seed": str(seed)})
