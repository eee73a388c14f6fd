"""Typed reading of config.json and the data that describes a model.

A model is described by data, not by a class per model: a `ModelPlan` lists,
layer by layer, which mixer, feed-forward, norms and position encoding the layer
uses (each a `PartSpec`: a kind tag, its sizes and constants, and the checkpoint
names of its tensors) and, separately, the order in which layers run
(`LayerCall` entries, which may name a layer twice or point at an earlier
call's cache).  An architecture is a function from its typed configuration to
such a plan; see `hos_b200.registry`.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..errors import FormatError, IoError, MissingMetaError, SpecError


class ConfigReader:
    """Typed access to a config.json dict.  A missing required key, or a value
    of the wrong type, raises `MissingMetaError` naming the key
    (the reference's `need_u`, src/hf.rs:173)."""

    def __init__(self, raw: Mapping[str, Any]):
        self.raw = raw

    def _get(self, key: str):
        v = self.raw.get(key)
        return None if v is None else v

    def need_int(self, key: str) -> int:
        v = self._get(key)
        if isinstance(v, bool) or not isinstance(v, int):
            raise MissingMetaError(f"missing model metadata: {key} (an integer is required)")
        return v

    def opt_int(self, key: str, default: Optional[int]) -> Optional[int]:
        v = self._get(key)
        if v is None:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            raise MissingMetaError(f"model metadata {key} must be an integer, found {v!r}")
        return v

    def opt_float(self, key: str, default: Optional[float]) -> Optional[float]:
        v = self._get(key)
        if v is None:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise MissingMetaError(f"model metadata {key} must be a number, found {v!r}")
        return float(v)

    def opt_bool(self, key: str, default: bool) -> bool:
        v = self._get(key)
        if v is None:
            return default
        if not isinstance(v, bool):
            raise MissingMetaError(f"model metadata {key} must be true or false, found {v!r}")
        return v

    def token_ids(self, key: str) -> Tuple[int, ...]:
        """A token id given as a scalar or as a list (src/tokenizer.rs:711-720
        takes the scalar or the first of the list; all of a list are kept here
        so that each of them stops a sequence)."""
        v = self._get(key)
        if v is None:
            return ()
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, list) and all(isinstance(t, int) and not isinstance(t, bool) for t in v):
            return tuple(v)
        raise MissingMetaError(f"model metadata {key} must be an integer or a list of integers")


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "rb") as f:
            data = f.read()
    except OSError as e:
        raise IoError(f"io error: {path}: {e.strerror or e}") from e
    try:
        raw = json.loads(data)
    except ValueError as e:
        raise FormatError(f"malformed file: {path}: {e}") from e
    if not isinstance(raw, dict):
        raise FormatError(f"malformed file: {path}: top level is not an object")
    return raw


# ---- the description of a model ---------------------------------------------------------

@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: `kind` selects the implementation in the registry,
    `params` holds every size and constant it needs, `weights` maps the part's
    own role names to tensor names in the checkpoint."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    weights: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (how norms, mixer, feed-forward and the residual
    stream are wired) and the parts it wires.  `norms` is keyed by the role names
    the arrangement defines."""
    arrangement: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.  `layer` indexes `ModelPlan.layers` (the same
    index may appear in several calls: shared weights, separate cache).
    `cache_from`, if set, is the index of an EARLIER call whose cache this call's
    mixer reads instead of keeping one of its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelPlan:
    width: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[LayerCall]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.layers:
            raise SpecError("arch spec error: a model needs at least one layer")
        for i, call in enumerate(self.schedule):
            if not (0 <= call.layer < len(self.layers)):
                raise SpecError(f"arch spec error: schedule entry {i} names layer {call.layer}, "
                                f"but there are {len(self.layers)} layers")
            if call.cache_from is not None:
                if not (0 <= call.cache_from < i):
                    raise SpecError(f"arch spec error: schedule entry {i} reads the cache of entry "
                                    f"{call.cache_from}, which does not run before it")
                if self.schedule[call.cache_from].cache_from is not None:
                    raise SpecError(f"arch spec error: schedule entry {i} reads the cache of entry "
                                    f"{call.cache_from}, which has no cache of its own")


class ModelConfig:
    """Base of the typed configurations.  A subclass is a dataclass whose fields
    are the architecture's config.json keys, with `from_dict` applying the
    defaults and checks, and `to_dict` writing a config.json back."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError
