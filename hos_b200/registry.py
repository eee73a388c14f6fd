"""The registries: architecture name -> (typed configuration, plan function), and
part kind -> implementation, one table per category of part.

The reference selects a model family from a string (`Arch::detect`,
src/model.rs:13-44; HF `model_type`, src/hf.rs:151-164) and answers an unknown
one with an error that lists what it supports (src/hf.rs:159-163).  Here the
tables are open: a new mixer, feed-forward, norm, position encoding, block
arrangement or whole architecture is added by calling `register_*` from any
module, without a change to this package.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Tuple, Type

from .config.base import ModelConfig, ModelPlan
from .errors import SpecError, UnsupportedArchError

PART_CATEGORIES = ("mixer", "feed_forward", "norm", "position", "arrangement", "embedding", "head")

_architectures: Dict[str, Tuple[Type[ModelConfig], Callable[[Any], ModelPlan]]] = {}
_model_types: Dict[str, str] = {}
_parts: Dict[str, Dict[str, Any]] = {c: {} for c in PART_CATEGORIES}


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          plan_fn: Callable[[Any], ModelPlan], model_type: str = "") -> None:
    """`name` is what config.json lists under `architectures`; `model_type`, if
    given, is accepted as a fallback when that list is absent."""
    _architectures[name] = (config_cls, plan_fn)
    if model_type:
        _model_types[model_type] = name


def registered_architectures():
    _load_builtins()
    return sorted(_architectures)


_builtins_loaded = False


def _load_builtins() -> None:
    """The package's own parts and architectures register themselves when their modules are imported; a look-up
    that finds nothing imports them once, so that the tables do not depend on what the caller imported before."""
    global _builtins_loaded
    if _builtins_loaded:
        return
    _builtins_loaded = True
    from . import models, parts  # noqa: F401


def resolve_architecture(raw: Mapping[str, Any]) -> str:
    _load_builtins()
    archs = raw.get("architectures")
    if isinstance(archs, list):
        for a in archs:
            if a in _architectures:
                return a
    mt = raw.get("model_type")
    if isinstance(mt, str) and mt in _model_types:
        return _model_types[mt]
    named = archs if archs else mt
    raise UnsupportedArchError(
        f"unsupported architecture: {named!r} - registered: {', '.join(registered_architectures())}")


def config_from_dict(raw: Mapping[str, Any]) -> ModelConfig:
    name = resolve_architecture(raw)
    return _architectures[name][0].from_dict(raw)


def plan_for(config: ModelConfig) -> ModelPlan:
    entry = _architectures.get(config.architecture)
    if entry is None:
        _load_builtins()
        entry = _architectures.get(config.architecture)
    if entry is None:
        raise UnsupportedArchError(
            f"unsupported architecture: {config.architecture!r} - registered: "
            f"{', '.join(registered_architectures())}")
    plan = entry[1](config)
    plan.validate()
    return plan


def register_part(category: str, kind: str, impl: Any) -> None:
    if category not in _parts:
        raise SpecError(f"arch spec error: unknown part category {category!r}")
    _parts[category][kind] = impl


def part_impl(category: str, kind: str) -> Any:
    table = _parts.get(category)
    if table is None:
        raise SpecError(f"arch spec error: unknown part category {category!r}")
    impl = table.get(kind)
    if impl is None:
        _load_builtins()
        impl = table.get(kind)
    if impl is None:
        raise SpecError(f"arch spec error: no {category} of kind {kind!r} is registered "
                        f"(known: {', '.join(sorted(table)) or 'none'})")
    return impl
