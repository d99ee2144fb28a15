"""One registry from an architecture's name to its configuration class and plan.

The reference dispatches with a ``match`` on the bundle's arch string
(src/main.rs:710-750) and maps a checkpoint's ``model_type`` to an arch by longest
prefix (src/convert.rs:392-445); an unknown name fails with the list of known
ones (src/main.rs:749).  Here the name is ``config.json["architectures"][0]``,
with ``model_type`` prefixes as the fallback.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .base import ConfigError, ModelConfig, read_config_json
from .plan import ModelPlan


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any], str], ModelConfig]
    plan: Callable[[ModelConfig], ModelPlan]
    model_type_prefixes: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def _load_builtin() -> None:
    from .. import models  # noqa: F401  (registers the built-in architecture on import)


def architecture_for(raw: Mapping[str, Any], where: str = "config.json") -> Architecture:
    """Choose the architecture a config.json names."""
    _load_builtin()
    names = raw.get("architectures")
    if isinstance(names, (list, tuple)) and names:
        name = names[0]
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    else:
        name = None
    model_type = raw.get("model_type")
    if isinstance(model_type, str):
        best: Architecture | None = None
        best_len = -1
        for arch in _ARCHITECTURES.values():
            for prefix in arch.model_type_prefixes:
                if model_type.startswith(prefix) and len(prefix) > best_len:
                    best, best_len = arch, len(prefix)
        if best is not None:
            return best
    raise ConfigError(
        f"{where}: architecture {name!r} (model_type {model_type!r}) is not registered; "
        f"registered: {', '.join(sorted(_ARCHITECTURES)) or 'none'}")


def load_config(model_dir: str) -> tuple[Architecture, ModelConfig]:
    raw = read_config_json(model_dir)
    arch = architecture_for(raw, where=f"{model_dir}/config.json")
    return arch, arch.config_from_dict(raw, f"{model_dir}/config.json")
