"""Typed reading of a model folder's config.json.

Every architecture declares a frozen dataclass whose fields are read from the
architecture's own config.json keys by :class:`KeyReader`; an error always names
the key.  The reference keeps an untyped ``Vec<i64>`` of sizes in its bundle
manifest (src/convert.rs:1220-1222, read back in src/minimax.rs:44-49); here the
sizes stay named from the file to the kernels.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type or an impossible value."""


_MISSING = object()


class KeyReader:
    """Reads keys of one config.json mapping and remembers which were used."""

    def __init__(self, raw: Mapping[str, Any], where: str = "config.json"):
        self.raw = raw
        self.where = where
        self.used: set[str] = set()

    def _get(self, names: Sequence[str], default: Any) -> tuple[str, Any]:
        for name in names:
            node: Any = self.raw
            ok = True
            for piece in name.split("."):
                if isinstance(node, Mapping) and piece in node and node[piece] is not None:
                    node = node[piece]
                else:
                    ok = False
                    break
            if ok:
                self.used.add(name.split(".")[0])
                return name, node
        if default is _MISSING:
            raise ConfigError(f"{self.where}: required key {' | '.join(names)!r} is missing")
        return names[0], default

    def integer(self, *names: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        name, value = self._get(names, default)
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value == int(value):
                value = int(value)
            else:
                raise ConfigError(f"{self.where}: key {name!r} must be an integer, found {value!r}")
        if minimum is not None and value < minimum:
            raise ConfigError(f"{self.where}: key {name!r} must be >= {minimum}, found {value}")
        return value

    def real(self, *names: str, default: Any = _MISSING, positive: bool = False) -> float:
        name, value = self._get(names, default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{self.where}: key {name!r} must be a number, found {value!r}")
        value = float(value)
        if positive and not value > 0.0:
            raise ConfigError(f"{self.where}: key {name!r} must be > 0, found {value}")
        return value

    def boolean(self, *names: str, default: Any = _MISSING) -> bool:
        name, value = self._get(names, default)
        if not isinstance(value, bool):
            raise ConfigError(f"{self.where}: key {name!r} must be true or false, found {value!r}")
        return value

    def text(self, *names: str, default: Any = _MISSING) -> str:
        name, value = self._get(names, default)
        if not isinstance(value, str):
            raise ConfigError(f"{self.where}: key {name!r} must be a string, found {value!r}")
        return value

    def present(self, name: str) -> bool:
        """Whether ``name`` (dotted for a nested key) holds a value other than null."""
        node: Any = self.raw
        for piece in name.split("."):
            if not isinstance(node, Mapping) or piece not in node or node[piece] is None:
                return False
            node = node[piece]
        return True

    def value(self, name: str) -> Any:
        """The raw value under ``name`` (dotted for a nested key), or None."""
        node: Any = self.raw
        for piece in name.split("."):
            if not isinstance(node, Mapping) or piece not in node or node[piece] is None:
                return None
            node = node[piece]
        return node

    def refuse_unless(self, name: str, allowed, meaning: str) -> None:
        """A key that would change the arithmetic: if it is present its value must satisfy ``allowed``
        (a predicate), else the configuration is refused with the key's name and ``meaning``."""
        found = self.value(name)
        if found is None:
            return
        try:
            ok = bool(allowed(found))
        except (TypeError, ValueError):
            ok = False
        if not ok:
            raise ConfigError(f"{self.where}: key {name!r} is {found!r}: {meaning}")
        self.used.add(name.split(".")[0])

    def integer_list(self, *names: str, default: Any = _MISSING) -> tuple[int, ...]:
        """An int or a list of ints (``eos_token_id`` is either, src/convert.rs:375-381)."""
        name, value = self._get(names, default)
        if isinstance(value, bool):
            raise ConfigError(f"{self.where}: key {name!r} must be an integer or a list of integers")
        if isinstance(value, int):
            return (value,)
        if isinstance(value, (list, tuple)) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return tuple(value)
        raise ConfigError(f"{self.where}: key {name!r} must be an integer or a list of integers, found {value!r}")


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration offers to the rest of the library."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    eos_token_id: tuple[int, ...] = field(default=())

    def to_json_dict(self) -> dict[str, Any]:  # pragma: no cover - overridden
        raise NotImplementedError


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json in this model folder")
    with open(path, "r", encoding="utf-8") as handle:
        try:
            raw = json.load(handle)
        except json.JSONDecodeError as err:
            raise ConfigError(f"{path}: not valid JSON ({err})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw
