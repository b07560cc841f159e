"""One registry from the architecture's name (``architectures[0]`` of config.json) to its model.

The reference keeps ``model_type -> (architectures, module, class)`` and checks both
(nanovllm/models/registry.py:36-149).  Here the key is the architecture name; the entry
gives the configuration class, the function that turns a configuration into a
:class:`~nanohybrid_vlm_b200.parts.spec.ModelSpec` (layers as data) and the allowed
``model_type`` values.  Everything else in the engine works from the spec.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    model_types: tuple[str, ...]
    parse_config: Callable[[dict], ModelConfig]
    build_spec: Callable[[ModelConfig], "ModelSpec"]  # noqa: F821


class ArchitectureRegistry:
    def __init__(self):
        self._entries: dict[str, ArchitectureEntry] = {}

    def register(self, name: str, *, model_types, parse_config, build_spec, replace: bool = False) -> None:
        if not name:
            raise ValueError("an architecture needs a name")
        if name in self._entries and not replace:
            raise ValueError(f"architecture {name!r} is already registered")
        if not callable(parse_config) or not callable(build_spec):
            raise TypeError(f"architecture {name!r}: parse_config and build_spec must be callable")
        self._entries[name] = ArchitectureEntry(name, tuple(model_types), parse_config, build_spec)

    def unregister(self, name: str) -> None:
        self._entries.pop(name, None)

    def names(self) -> list[str]:
        return sorted(self._entries)

    def resolve(self, raw_config: dict) -> ArchitectureEntry:
        archs = raw_config.get("architectures") or ()
        if isinstance(archs, str):
            archs = (archs,)
        if not archs:
            raise ConfigError("config.json: key 'architectures' is missing or empty; "
                              f"supported architectures: {self.names()}")
        known = [a for a in archs if a in self._entries]
        if not known:
            raise ConfigError(f"unsupported architectures {tuple(archs)!r}; supported: {self.names()}")
        entry = self._entries[known[0]]
        model_type = raw_config.get("model_type")
        if model_type is not None and entry.model_types and model_type not in entry.model_types:
            raise ConfigError(f"architecture {entry.name!r} does not go with model_type {model_type!r} "
                              f"(expected one of {entry.model_types})")
        return entry


ARCHITECTURES = ArchitectureRegistry()


def register_architecture(name: str, *, model_types=(), parse_config, build_spec, replace=False) -> None:
    ARCHITECTURES.register(name, model_types=model_types, parse_config=parse_config,
                           build_spec=build_spec, replace=replace)


def load_model_config(model_dir: str) -> tuple[ArchitectureEntry, ModelConfig]:
    """Read ``model_dir/config.json``, pick the architecture, parse its typed configuration."""
    from .. import models  # noqa: F401  (registers the built-in architecture)
    raw = read_config_json(model_dir)
    entry = ARCHITECTURES.resolve(raw)
    return entry, entry.parse_config(raw)
