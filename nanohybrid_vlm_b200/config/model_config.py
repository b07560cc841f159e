"""Typed model configuration, read from the architecture's own ``config.json`` keys.

A model folder's ``config.json`` is parsed with the standard ``json`` module only.
Each architecture owns a subclass of :class:`ModelConfig` that names its keys, their
defaults and their checks; nothing in the engine hard-codes a size.  The reference
reads the same keys through ``transformers.AutoConfig`` (nanovllm/config.py:318-323)
and its model code picks them at nanovllm/models/qwen3.py:128-144.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any

import torch


class ConfigError(ValueError):
    """A config.json that cannot be used: a missing key, a bad value, an unknown architecture."""


_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
}


def parse_dtype(name: Any) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    key = str(name).replace("torch.", "")
    if key not in _DTYPES:
        raise ConfigError(f"unknown dtype {name!r}; known: {sorted(_DTYPES)}")
    return _DTYPES[key]


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir!r} has no config.json")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return raw


class _Required:
    pass


REQUIRED = _Required()


def take(raw: dict, key: str, kind, default: Any = REQUIRED, *, where: str = "config.json"):
    """Fetch ``raw[key]`` and check its type.  ``kind`` is int, float, bool or str."""
    if key not in raw or raw[key] is None:
        if default is REQUIRED:
            raise ConfigError(f"{where}: required key {key!r} is missing")
        return default
    v = raw[key]
    if kind is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if kind is int and isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"{where}: key {key!r} must be {kind.__name__}, got {v!r}")
    return v


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration carries.  Subclasses add their own keys."""
    architecture: str
    model_type: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    dtype: torch.dtype
    eos_token_id: int | None

    def to_json_dict(self) -> dict:
        """The config.json that parses back to this object (used by the random-weights mode)."""
        raise NotImplementedError

    def describe(self) -> dict:
        return {f.name: getattr(self, f.name) for f in fields(self)}
