"""The description of a model as data: which parts each layer is made of, with what sizes
and constants, and in which order the layers run.

A :class:`PartSpec` names a registered part (``kind``) and carries its parameters.  A
:class:`LayerSpec` picks a mixer, a feed-forward, their norms and the arrangement (block)
for one layer, so different layers of one model may use different parts.  The order of
execution is a list of :class:`LayerRun`: it may name a layer twice (shared weights, each
run with a cache of its own) or let a run read the cache that an earlier run wrote.
Nothing here knows a model's name; an architecture is a function from its configuration
to a :class:`ModelSpec`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    kind: str
    items: tuple[tuple[str, Any], ...] = ()

    @property
    def params(self) -> dict:
        return dict(self.items)

    def __getitem__(self, key: str):
        for k, v in self.items:
            if k == key:
                return v
        raise KeyError(f"part {self.kind!r} has no parameter {key!r}")

    def get(self, key: str, default=None):
        for k, v in self.items:
            if k == key:
                return v
        return default


def part(kind: str, **params) -> PartSpec:
    return PartSpec(kind, tuple(sorted(params.items())))


@dataclass(frozen=True)
class Source:
    """A checkpoint tensor that fills rows [row, row + rows) of a parameter."""
    name: str
    row: int
    rows: int


@dataclass(frozen=True)
class ParamDecl:
    """One tensor that a part owns.

    ``storage``: "model" follows the engine's dtype (bfloat16 or float32); "float32" stays
    32-bit whatever the engine's dtype; "int32" is an integer table.
    ``init``: how the random-weights mode fills it: "normal" N(0, 0.02), "norm" 1 + N(0, 0.01),
    "zeros".
    ``sources``: checkpoint tensors (local names) stacked along dim 0; empty means one tensor
    of the parameter's own name.
    """
    name: str
    shape: tuple[int, ...]
    init: str = "normal"
    storage: str = "model"
    sources: tuple[Source, ...] = ()

    def resolved_sources(self) -> tuple[Source, ...]:
        return self.sources or (Source(self.name, 0, self.shape[0]),)


@dataclass(frozen=True)
class PartUse:
    """A part as used at one place of the model: its spec and the checkpoint-name prefix of its tensors."""
    spec: PartSpec
    prefix: str


@dataclass(frozen=True)
class LayerSpec:
    block: PartSpec          # the arrangement of the parts below (kind registered in BLOCKS)
    mixer: PartUse
    mixer_norm: PartUse
    ffn: PartUse
    ffn_norm: PartUse


@dataclass(frozen=True)
class LayerRun:
    """One entry of the execution order: run layer ``layer``; ``cache_from`` is the index (in the
    order list) of an earlier run whose cache this run reads instead of writing its own."""
    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartUse
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerRun, ...]
    final_norm: PartUse
    head: PartUse
    ignored_checkpoint_tensors: tuple[str, ...] = field(default=())
    # position encodings that act on the embedded tokens or own tensors (kind registered in POSITIONS), with
    # the prefix of their tensors; one that a mixer names by an equal spec is the same object
    positions: tuple[PartUse, ...] = field(default=())

    def validate(self) -> None:
        if not self.layers or not self.order:
            raise ValueError("a model needs at least one layer and one run")
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run {i} names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < i:
                    raise ValueError(f"run {i} reads the cache of run {run.cache_from}, which is not an earlier run")
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"run {i} reads the cache of run {run.cache_from}, which owns none")
