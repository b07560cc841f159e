"""The description of a model as data: which parts each layer is made of, with what sizes
and constants, and in which order the layers run.

A :class:`PartSpec` names a registered part (``kind``) and carries its parameters.  A
:class:`LayerSpec` picks the arrangement (block) of one layer and, under the names that
this block kind reads, the parts it arranges (for the pre-norm block a mixer, a
feed-forward and their two norms; another block kind may name four norms, no feed-forward,
or anything else it declares), so different layers of one model may use different parts.  The order of
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
    """A checkpoint tensor that fills the slice [row, row + rows) along dimension ``dim`` of a parameter.

    ``transpose``: the checkpoint stores the tensor with its last two dimensions exchanged ([in, out] files).
    ``squeeze``: the checkpoint tensor lacks dimension ``dim`` altogether (``rows`` must be 1): one expert's
    matrix filling entry e of a stacked parameter is ``Source(name, e, 1, squeeze=True)``."""
    name: str
    row: int
    rows: int
    dim: int = 0
    transpose: bool = False
    squeeze: bool = False

    def slice_shape(self, param_shape: tuple[int, ...]) -> tuple[int, ...]:
        """Shape of the part of the parameter that this source fills."""
        shape = list(param_shape)
        shape[self.dim] = self.rows
        return tuple(shape)

    def checkpoint_shape(self, param_shape: tuple[int, ...]) -> tuple[int, ...]:
        """Shape of the tensor as the checkpoint stores it."""
        shape = list(self.slice_shape(param_shape))
        if self.squeeze:
            if self.rows != 1:
                raise ValueError(f"source {self.name!r}: squeeze needs rows == 1")
            del shape[self.dim]
        if self.transpose:
            shape[-1], shape[-2] = shape[-2], shape[-1]
        return tuple(shape)

    def to_slice(self, tensor, param_shape: tuple[int, ...]):
        """The checkpoint tensor brought into the slice's layout, or None if its shape does not fit."""
        if tuple(tensor.shape) != self.checkpoint_shape(param_shape):
            return None
        if self.transpose:
            tensor = tensor.transpose(-1, -2)
        if self.squeeze:
            tensor = tensor.unsqueeze(self.dim)
        return tensor


@dataclass(frozen=True)
class ParamDecl:
    """One tensor that a part owns.

    ``storage``: "model" follows the engine's dtype (bfloat16 or float32); "float32" stays
    32-bit whatever the engine's dtype; "int32" is an integer table.
    ``init``: how the random-weights mode fills it: "normal" N(0, 0.02), "norm" 1 + N(0, 0.01),
    "zeros_noise" N(0, 0.01), "zeros", or a kind added with ``weights.random_init.register_init``.
    ``sources``: checkpoint tensors (local names), each filling a slice of the parameter (rows of a
    packed matrix, columns, an entry of a stack; see :class:`Source`); empty means one tensor of
    the parameter's own name and shape.
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


@dataclass(frozen=True, init=False)
class LayerSpec:
    """``block``: the arrangement (kind registered in BLOCKS).  ``parts``: the uses it arranges, under the names
    that the block kind declares in its ``SLOTS`` (name -> registry of that part).  Written
    ``LayerSpec(block, mixer=..., mixer_norm=..., ffn=..., ffn_norm=...)`` for the pre-norm block, or with
    whatever names another block kind reads; the four pre-norm names may also be given by position."""
    block: PartSpec
    parts: tuple[tuple[str, PartUse], ...]

    def __init__(self, block: PartSpec, *positional: PartUse, **named: PartUse):
        names = ("mixer", "mixer_norm", "ffn", "ffn_norm")
        if len(positional) > len(names):
            raise TypeError("at most four parts can be given by position (mixer, mixer_norm, ffn, ffn_norm)")
        uses = dict(zip(names, positional))
        for name, use in named.items():
            if name in uses:
                raise TypeError(f"part {name!r} is given twice")
            uses[name] = use
        for name, use in uses.items():
            if not isinstance(use, PartUse):
                raise TypeError(f"part {name!r} of a layer must be a PartUse, got {type(use).__name__}")
        object.__setattr__(self, "block", block)
        object.__setattr__(self, "parts", tuple(uses.items()))

    def __getattr__(self, name: str) -> PartUse:
        for n, use in object.__getattribute__(self, "parts"):
            if n == name:
                return use
        raise AttributeError(f"this layer has no part named {name!r}")


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
    # numbers that stand for one token's position (1: its index; 3: e.g. time, height, width): the step's
    # ``batch.position_axes`` is [position_axes, T]; callers that give no positions get the index on every axis
    position_axes: int = 1

    def validate(self) -> None:
        if not self.layers or not self.order:
            raise ValueError("a model needs at least one layer and one run")
        if self.position_axes < 1:
            raise ValueError("position_axes must be at least 1")
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"run {i} names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < i:
                    raise ValueError(f"run {i} reads the cache of run {run.cache_from}, which is not an earlier run")
                if self.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"run {i} reads the cache of run {run.cache_from}, which owns none")
