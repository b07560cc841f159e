"""Interfaces of the parts a layer is put together from, and the registries that map a
``PartSpec.kind`` to its class.

A part is built from its spec and a :class:`BuildEnv` (width of the residual stream,
dtype, device); it declares its tensors (:class:`~.spec.ParamDecl`), receives them with
``bind`` and then computes on device tensors.  No part knows which model it is in.

Adding a part: subclass the interface, then ``MIXERS.register("name", Class)`` (or
``FEED_FORWARDS``, ``NORMS``, ``POSITIONS``, ``BLOCKS``, ``EMBEDDINGS``, ``HEADS``).  A model
description refers to it as ``part("name", ...)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from .spec import ParamDecl, PartSpec


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._classes: dict[str, type] = {}

    def register(self, kind: str, cls: type, replace: bool = False) -> None:
        if kind in self._classes and not replace:
            raise ValueError(f"{self.what} {kind!r} is already registered")
        self._classes[kind] = cls

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def get(self, kind: str) -> type:
        if kind not in self._classes:
            raise KeyError(f"unknown {self.what} {kind!r}; registered: {sorted(self._classes)}")
        return self._classes[kind]

    def kinds(self) -> list[str]:
        return sorted(self._classes)


EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block arrangement")


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values of every token (or of the last ``window`` tokens) in pages."""
    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedStateNeed:
    """A tensor of fixed shape per live request (``dtype``: "float32" or "model")."""
    shape: tuple[int, ...]
    dtype: str = "float32"


class BuildEnv:
    """What a part may know about its surroundings."""

    def __init__(self, hidden_size: int, dtype: torch.dtype, device: torch.device | str, max_position: int):
        self.hidden_size = hidden_size
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_position = max_position
        self._positions: dict[PartSpec, "PositionEncoding"] = {}

    def position(self, spec: PartSpec | None):
        """The position encoding for ``spec``; equal specs share one object (one table on the device)."""
        if spec is None:
            return None
        if spec not in self._positions:
            self._positions[spec] = POSITIONS.get(spec.kind)(spec, self)
        return self._positions[spec]


class Part:
    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def params(self) -> list[ParamDecl]:
        return []

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the tensors declared by ``params`` (keyed by their local names)."""
        for name, t in tensors.items():
            setattr(self, "w_" + name.replace(".", "_"), t)

    def streamed_weights(self) -> list[tuple[torch.Tensor, int]]:
        """The matrices that a decode step reads once from end to end, with the mode in which
        ``kernels.ops`` streams them (0: plain product, 1: fp32 logits, 2: [gate; up] rows with SiLU).  The
        engine may keep a second copy of each, laid out for the weight-streaming kernel.  Default: none."""
        return []

    def new(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(*shape, dtype=dtype or self.env.dtype, device=self.env.device)


@dataclass
class CacheView:
    """What one run of a mixer sees of the cache.

    Paged: ``pages`` [num_pages, 2, kv_heads, page_size, head_dim] of this run (or of the run it
    reads from), ``tables`` the step's block tables and slot mapping for the run's group,
    ``writes`` False if the run must not store keys and values.
    Fixed state: ``state`` [num_slots, *shape]; the step's slots are ``batch.state_slots``.
    """
    pages: torch.Tensor | None = None
    tables: Any = None
    writes: bool = True
    state: torch.Tensor | None = None


class Mixer(Part):
    def cache_need(self) -> PagedKVNeed | FixedStateNeed | None:
        return None

    def forward(self, x: torch.Tensor, batch, cache: CacheView) -> torch.Tensor:
        """x [T, hidden] (normed) -> [T, hidden]; tokens of all requests of the step, packed."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """residual += x (in place, fp32 sum rounded once); returns norm of the unrounded sum."""
        raise NotImplementedError

    def forward_add_rows(self, x: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """Norm of (x + residual) at the given rows only; nothing is written back."""
        raise NotImplementedError


class PositionEncoding(Part):
    """How positions enter the model.  ``rotary()`` gives (table [max_position, rotary_dim] fp32 with
    cos then sin halves, rotary_dim) for mixers that rotate queries and keys, or None;
    ``add_to_embeddings`` lets an absolute encoding change the embedded tokens."""

    def rotary(self):
        return None

    def add_to_embeddings(self, h: torch.Tensor, batch) -> torch.Tensor:
        return h


class Embedding(Part):
    """Token ids to the first hidden states.  ``forward(token_ids [T] int32, batch) -> [T, hidden]``."""

    def forward(self, token_ids: torch.Tensor, batch) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    """Hidden states of the wanted rows (after the final norm) to fp32 logits [rows, vocab].  ``tied`` True: the
    head owns no table and is handed the embedding part with ``tie`` once the tensors are bound."""
    tied = False

    def tie(self, embedding: Embedding) -> None:
        raise NotImplementedError

    def forward(self, rows_hidden: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """The arrangement of a layer's parts.  ``SLOTS`` names the parts this kind of block arranges and the
    registry each is built from; ``OPTIONAL`` those a layer may leave out.  The model builds them and hands
    them over as ``parts`` (name -> part; each is also set as an attribute of that name).  ``forward`` takes and
    returns (hidden, residual): the sub-block output not yet added, and the residual stream; residual None means
    "first layer".  ``cache_owner`` is the part whose ``cache_need`` decides what a run of this layer keeps
    between steps (one per layer)."""
    SLOTS: dict[str, Registry] = {"mixer": MIXERS, "mixer_norm": NORMS, "ffn": FEED_FORWARDS, "ffn_norm": NORMS}
    OPTIONAL: tuple[str, ...] = ()

    def __init__(self, spec: PartSpec, parts: dict[str, Part]):
        self.spec = spec
        self.parts = dict(parts)
        for name, obj in parts.items():
            setattr(self, name, obj)

    @property
    def cache_owner(self) -> Mixer | None:
        return self.parts.get("mixer")

    def forward(self, hidden, residual, batch, cache: CacheView):
        raise NotImplementedError
