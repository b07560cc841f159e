"""The cache's device tensors and the views that mixers get of them.

For every layer run whose mixer keeps keys and values: one tensor
[num_pages, 2 (K, V), kv_heads, page_size, head_dim] in the engine's dtype, indexed by the
page ids of the run's group.  Inside a page each KV head's tokens are contiguous, so a
decode kernel streams page_size * head_dim elements per head in one piece.  (The reference
keeps [2, layers, pages, page_size, kv_heads, head_dim], nanovllm/engine/model_runner.py:870-881.)
For every run with fixed-size state: one zeroed tensor [num_slots, *shape].
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import CacheView, FixedStateNeed, PagedKVNeed
from .manager import GroupSpec


@dataclass
class CacheLayout:
    """Which group each run belongs to (None: the run keeps no pages)."""
    groups: list[GroupSpec]
    run_group: list[int | None]
    needs: list

    @classmethod
    def from_needs(cls, needs: list) -> "CacheLayout":
        groups: list[GroupSpec] = []
        run_group: list[int | None] = []
        for need in needs:
            if isinstance(need, PagedKVNeed):
                g = GroupSpec(need.window)
                if g not in groups:
                    groups.append(g)
                run_group.append(groups.index(g))
            else:
                run_group.append(None)
        return cls(groups, run_group, list(needs))

    @property
    def needs_state_slots(self) -> bool:
        return any(isinstance(n, FixedStateNeed) for n in self.needs)

    def page_bytes(self, page_size: int, dtype: torch.dtype) -> list[int]:
        """Bytes that one page id of each group stands for (summed over the group's runs)."""
        item = torch.empty((), dtype=dtype).element_size()
        out = [0] * len(self.groups)
        for need, g in zip(self.needs, self.run_group):
            if g is not None:
                out[g] += 2 * need.num_kv_heads * page_size * need.head_dim * item
        return out

    def state_bytes_per_slot(self, dtype: torch.dtype) -> int:
        total = 0
        for need in self.needs:
            if isinstance(need, FixedStateNeed):
                n = 1
                for s in need.shape:
                    n *= s
                total += n * (4 if need.dtype == "float32" else torch.empty((), dtype=dtype).element_size())
        return total


class CacheStorage:
    def __init__(self, layout: CacheLayout, order, page_size: int, num_pages: list[int], num_state_slots: int,
                 dtype: torch.dtype, device, poison: bool = False):
        """``poison``: the pools start as NaN instead of zeros, so that a kernel that reads a slot which no step
        has written (beyond a request's tokens, or a page of another request) cannot go unnoticed."""
        self.layout = layout
        self.order = list(order)
        self.page_size = page_size
        self.num_pages = list(num_pages)
        self.pages: list[torch.Tensor | None] = []
        self.states: list[torch.Tensor | None] = []
        for need, g in zip(layout.needs, layout.run_group):
            if isinstance(need, PagedKVNeed):
                self.pages.append(torch.full((num_pages[g], 2, need.num_kv_heads, page_size, need.head_dim),
                                             float("nan") if poison else 0.0, dtype=dtype, device=device))
                self.states.append(None)
            elif isinstance(need, FixedStateNeed):
                sdt = torch.float32 if need.dtype == "float32" else dtype
                self.pages.append(None)
                self.states.append(torch.full((max(num_state_slots, 1), *need.shape), float("nan") if poison else 0.0,
                                              dtype=sdt, device=device))
            else:
                self.pages.append(None)
                self.states.append(None)

    def view(self, run: int, cache_from: int | None, batch) -> CacheView:
        src = run if cache_from is None else cache_from
        g = self.layout.run_group[src]
        return CacheView(pages=self.pages[src], tables=batch.groups[g] if g is not None else None,
                         writes=cache_from is None, state=self.states[src])

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.pages + self.states if t is not None)
