"""A causal language model put together from a :class:`ModelSpec`.

It builds the parts, lists every tensor they own with the checkpoint tensors that fill it,
and runs one step over a packed batch: embed, the layer runs in the order the spec gives,
the final norm at the wanted rows only, the head.  It is the same object for every
architecture; what differs is the spec.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from .. import parts as _registered_parts  # noqa: F401  (importing the package registers the built-in parts)
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, BuildEnv, FixedStateNeed, PagedKVNeed, Part
from ..parts.spec import ModelSpec, ParamDecl, PartUse


@dataclass(frozen=True)
class BoundParam:
    """A tensor of the model: its full name, declaration (sources carry full checkpoint names) and owner."""
    name: str
    decl: ParamDecl
    owner: Part
    local: str


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        env = self.env = BuildEnv(spec.hidden_size, dtype, device, spec.max_position)
        self._uses: list[tuple[PartUse, Part]] = []

        def build(registry, use: PartUse):
            obj = registry.get(use.spec.kind)(use.spec, env)
            self._uses.append((use, obj))
            return obj

        self.embedding = build(EMBEDDINGS, spec.embedding)
        for use in spec.positions:                 # before the layers, so that mixers naming the same spec share them
            self._uses.append((use, env.position(use.spec)))
        self.blocks = []
        for i, layer in enumerate(spec.layers):
            block_cls = BLOCKS.get(layer.block.kind)
            given = dict(layer.parts)
            unknown = set(given) - set(block_cls.SLOTS)
            missing = set(block_cls.SLOTS) - set(given) - set(block_cls.OPTIONAL)
            if unknown or missing:
                raise ValueError(f"layer {i}: block {layer.block.kind!r} arranges {sorted(block_cls.SLOTS)}; "
                                 f"missing {sorted(missing)}, unknown {sorted(unknown)}")
            built = {name: build(block_cls.SLOTS[name], use) for name, use in layer.parts}
            self.blocks.append(block_cls(layer.block, built))
        self.final_norm = build(NORMS, spec.final_norm)
        self.head = build(HEADS, spec.head)
        self.positions = list(env._positions.values())

    # ------------------------------------------------------------------ tensors
    def param_table(self) -> list[BoundParam]:
        table, seen = [], set()
        for use, obj in self._uses:
            for decl in obj.params():
                full = use.prefix + decl.name
                if full in seen:
                    raise ValueError(f"two parts declare the tensor {full!r}")
                seen.add(full)
                srcs = tuple(replace(s, name=use.prefix + s.name) for s in decl.resolved_sources())
                table.append(BoundParam(full, ParamDecl(decl.name, decl.shape, decl.init, decl.storage, srcs), obj,
                                        decl.name))
        return table

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        """Hand every part its tensors (``tensors`` is keyed by full names)."""
        per_part: dict[int, dict[str, torch.Tensor]] = {}
        owners = {}
        for bp in self.param_table():
            if bp.name not in tensors:
                raise KeyError(f"no tensor for {bp.name}")
            per_part.setdefault(id(bp.owner), {})[bp.local] = tensors[bp.name]
            owners[id(bp.owner)] = bp.owner
        for key, owner in owners.items():
            owner.bind(per_part[key])
        if self.head.tied:
            self.head.tie(self.embedding)
        self.tensors = tensors

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())

    def streamed_weights(self) -> list[tuple[torch.Tensor, int]]:
        """Every matrix that a decode step streams once (each once, though several parts may share it)."""
        seen, out = set(), []
        for _, obj in self._uses:
            for w, mode in obj.streamed_weights():
                if w.data_ptr() not in seen:
                    seen.add(w.data_ptr())
                    out.append((w, mode))
        return out

    # ------------------------------------------------------------------ cache needs
    def cache_needs(self) -> list[PagedKVNeed | FixedStateNeed | None]:
        """For every run of the order: what its mixer keeps between steps (None: nothing, or it reads
        another run's cache)."""
        needs = []
        for run in self.spec.order:
            owner = self.blocks[run.layer].cache_owner
            need = owner.cache_need() if owner is not None else None
            if run.cache_from is not None:
                src_owner = self.blocks[self.spec.order[run.cache_from].layer].cache_owner
                src = src_owner.cache_need() if src_owner is not None else None
                if need != src:
                    raise ValueError(f"a run reads the cache of run {run.cache_from}, whose shape differs from its own")
                need = None
            needs.append(need)
        return needs

    # ------------------------------------------------------------------ one step
    profile_ranges = False      # set by the runner from the engine option of that name

    def forward(self, batch, storage) -> torch.Tensor:
        """Run the batch's tokens through every layer run; returns fp32 logits [wanted rows, vocab]."""
        if self.profile_ranges:
            return self._forward_with_ranges(batch, storage)
        h = self.embedding.forward(batch.token_ids, batch)
        for pos in self.positions:
            h = pos.add_to_embeddings(h, batch)
        residual = None
        for i, run in enumerate(self.spec.order):
            view = storage.view(i, run.cache_from, batch)
            h, residual = self.blocks[run.layer].forward(h, residual, batch, view)
        if batch.n_logit_rows == 0:
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=self.device)
        x = self.final_norm.forward_add_rows(h, residual, batch.logit_rows)
        return self.head.forward(x)

    def _forward_with_ranges(self, batch, storage) -> torch.Tensor:
        """``forward`` with an NVTX range around the step ("step T=<tokens> S=<requests>"), the embedding, every
        layer run ("run <i> layer <j>"), and the final norm with the head."""
        nvtx = torch.cuda.nvtx
        nvtx.range_push(f"step T={batch.n_tokens} S={batch.n_seqs}")
        try:
            nvtx.range_push("embedding")
            h = self.embedding.forward(batch.token_ids, batch)
            for pos in self.positions:
                h = pos.add_to_embeddings(h, batch)
            nvtx.range_pop()
            residual = None
            for i, run in enumerate(self.spec.order):
                nvtx.range_push(f"run {i} layer {run.layer}")
                view = storage.view(i, run.cache_from, batch)
                h, residual = self.blocks[run.layer].forward(h, residual, batch, view)
                nvtx.range_pop()
            if batch.n_logit_rows == 0:
                return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=self.device)
            nvtx.range_push("final norm and head")
            x = self.final_norm.forward_add_rows(h, residual, batch.logit_rows)
            logits = self.head.forward(x)
            nvtx.range_pop()
            return logits
        finally:
            nvtx.range_pop()
