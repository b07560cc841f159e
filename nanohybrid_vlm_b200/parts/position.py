"""Rotary position encoding: the fp32 cos/sin table of nanovllm/layers/rotary_embedding.py:83-89.

Parameters: ``theta`` (base), ``rotary_dim`` (how many leading elements of a head rotate;
the rest pass through), ``max_position``.  The angles are position * inv_freq in fp32, as
the reference computes them; mixers that rotate queries and keys read the table in their
fused kernel.
"""
from __future__ import annotations

import torch

from .base import POSITIONS, PositionEncoding


class RotaryTable(PositionEncoding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.rotary_dim = int(spec["rotary_dim"])
        self.theta = float(spec["theta"])
        self.max_position = int(spec["max_position"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        # Built once on the host in fp32 so that every device sees the same angles.
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim))
        t = torch.arange(self.max_position, dtype=torch.float32)
        freqs = t[:, None] * inv_freq[None, :]
        self.table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(env.device)

    def rotary(self):
        return self.table, self.rotary_dim


class NoPosition(PositionEncoding):
    """No position signal at all (order then enters only through causality)."""


POSITIONS.register("rope", RotaryTable)
POSITIONS.register("none", NoPosition)
