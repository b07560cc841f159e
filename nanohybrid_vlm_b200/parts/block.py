"""Pre-norm block with the residual carried apart (nanovllm/models/qwen3.py:146-159).

Every sub-block's output is added to the residual stream inside the next norm, so the
block hands on (output of its feed-forward, residual) and the model's final norm does the
last add.
"""
from __future__ import annotations

from .base import BLOCKS, Block


class PreNormResidualBlock(Block):
    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden
            x = self.mixer_norm.forward(hidden)
        else:
            x = self.mixer_norm.forward_add(hidden, residual)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm.forward_add(a, residual)
        m = self.ffn.forward(x, batch)
        return m, residual


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
