"""RMSNorm with the residual add fused in (nanovllm/layers/layernorm.py:5-50).

Parameters: ``width``, ``eps``, ``weight_offset`` (0 for ``x * w``; 1 for the ``x * (1 + w)``
convention some models store).
"""
from __future__ import annotations

from ..kernels import ops
from .base import NORMS, Norm
from .spec import ParamDecl


class RMSNorm(Norm):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = spec["width"]
        self.eps = float(spec["eps"])
        self.weight_offset = float(spec.get("weight_offset", 0.0))

    def params(self):
        return [ParamDecl("weight", (self.width,), init="norm" if self.weight_offset == 0.0 else "zeros_noise")]

    def forward(self, x):
        out = self.new(*x.shape)
        ops.rmsnorm(out, x, self.w_weight, self.eps, weight_offset=self.weight_offset)
        return out

    def forward_add(self, x, residual):
        out = self.new(*x.shape)
        ops.rmsnorm(out, x, self.w_weight, self.eps, residual=residual, weight_offset=self.weight_offset)
        return out

    def forward_add_rows(self, x, residual, rows):
        out = self.new(rows.numel(), x.shape[-1])
        ops.rmsnorm(out, x, self.w_weight, self.eps, residual=residual, rows=rows, write_residual=False,
                    weight_offset=self.weight_offset)
        return out


NORMS.register("rmsnorm", RMSNorm)
