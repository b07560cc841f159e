"""SwiGLU feed-forward (nanovllm/models/qwen3.py:91-117, nanovllm/layers/activation.py:6-11).

Parameters: ``intermediate_size``.  Tensors: ``gate_up_proj.weight`` [2 I, width], rows gate
then up, packed from gate_proj / up_proj (nanovllm/layers/linear.py:102-108);
``down_proj.weight`` [width, I].
"""
from __future__ import annotations

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .spec import ParamDecl, Source


class SwiGLU(FeedForward):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.inter = int(spec["intermediate_size"])

    def params(self):
        H, I = self.env.hidden_size, self.inter
        return [
            ParamDecl("gate_up_proj.weight", (2 * I, H), sources=(
                Source("gate_proj.weight", 0, I), Source("up_proj.weight", I, I))),
            ParamDecl("down_proj.weight", (H, I)),
        ]

    def streamed_weights(self):
        return [(self.w_gate_up_proj_weight, 2), (self.w_down_proj_weight, 0)]

    def forward(self, x, batch):
        T = x.shape[0]
        act = self.new(T, self.inter)
        if not ops.swiglu_first_half(act, x, self.w_gate_up_proj_weight):
            gate_up = self.new(T, 2 * self.inter)
            ops.linear(gate_up, x, self.w_gate_up_proj_weight)
            ops.silu_mul(act, gate_up)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, act, self.w_down_proj_weight)
        return y


FEED_FORWARDS.register("swiglu", SwiGLU)
