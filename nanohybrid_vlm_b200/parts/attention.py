"""Grouped-query attention over the paged cache (nanovllm/models/qwen3.py:14-88).

Parameters: ``num_heads``, ``num_kv_heads``, ``head_dim`` (num_heads * head_dim need not
equal the model width), ``qk_norm_eps`` (None: no per-head q/k RMSNorm), ``position`` (a
PartSpec of a position encoding, or None), ``scale`` (None: head_dim ** -0.5), ``window``
(None: all keys; n: the last n keys), ``qk_norm_weight_offset``.

Tensors: ``qkv_proj.weight`` [(nq + 2 nkv) d, width], rows q then k then v, packed from the
checkpoint's q_proj / k_proj / v_proj (nanovllm/layers/linear.py:153-167);
``q_norm.weight`` / ``k_norm.weight`` [d]; ``o_proj.weight`` [width, nq d].
"""
from __future__ import annotations

from ..kernels import ops
from .base import MIXERS, Mixer, PagedKVNeed
from .spec import ParamDecl, Source


class GQAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads do not divide into {self.nkv} KV heads")
        eps = spec.get("qk_norm_eps")
        self.qk_norm = eps is not None
        self.eps = float(eps) if eps is not None else 0.0
        self.norm_offset = float(spec.get("qk_norm_weight_offset", 0.0))
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.d ** -0.5
        self.window = spec.get("window")
        self.position = env.position(spec.get("position"))
        self.q_size, self.kv_size = self.nq * self.d, self.nkv * self.d

    def params(self):
        H = self.env.hidden_size
        decls = [
            ParamDecl("qkv_proj.weight", (self.q_size + 2 * self.kv_size, H), sources=(
                Source("q_proj.weight", 0, self.q_size),
                Source("k_proj.weight", self.q_size, self.kv_size),
                Source("v_proj.weight", self.q_size + self.kv_size, self.kv_size))),
            ParamDecl("o_proj.weight", (H, self.q_size)),
        ]
        if self.qk_norm:
            init = "norm" if self.norm_offset == 0.0 else "zeros_noise"
            decls += [ParamDecl("q_norm.weight", (self.d,), init=init), ParamDecl("k_norm.weight", (self.d,), init=init)]
        return decls

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def streamed_weights(self):
        return [(self.w_qkv_proj_weight, 0), (self.w_o_proj_weight, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        qkv = self.new(T, self.q_size + 2 * self.kv_size)
        ops.linear(qkv, x, self.w_qkv_proj_weight)
        rot = self.position.rotary() if self.position is not None else None
        table, rotary_dim = rot if rot is not None else (None, 0)
        q_w = self.w_q_norm_weight if self.qk_norm else None
        k_w = self.w_k_norm_weight if self.qk_norm else None
        o = self.new(T, self.q_size)
        # a step of single tokens: the decode kernel takes qkv as it is (norm, rotation and store inside it)
        if not ops.attention_decode_fused(o, qkv, cache.pages, cache.tables, batch, self.nq, self.nkv, self.d,
                                          self.scale, self.window or 0, q_w, k_w, table, rotary_dim, self.eps,
                                          self.norm_offset, cache.writes):
            q = self.new(T, self.q_size)
            ops.qk_norm_rope_store(
                qkv, q, cache.pages if cache.writes else None, cache.tables.slot_mapping, batch.positions,
                q_w, k_w, table, rotary_dim, self.nq, self.nkv, self.d, self.eps, self.norm_offset)
            self.attend(o, q, batch, cache)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, o, self.w_o_proj_weight)
        return y

    def attend(self, o, q, batch, cache):
        ops.attention(o, q, cache.pages, cache.tables, batch, self.nq, self.nkv, self.d, self.scale,
                      self.window or 0)


MIXERS.register("gqa_attention", GQAttention)
