"""Token embedding and output head (nanovllm/layers/embed_head.py:9-66).

The head takes only the rows whose logits are wanted and returns them in fp32.  A tied head
owns no tensor: it is given the embedding's table.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import EMBEDDINGS, HEADS, Embedding, Head
from .spec import ParamDecl


class TokenEmbedding(Embedding):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])

    def params(self):
        return [ParamDecl("weight", (self.vocab, self.env.hidden_size))]

    def forward(self, token_ids, batch=None):
        out = self.new(token_ids.numel(), self.env.hidden_size)
        ops.embed(out, self.w_weight, token_ids)
        return out


class LMHead(Head):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.tied = bool(spec.get("tied", False))

    def params(self):
        return [] if self.tied else [ParamDecl("weight", (self.vocab, self.env.hidden_size))]

    def tie(self, embedding) -> None:
        self.w_weight = embedding.w_weight

    def streamed_weights(self):
        return [(self.w_weight, 1)]

    def forward(self, rows_hidden):
        logits = self.new(rows_hidden.shape[0], self.vocab, dtype=torch.float32)
        ops.linear(logits, rows_hidden, self.w_weight)
        return logits


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("lm_head", LMHead)
