"""The two ends of a model: the token embedding and the linear head.

The embedding gathers rows of its table into the 32-bit residual stream (the reference gathers on
the host, src/transformer/embedding.zig:6-31); the head multiplies the final norm's rows with its
matrix into 32-bit logits (src/main.zig:867-881).  When the embedding is tied the head uses the
embedding's table (src/loader/gguf_model.zig:47-54).
"""
from __future__ import annotations

import torch

from .base import Embedding, Head, ParamDecl, register_part


class TokenEmbedding(Embedding):
    graph_safe = True      # forward launches kernels only; nothing is read back to the host

    def __init__(self, weight: str, vocab: int, hidden: int):
        self.weight_name, self.vocab, self.hidden = weight, int(vocab), int(hidden)
        self.table = None

    def params(self):
        return {self.weight_name: ParamDecl((self.vocab, self.hidden), "table")}

    def bind(self, tensors, dtype):
        self.table = tensors[self.weight_name]

    def forward(self, token_ids, step):
        return step.ops.embed(token_ids, self.table)


class LinearHead(Head):
    accepts_lazy_input = True     # x goes straight into a product
    graph_safe = True

    def __init__(self, weight: str, tied: bool, vocab: int, hidden: int):
        self.weight_name, self.tied, self.vocab, self.hidden = weight, bool(tied), int(vocab), int(hidden)
        self.w = None

    def params(self):
        return {} if self.tied else {self.weight_name: ParamDecl((self.vocab, self.hidden), "matrix")}

    def bind(self, tensors, dtype):
        if not self.tied:
            self.w = tensors[self.weight_name]

    def tie(self, embedding):
        self.w = embedding.table

    def forward(self, x, step):
        return step.ops.linear(x, self.w, out_dtype=torch.float32)


register_part("embedding", "embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
