"""Token embedding: x[t] = table[id_t] (+ the position table's row, fused into
the same kernel when the position encoding is an additive table;
src/kernels/embedding.cu:23-43).  The result is the 32-bit residual stream; with ``copies`` > 1
a token's row holds that many copies side by side: the start of a residual of several streams.  With ``norm_eps`` the
rows are RMS-normed with a weight of their own before anything reads them (x / sqrt(mean(x^2) + eps) * w, 32-bit), and a
copy in the activation dtype is left for the first layer."""
from __future__ import annotations

import torch

from .base import Embedding, ParamSpec, register_part


class TokenEmbedding(Embedding):
    def __init__(self, hidden_size: int, vocab_size: int, copies: int = 1, norm_eps=None):
        self.hidden_size = int(hidden_size)
        self.vocab_size = int(vocab_size)
        self.copies = int(copies)
        self.norm_eps = None if norm_eps is None else float(norm_eps)
        if self.copies < 1:
            raise ValueError("TokenEmbedding: copies must be at least 1")
        if self.norm_eps is not None and self.copies != 1:
            raise ValueError("TokenEmbedding: the norm of the embedded rows takes one copy")

    def param_specs(self):
        p = {"table": ParamSpec((self.vocab_size, self.hidden_size), "table")}
        if self.norm_eps is not None:
            p["norm_weight"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def forward(self, ctx, positions):
        x = ctx.ws.buf("residual", ctx.T, self.hidden_size * self.copies, torch.float32)
        pos_table = positions.embedding_table() if positions is not None else None
        self.rt.ops.embed(ctx.token_ids, ctx.positions, self.table, pos_table, x, copies=self.copies)
        if self.norm_eps is not None:
            from .block import leave_act_copy
            h = None
            if self.rt.act_dtype != torch.float32:
                h = ctx.ws.buf("post_norm_out", ctx.T, self.hidden_size, self.rt.act_dtype)
            self.rt.ops.post_norm(x, self.norm_weight, self.norm_eps, 1.0, h=h)
            leave_act_copy(ctx, x, x if h is None else h)
        return x


register_part("embedding", "token", TokenEmbedding)
