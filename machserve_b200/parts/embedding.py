"""The two ends of the model: token embedding, and the head that turns the final hidden rows into logits."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorDecl
from .base import Head, TokenEmbedding, matrix, register_embedding, register_head


@register_embedding("embedding")
class Embedding(TokenEmbedding):
    """x[r, :] = E[token[r], :] into the float32 residual stream, no scaling
    (crates/mach-model/src/kernels.rs:578-585 of gqf2008/machserve).

    params: tensor, vocab_size, hidden_size.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.vocab, self.hidden = spec["tensor"], int(spec["vocab_size"]), int(spec["hidden_size"])

    def tensors(self):
        return [TensorDecl(self.name, (self.vocab, self.hidden))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.table = matrix(tensors[self.name], rt)

    def forward(self, ctx, out):
        return ops.embed_gather(self.table, ctx.token_ids, out)


@register_head("lm_head")
class LMHead(Head):
    """logits = x . W^T in float32, for the rows that are asked for only (the reference computes
    every row, crates/mach-model/src/batched.rs:4594-4626).  With `tied_to` set, the head's own
    tensor may be absent and the embedding table stands in
    (crates/mach-model/src/loader.rs:1025-1033); if it is present it is used.

    params: tensor, tied_to (name of the embedding tensor, or None), vocab_size, hidden_size.
    """

    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.name, self.tied_to = spec["tensor"], spec.get("tied_to")
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])

    def tensors(self):
        out = [TensorDecl(self.name, (self.vocab, self.hidden), required=self.tied_to is None, random=self.tied_to is None)]
        if self.tied_to is not None:
            out.append(TensorDecl(self.tied_to, (self.vocab, self.hidden)))
        return out

    def bind(self, tensors, rt, embedding=None):
        super().bind(tensors, rt, embedding)
        if self.name in tensors:
            self.weight = matrix(tensors[self.name], rt)
        elif embedding is not None and getattr(embedding, "name", None) == self.tied_to and hasattr(embedding, "table"):
            self.weight = embedding.table  # the embedding's own device tensor: one copy in memory
        else:
            self.weight = matrix(tensors[self.tied_to], rt)

    def forward(self, ctx, x, out):
        return ops.linear(x, self.weight, None, out)
