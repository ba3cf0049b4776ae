"""Token embedding (a row gather without scaling, src/kernels.cuh:1877-1881) into the 32-bit
residual stream, and the output head (logits = xn W^T, W the embedding table when tied,
src/api.cu:1367, 1795-1812) producing 32-bit logits."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import ParamSpec
from .registry import Part, register_part, to_compute


class TokenEmbedding(Part):
    """params: name, vocab_size, hidden_size."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.name, self.vocab, self.hidden = params["name"], int(params["vocab_size"]), int(params["hidden_size"])
        self.table = None

    def param_specs(self):
        return [ParamSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.table = to_compute(tensors[self.name], self.ctx)

    def forward(self, tokens):
        x = torch.empty(tokens.numel(), self.hidden, dtype=torch.float32, device=tokens.device)
        return ops.embedding(self.table, tokens, x)


class LMHead(Part):
    """params: name (its own tensor) or tied_to (the embedding's tensor name), vocab_size, hidden_size."""

    def __init__(self, params, ctx, prefix=""):
        super().__init__(params, ctx, prefix)
        self.tied = params.get("tied_to")
        self.name = self.tied or params["name"]
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.weight = None

    def param_specs(self):
        return [] if self.tied else [ParamSpec(self.name, (self.vocab, self.hidden))]

    def load(self, tensors):
        self.weight = ops.Weight(to_compute(tensors[self.name], self.ctx))

    def weight_bytes(self):
        return self.weight.nbytes

    def forward(self, xn):
        logits = torch.empty(xn.shape[0], self.vocab, dtype=torch.float32, device=xn.device)
        if xn.shape[0]:
            ops.linear(xn, self.weight, logits)
        return logits


register_part("embedding", "token", TokenEmbedding)
register_part("head", "linear", LMHead)
