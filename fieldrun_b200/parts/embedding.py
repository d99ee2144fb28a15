"""Token embedding rows into the float32 residual stream (no multiplier, src/minimax.rs:132)
and the vocabulary head: logits = rows @ W^T in float32, W the head's own matrix or the
embedding's when tied (src/minimax.rs:54,373-376)."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, TensorNeed, TensorSource
from .base import Part, register_part
from .linear import linear


class TokenEmbedding(Part):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab_size = int(spec.args["vocab_size"])
        self.width = int(spec.args["width"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.vocab_size, self.width), MATRIX, "normal")]

    def load(self, source: TensorSource) -> None:
        self.weight = source.fetch(self.tensor_needs()[0])

    def forward(self, ctx, tokens: torch.Tensor) -> torch.Tensor:
        x = ctx.buffer("stream", (tokens.numel(), self.width), torch.float32)
        ops.embed_rows(tokens, self.weight, x)
        return x


class VocabHead(Part):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab_size = int(spec.args["vocab_size"])
        self.width = int(spec.args["width"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.vocab_size, self.width), MATRIX, "normal")]

    def load(self, source: TensorSource, shared: Optional[torch.Tensor] = None) -> None:
        self.weight = shared if shared is not None else source.fetch(self.tensor_needs()[0])

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        return linear(rows, self.weight)


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("head", "vocab_head", VocabHead, replace=True)
