"""The two ends of the model: the token embedding and the output head."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels as K
from ..registry import register_embedding, register_head
from .base import Embedding, Head, StepContext
from .linear import linear


@register_embedding("table")
class TableEmbedding(Embedding):
    """x[t] = weight[token_ids[t]], widened to float32 (crates/aien-inference-abi/src/
    transformer_backend.rs:1179-1181, src/weights.rs:140-146; ids are checked against the
    vocabulary before a step is accepted instead of being reduced modulo it)."""

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {"weight": ((self.vocab_size, self.hidden_size), "embedding")}

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def tied_weight(self):
        return self.weight

    def forward(self, ctx: StepContext, token_ids: torch.Tensor, x: torch.Tensor) -> None:
        K.embed_gather(self.weight, token_ids, x)


@register_head("linear")
class LinearHead(Head):
    """logits = rows . W^T with W = ``weight`` [vocab, hidden], or the embedding's table when
    tied: the same buffer, no copy (crates/aien-inference-abi/src/weights.rs:131-136,
    src/transformer_backend.rs:1370-1386)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool = False):
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.weight: Optional[torch.Tensor] = None

    def param_shapes(self):
        return {} if self.tied else {"weight": ((self.vocab_size, self.hidden_size), "matrix")}

    def bind(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: Embedding) -> None:
        w = embedding.tied_weight()
        if w is None or tuple(w.shape) != (self.vocab_size, self.hidden_size):
            raise ValueError("the head is tied to an embedding that offers no [vocab, hidden] matrix")
        self.weight = w

    def forward(self, ctx: StepContext, rows: torch.Tensor, logits: torch.Tensor) -> None:
        linear(ctx, rows, self.weight, out=logits)
