"""Token embedding and output head.

x[t] = E[token_t] without scaling (src/model.rs:987-990); logits = W normed with no bias, no cap, no
scaling, where W is the embedding table when the model ties them (src/model.rs:637-638, :1183-1186).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Part, WeightSpec
from .linear import linear
from .registry import register


@register("embedding", "token_embedding")
class TokenEmbedding(Part):
    def __init__(self, params, prefix="model.embed_tokens."):
        super().__init__(params, prefix)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])

    def weights(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor_name("weight", "weight"), (self.vocab, self.hidden))]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.weight = rt.place(tensors[self.tensor_name("weight", "weight")])

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        with ops.bucket("embed"):
            return ops.embed(self.weight, tokens)


@register("head", "linear_head")
class LinearHead(Part):
    def __init__(self, params, prefix="lm_head."):
        super().__init__(params, prefix)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied = bool(params.get("tied", False))
        self.weight: Optional[torch.Tensor] = None

    def weights(self) -> List[WeightSpec]:
        return [] if self.tied else [WeightSpec(self.tensor_name("weight", "weight"), (self.vocab, self.hidden))]

    def ignorable(self) -> List[str]:
        """Names a file may carry without their being used (a tied model that still stores its head)."""
        return [self.tensor_name("weight", "weight")] if self.tied else []

    def bind(self, tensors, rt, embedding: Optional[TokenEmbedding] = None) -> None:
        super().bind(tensors, rt)
        if self.tied:
            if embedding is None:
                raise ValueError("a tied head needs the embedding it is tied to")
            self.weight = embedding.weight
        else:
            self.weight = rt.place(tensors[self.tensor_name("weight", "weight")])

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        with ops.bucket("logits"):
            return linear(h, self.weight, out_dtype=torch.float32)
