"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in 32-bit.

eps sits inside the square root and the weight multiplies last, with no bias and no "+1"
(src/model.rs:919-928, src/cuda.rs:505-515).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Norm, WeightSpec
from .registry import register


@register("norm", "rmsnorm")
class RmsNorm(Norm):
    settles_pending = True      # its kernel adds partial sums a deferred product left for the rows it reads

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.size = int(params["size"])
        self.eps = float(params["eps"])

    def weights(self) -> List[WeightSpec]:
        return [WeightSpec(self.tensor_name("weight", "weight"), (self.size,), "ones")]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.weight = rt.place(tensors[self.tensor_name("weight", "weight")])

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        with ops.bucket("norm"):
            return ops.rmsnorm(x, self.weight, self.eps, self.rt.dtype, rows=rows)
