"""Matrix products of the parts: out (+)= h @ W^T with W stored [out, in], no bias (src/model.rs:1019).

One place decides which kernel runs a product, from the dtypes and sizes alone; parts only say what
they want computed.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


def linear(h: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    """`accumulate=True`: `out` is the float32 residual stream and the product is added to it."""
    return ops.linear(h, w, out=out, out_dtype=out_dtype, accumulate=accumulate)
