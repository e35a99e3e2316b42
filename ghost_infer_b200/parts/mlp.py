"""SwiGLU feed-forward: residual += Wdown (silu(Wgate h) * (Wup h)), silu(g) = g / (1 + exp(-g)).

No biases; gate and up are one product over the two matrices stacked by rows, as the reference's GPU
path packs them (src/quant.rs:1135-1154, src/model.rs:1133-1147, src/cuda.rs:9238-9256).

Tensor names: prefix + "mlp.{gate,up,down}_proj.weight" unless `params["tensor_names"]` gives others for the
keys "gate", "up", "down".
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import FeedForward, WeightSpec
from .linear import linear
from .registry import register


@register("feed_forward", "swiglu")
class SwiGlu(FeedForward):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.names = {k: self.tensor_name(k, f"mlp.{k}_proj.weight") for k in ("gate", "up", "down")}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(n["gate"], (self.inter, self.hidden)), WeightSpec(n["up"], (self.inter, self.hidden)),
                WeightSpec(n["down"], (self.hidden, self.inter))]

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        g, u = rt.place(tensors[self.names["gate"]]), rt.place(tensors[self.names["up"]])
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        # 16-bit path: gate and up rows interleaved in blocks of 8, so that one block of the decode kernel
        # holds both halves of an activation and applies SwiGLU before anything is written
        self.interleaved = (rt.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and self.inter % 8 == 0
                            and rt.device.type == "cuda")
        if self.interleaved:
            blocks = self.inter // 8
            self.w_gate_up = torch.stack([g.view(blocks, 8, self.hidden), u.view(blocks, 8, self.hidden)], dim=1) \
                .reshape(2 * self.inter, self.hidden).contiguous()
        else:
            self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        del g, u
        self.w_down = rt.place(tensors[self.names["down"]])

    def forward(self, h, residual, step) -> None:
        with ops.bucket("ffn matmul"):
            if self.interleaved:
                act = ops.swiglu_interleaved(h, self.w_gate_up)
            else:
                gu = linear(h, self.w_gate_up, out_dtype=self.rt.dtype)
                act = ops.silu_mul(gu)
            linear(act, self.w_down, out=residual, accumulate=True)
