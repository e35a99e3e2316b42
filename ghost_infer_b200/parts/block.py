"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import Block
from .registry import register


@register("block", "prenorm_residual")
class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x)), the residual stream x kept in 32-bit
    (src/model.rs:996-1147; the reference's stream is f32 too, src/model.rs:704-705)."""

    def forward(self, x, step, memory) -> None:
        h = self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, memory)
        h = self.ffn_norm.forward(x)
        self.ffn.forward(h, x, step)
