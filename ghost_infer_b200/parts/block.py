"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from ..kernels import ops
from .base import Block
from .registry import register


@register("block", "prenorm_residual")
class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x)), the residual stream x kept in 32-bit
    (src/model.rs:996-1147; the reference's stream is f32 too, src/model.rs:704-705)."""

    def forward(self, x, step, memory) -> None:
        # The last product of the mixer and of the feed-forward adds into x; in a decode step it may leave
        # partial sums pending for the norm that reads x next (a norm that cannot add them has them settled first).
        if x.is_cuda and not getattr(self.mixer_norm, "settles_pending", False):
            ops.settle(x)
        h = self.mixer_norm.forward(x)
        with ops.defer_into(x):
            self.mixer.forward(h, x, step, memory)
        if x.is_cuda and not getattr(self.ffn_norm, "settles_pending", False):
            ops.settle(x)
        h = self.ffn_norm.forward(x)
        with ops.defer_into(x):
            self.ffn.forward(h, x, step)
