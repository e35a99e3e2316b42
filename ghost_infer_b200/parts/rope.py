"""Rotary position encoding with the llama3 frequency scaling.

Rotation (src/model.rs:942-953): for pair i of a head, theta = pos * inv_freq[i] in 32-bit and
(a, b) <- (a cos - b sin, a sin + b cos); q and k are rotated before the cache write, v is not.
Plain frequencies: inv_freq[i] = theta_base ** (-2 i / rotary_dim) (src/model.rs:768).  The reference
divides them by a per-pair table it finds in the file (`rope_freqs`, src/model.rs:30-31, :229-231);
here that table comes from config.json's rope_scaling with the llama3 rule: a pair whose wavelength
2 pi / inv_freq is shorter than original_max / high_freq_factor keeps its frequency, one longer than
original_max / low_freq_factor has it divided by `factor`, and those between are blended linearly
in original_max / wavelength.  The table is computed once in 64-bit and rounded to 32-bit.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register


def rotary_inv_freq(rotary_dim: int, theta: float, scaling: Optional[Mapping]) -> torch.Tensor:
    """float32 [rotary_dim / 2]."""
    half = rotary_dim // 2
    out = []
    for i in range(half):
        f = theta ** (-(2.0 * i) / rotary_dim)
        if scaling is not None:
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen > orig / low:
                f = f / factor
            elif wavelen >= orig / high:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


@register("position", "rotary")
class Rotary(PositionEncoding):
    settles_pending = True      # its kernel adds partial sums a deferred product left in place of row values

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.pairing = params.get("pairing", "half")
        if self.pairing not in ("half", "adjacent"):
            raise ValueError(f"rotary pairing must be \"half\" or \"adjacent\", got {self.pairing!r}")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        scaling = params.get("scaling")
        if scaling is not None and scaling.get("rope_type", "llama3") != "llama3":
            raise ValueError(f"rotary scaling of type {scaling.get('rope_type')!r} is not supported")
        self.scaling = scaling
        self.inv_freq_host = rotary_inv_freq(self.rotary_dim, self.theta, scaling)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        self.inv_freq = self.inv_freq_host.to(rt.device)
        sc = self.scaling
        self.table_key = ("rotary", self.rotary_dim, self.theta, repr(sorted(sc.items())) if sc else None)

    def _table(self, step):
        # the angles depend on the step's positions and this encoding's constants only: one table per step
        # serves every layer that rotates the same way
        table = step.shared.get(self.table_key)
        if table is None:
            table = ops.rope_table(step.positions, self.inv_freq)
            step.shared[self.table_key] = table
        return table

    def project_and_store(self, h, w_qkv, step, memory, n_heads, n_kv_heads, head_dim):
        # a prompt step's product on the tensor cores rotates its own rows: every thread of its epilogue holds one token's row
        if step.is_decode or self.pairing != "half" or not ops.qkv_rope_ok(h, w_qkv, memory, head_dim, self.rotary_dim):
            return None
        writes = bool(memory.writes and memory.k is not None)
        return ops.gemm_tc_qkv_rope(h, w_qkv, self._table(step), step.positions, step.token_slots, memory.block_table,
                                    memory.k, memory.v, n_heads, n_kv_heads, head_dim, writes)

    def left_to_attention(self, qkv, step, memory, n_heads, n_kv_heads, head_dim):
        # one token per sequence: the decode attention's blocks rotate the heads they read and the newest key
        if self.pairing != "half" or self.rotary_dim < 2 or not ops.attn_rope_inside_ok(qkv, memory, step, head_dim):
            return None
        return self._table(step), self.rotary_dim

    def encode_and_store(self, qkv, step, memory, n_heads, n_kv_heads, head_dim) -> None:
        table = self._table(step)
        ops.rope_cache_write(qkv, table, step.positions, step.token_slots, memory.block_table, memory.k, memory.v,
                             n_heads, n_kv_heads, head_dim, self.rotary_dim,
                             self.pairing == "adjacent", memory.writes and memory.k is not None)
