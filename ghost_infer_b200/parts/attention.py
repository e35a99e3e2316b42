"""Causal grouped-query attention as a mixer.

Order of operations (src/model.rs:1000-1101): q, k, v = Wq h, Wk h, Wv h (one product over the three
matrices stacked by rows, as the reference's GPU path merges them: src/cuda.rs:7908-7909); position
encoding on q and k; k and v appended to the cache; head h attends with kv head h / (H / KV) over every
cached position up to its own (src/model.rs:1320-1419), scores scaled by `scale` (1/sqrt(head_dim) for
Llama, src/model.rs:271); residual += Wo att.  With `window` = w a query sees only the last w positions.

Tensor names: prefix + "self_attn.{q,k,v,o}_proj.weight" unless `params["tensor_names"]` gives others for the
keys "q", "k", "v", "o".
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import CacheRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .registry import lookup, register


@register("mixer", "gqa_attention")
class GqaAttention(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = params.get("window")
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv} kv heads")
        pos = params["position"]
        self.position = lookup("position", pos.kind)(pos.params, prefix) if pos is not None else None
        self.q_dim = self.n_heads * self.head_dim
        self.kv_dim = self.n_kv * self.head_dim
        self.names = {k: self.tensor_name(k, f"self_attn.{k}_proj.weight") for k in ("q", "k", "v", "o")}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(n["q"], (self.q_dim, self.hidden)), WeightSpec(n["k"], (self.kv_dim, self.hidden)),
                WeightSpec(n["v"], (self.kv_dim, self.hidden)), WeightSpec(n["o"], (self.hidden, self.q_dim))]

    def cache_request(self) -> Optional[CacheRequest]:
        if self.window:
            return CacheRequest("window", self.n_kv, self.head_dim, int(self.window))
        return CacheRequest("full", self.n_kv, self.head_dim)

    @property
    def plans_on_host(self) -> bool:
        return bool(self.position is not None and self.position.plans_on_host)

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None):
        """Into how many slices the decode attention cuts the contexts (the kernels' own rule)."""
        return ops.attn_decode_plan(n_seqs, max_kv_len, sm_count, self.n_heads, self.n_kv, self.head_dim, self.window,
                                    self.rt.dtype, kv_lens)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        q, k, v = (rt.place(tensors[self.names[x]]) for x in ("q", "k", "v"))
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = (t.to(torch.float32) for t in (q, k, v))
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        del q, k, v
        self.w_o = rt.place(tensors[self.names["o"]])
        if self.position is not None:
            self.position.bind(tensors, rt)

    def forward(self, h, residual, step, memory) -> None:
        # in a decode step the product may leave partial sums for the kernel that rotates and stores (it reads
        # every value anyway); an encoding that does not go through that kernel gets plain rows
        qkv = None
        if self.position is not None:
            with ops.bucket("qkv matmul"):
                qkv = self.position.project_and_store(h, self.w_qkv, step, memory, self.n_heads, self.n_kv, self.head_dim)
        if qkv is not None:
            return self._attend(qkv, None, residual, step, memory)
        with ops.bucket("qkv matmul"):
            if self.position is None or getattr(self.position, "settles_pending", False):
                with ops.defer_store():
                    qkv = linear(h, self.w_qkv, out_dtype=self.rt.dtype)
            else:
                qkv = linear(h, self.w_qkv, out_dtype=self.rt.dtype)
        inside = None
        with ops.bucket("rope+cache"):
            if self.position is not None:
                inside = self.position.left_to_attention(qkv, step, memory, self.n_heads, self.n_kv, self.head_dim)
                if inside is None:
                    self.position.encode_and_store(qkv, step, memory, self.n_heads, self.n_kv, self.head_dim)
            else:
                ops.rope_cache_write(qkv, None, step.positions, step.token_slots, memory.block_table, memory.k, memory.v,
                                     self.n_heads, self.n_kv, self.head_dim, 0, False,
                                     memory.writes and memory.k is not None)
        self._attend(qkv, inside, residual, step, memory)

    def _attend(self, qkv, inside, residual, step, memory) -> None:
        with ops.bucket("attention"):
            att = torch.empty((qkv.shape[0], self.q_dim), dtype=self.rt.dtype, device=qkv.device)
            ops.attention(qkv, memory, step, self.n_heads, self.n_kv, self.head_dim, self.scale, self.window, att,
                          plan=step.plan_of(self), rope=inside)
        with ops.bucket("out matmul"):
            linear(att, self.w_o, out=residual, accumulate=True)
