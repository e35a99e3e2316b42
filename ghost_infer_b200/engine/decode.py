"""Decode steps of a fixed set of sequences: one token each, replayed from a CUDA graph.

The reference captures its whole one-token step in a CUDA graph on a session's first step and replays it
afterwards; kernels read the position from device memory and attention uses a fixed split grid so that
one graph fits every position (src/cuda.rs:8690-8711, :8494-8495).  The same is done here for a batch:
tokens, positions, slots and lengths live in a device buffer that one small host-to-device copy refreshes
per step; the graph holds embedding, the layers, the final norm and the head.  A graph is kept per
(rows, what each mixer plans for that many rows and that length bucket); rows beyond the live sequences are
padding with slot -1: they write to the cache's trash page and to the trash row of per-sequence state, and
change no live row.  Sampling runs after the replay, so one graph serves every sampling setting.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .step import StepContext

_ROW_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512, 768, 1024)


def _bucket_rows(n: int) -> int:
    for b in _ROW_BUCKETS:
        if n <= b:
            return b
    return ((n + 255) // 256) * 256


def _bucket_len(n: int) -> int:
    b = 256
    while b < n:
        b *= 2
    return b


class _DecodeGraph:
    """Device buffers of one (rows, mixers' plans) shape and, once captured, the graph over them."""

    def __init__(self, engine, rows: int, plans: dict, replayed: bool):
        dev = engine.device
        self.rows, self.plans = rows, plans
        # [tokens | positions | token_slots | seq_lens] then the fixed [cu_seqlens | logit_rows]
        self.meta = torch.zeros(4 * rows, dtype=torch.int32, device=dev)
        fixed = np.concatenate([np.arange(rows + 1, dtype=np.int32), np.arange(rows, dtype=np.int32)])
        self.fixed = torch.from_numpy(fixed).to(dev)
        self.host = torch.zeros(4 * rows, dtype=torch.int32, pin_memory=True)
        self.host_event: Optional[torch.cuda.Event] = None
        ctx = StepContext()
        ctx.n_tokens = ctx.n_seqs = rows
        ctx.max_q_len = 1
        ctx.is_decode = True
        ctx.tokens = self.meta[0:rows]
        ctx.positions = self.meta[rows:2 * rows]
        ctx.token_slots = self.meta[2 * rows:3 * rows]
        ctx.seq_slots = ctx.token_slots
        ctx.seq_pos0 = ctx.positions
        ctx.seq_lens = self.meta[3 * rows:4 * rows]
        ctx.cu_seqlens = self.fixed[0:rows + 1]
        ctx.logit_rows = self.fixed[rows + 1:]
        ctx.empty_f32 = engine._empty_f32
        ctx.sm_count = engine._sm_count
        ctx.fixed_plans = plans
        if replayed:
            ctx._host_q_lens = ctx._host_slots = ctx._host_pos0 = None    # Python is not run again on replay
        self.ctx = ctx
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.warm = False
        self.launches = 0


class DecodeRunner:
    def __init__(self, engine, slots: Sequence[int], use_graph: bool = True):
        self.engine = engine
        self.cache = engine.cache
        self.slots = list(slots)
        self.n = len(self.slots)
        if self.n == 0:
            raise ValueError("a decode runner needs at least one sequence")
        # a model with a part that plans its work in Python per step cannot be replayed: it decodes launch by
        # launch, with exactly the live rows and the host-side lists filled in
        from ..kernels import ops
        self.use_graph = use_graph and engine.device.type == "cuda" and not engine.plans_on_host and not ops.profiling()
        self.rows = _bucket_rows(self.n) if self.use_graph else self.n
        self._g: Optional[_DecodeGraph] = None
        self._plans: Dict[int, dict] = {}

    def _graph_for(self, lens: Sequence[int]) -> _DecodeGraph:
        """The recording for these rows and this length bucket.  The mixers' plans are asked for once per bucket, with
        the lengths the sequences have then; they hold until a sequence outgrows the bucket."""
        eng = self.engine
        bucket = _bucket_len(max(lens) + 1)
        plans = self._plans.get(bucket)
        if plans is None:
            plans = self._plans[bucket] = eng.decode_plans(self.rows, bucket, [n + 1 for n in lens])
        key = (self.rows, self.use_graph, tuple(repr(plans[id(m)]) for m in eng._mixers))
        g = eng._decode_graphs.get(key)
        if g is None:
            g = _DecodeGraph(eng, self.rows, plans, self.use_graph)
            eng._decode_graphs[key] = g
        return g

    def launches_per_step(self) -> int:
        return self._g.launches if self._g is not None else 0

    def forward(self, tokens: Optional[Sequence[int]] = None, dev_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per sequence, from the host (`tokens`) or already on the device (`dev_tokens`, int32).
        Returns float32 logits [sequences, vocab] on the device (a view of a buffer the next call reuses)."""
        from ..kernels import ops
        cache, n, rows = self.cache, self.n, self.rows
        lens = [cache.length(s) for s in self.slots]
        cache.reserve([(s, l + 1) for s, l in zip(self.slots, lens)])
        cache.sync_tables()
        g = self._graph_for(lens)
        self._g = g
        if g.host_event is not None:
            g.host_event.synchronize()
        h = g.host.numpy()
        h[:] = 0
        if tokens is not None:
            toks = np.asarray(tokens, dtype=np.int32)
            if toks.shape != (n,) or toks.min() < 0 or toks.max() >= self.engine.vocab:
                raise ValueError(f"decode step: {n} token ids inside the vocabulary ({self.engine.vocab}) are wanted")
            h[0:n] = toks
        h[rows:rows + n] = lens
        h[2 * rows:2 * rows + n] = self.slots
        h[2 * rows + n:3 * rows] = -1                 # padding rows: the trash page
        h[3 * rows:3 * rows + n] = np.asarray(lens, dtype=np.int32) + 1
        h[3 * rows + n:4 * rows] = 1
        if tokens is not None:
            g.meta.copy_(g.host, non_blocking=True)
        else:
            g.meta[rows:].copy_(g.host[rows:], non_blocking=True)
            g.meta[0:n].copy_(dev_tokens[0:n])
        ev = torch.cuda.Event()
        ev.record()
        g.host_event = ev
        self.engine.bytes_h2d = g.host.numel() * 4
        g.ctx.max_kv_len = max(lens) + 1
        if not self.use_graph:
            g.ctx._host_q_lens, g.ctx._host_slots, g.ctx._host_pos0 = [1] * n, list(self.slots), list(lens)
        if g.graph is None:
            g.ctx.shared.clear()                       # per-step tables are made anew (inside the graph once captured)
        if not self.use_graph:
            l0 = ops.launches
            g.logits = self.engine.forward(g.ctx)
            g.launches = ops.launches - l0
        elif not g.warm:
            l0 = ops.launches
            g.logits = self.engine.forward(g.ctx)      # an eager step first: settles lazy set-up outside capture
            g.launches = ops.launches - l0
            g.warm = True
        else:
            if g.graph is None:
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    g.logits = self.engine.forward(g.ctx)
                g.graph = graph
            g.graph.replay()
            ops.launches += g.launches
        for s, l in zip(self.slots, lens):
            cache.commit(s, l + 1)
        return g.logits[0:n]
