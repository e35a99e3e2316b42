"""The step function: a batch of sequences, the tokens each brings, logits at the wanted places.

The reference's surface is `prefill(ids)`, `step(id)`, `logits()` for its one sequence
(src/main.rs:455-478); its GPU forward takes n tokens at positions pos..pos+n, causal among themselves
and over the cache, and returns logits for the last row or for all (src/cuda.rs:8636-8751, :9807-9817).
Here one call takes several sequences at once: each entry names a slot of the cache, the next tokens of
that sequence (a whole prompt, a chunk of one, or one decoded token) and the places among them whose
logits are wanted.  Positions follow from the slot's length.  Only the tokens given are run, as one flat
batch `[total tokens]` with per-sequence offsets; nothing is padded, so padding cannot change a result.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.sequence_cache import SequenceCache


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among `tokens` whose logits are asked for


class StepContext:
    """What the parts see of a step: flat per-token and per-sequence index arrays on the device."""

    def __init__(self):
        self.n_tokens = 0
        self.n_seqs = 0
        self.max_q_len = 0
        self.max_kv_len = 0
        self.is_decode = False
        self.tokens: torch.Tensor = None        # int32 [T]
        self.positions: torch.Tensor = None     # int32 [T] position of each token in its sequence
        self.token_slots: torch.Tensor = None   # int32 [T] slot of each token's sequence (-1: a padding row)
        self.cu_seqlens: torch.Tensor = None    # int32 [B + 1] offsets of the sequences' tokens
        self.seq_slots: torch.Tensor = None     # int32 [B] (-1: a padding row)
        self.seq_pos0: torch.Tensor = None      # int32 [B] cached length before the step
        self.seq_lens: torch.Tensor = None      # int32 [B] cached length after the step
        self.logit_rows: Optional[torch.Tensor] = None   # int32 [R] flat token indices
        self.empty_f32: torch.Tensor = None
        self.shared: dict = {}                  # what parts compute once per step and share (e.g. rotary angles)
        self.sm_count = 148
        # A step whose launches are recorded once and replayed (a CUDA graph) keeps the plans it was recorded
        # with: id(mixer) -> what the mixer's `decode_plan` returned for the recording's shape.
        self.fixed_plans: Optional[Dict[int, Any]] = None
        # the same facts on the host, for parts that plan their work there (see `Part.plans_on_host`)
        self._host_q_lens: Optional[List[int]] = []
        self._host_slots: Optional[List[int]] = []
        self._host_pos0: Optional[List[int]] = []

    def plan_of(self, mixer) -> Any:
        """The mixer's plan for this step: the recorded one in a replayed step, else worked out for the step."""
        if self.fixed_plans is not None and id(mixer) in self.fixed_plans:
            return self.fixed_plans[id(mixer)]
        if not self.is_decode:
            return None
        lens = None
        if self._host_pos0 is not None and len(self._host_pos0) == self.n_seqs:
            lens = [p + n for p, n in zip(self._host_pos0, self._host_q_lens)]
        return mixer.decode_plan(self.n_seqs, self.max_kv_len, self.sm_count, lens)

    def _host(self, name: str):
        v = getattr(self, name)
        if v is None:
            raise RuntimeError(
                "this step is recorded once and replayed (a CUDA graph): Python that reads the step's host-side lists "
                "would not run again.  A part that plans on the host sets `plans_on_host = True`; its model then "
                "decodes without a graph")
        return v

    @property
    def host_q_lens(self) -> List[int]:
        return self._host("_host_q_lens")

    @property
    def host_slots(self) -> List[int]:
        return self._host("_host_slots")

    @property
    def host_pos0(self) -> List[int]:
        return self._host("_host_pos0")


class _Staging:
    """A small ring of pinned host buffers for the step's index arrays: one host-to-device copy per step."""

    def __init__(self, device: torch.device, depth: int = 4):
        self.device = device
        self.depth = depth
        self.bufs: List[Optional[torch.Tensor]] = [None] * depth
        self.events: List[Optional[torch.cuda.Event]] = [None] * depth
        self.i = 0

    def upload(self, arr: np.ndarray) -> torch.Tensor:
        n = arr.size
        k = self.i
        self.i = (self.i + 1) % self.depth
        if self.events[k] is not None:
            self.events[k].synchronize()
        if self.bufs[k] is None or self.bufs[k].numel() < n:
            self.bufs[k] = torch.empty((max(1024, 2 * n),), dtype=torch.int32, pin_memory=True)
        host = self.bufs[k][:n]
        host.numpy()[:] = arr
        dev = host.to(self.device, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[k] = ev
        return dev


class Engine:
    """A bound model and a cache; `step` runs tokens through them."""

    def __init__(self, model, cache: SequenceCache):
        if model.rt is None:
            raise RuntimeError("the model has no weights yet")
        self.model = model
        self.cache = cache
        self.device = model.rt.device
        self.vocab = model.spec.vocab_size
        self._staging = _Staging(self.device) if self.device.type == "cuda" else None
        self._empty_f32 = torch.empty((0,), dtype=torch.float32, device=self.device)
        self._sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 148
        self.bytes_h2d = 0
        self._decode_graphs = {}
        # the mixers in the order they run (a layer named twice appears once: its plan is the same both times)
        self._mixers = []
        layers = getattr(model, "layers", [])
        for e in getattr(model.spec, "schedule", ()):
            m = layers[e.layer].block.mixer
            if m is not None and all(m is not seen for seen in self._mixers):
                self._mixers.append(m)
        parts = [getattr(model, n, None) for n in ("embedding", "final_norm", "head")] + [p for layer in layers for p in layer.block.parts()]
        self.plans_on_host = any(getattr(p, "plans_on_host", False) for p in parts)

    # ---- host-side checks, before anything is launched (src/model.rs:974-982) -------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.live(e.slot):
                raise ValueError(f"slot {e.slot} is not open")
            if len(e.tokens) == 0:
                raise ValueError(f"slot {e.slot}: a step entry needs at least one token")
            ids = np.asarray(e.tokens)
            if ids.ndim != 1 or ids.dtype.kind not in "iu":
                raise ValueError(f"slot {e.slot}: tokens must be a flat list of integers")
            bad = (ids < 0) | (ids >= self.vocab)
            if bad.any():
                raise ValueError(f"token id {int(ids[bad][0])} is outside the vocabulary ({self.vocab})")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise ValueError(f"slot {e.slot}: wanted place {w} is outside this step's {len(e.tokens)} tokens")

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        B = len(entries)
        lens = [len(e.tokens) for e in entries]
        T = sum(lens)
        R = sum(len(e.want) for e in entries)
        pos0 = [self.cache.length(e.slot) for e in entries]
        packed = np.empty(3 * T + (B + 1) + 3 * B + R, dtype=np.int32)
        tokens, positions, token_slots = packed[0:T], packed[T:2 * T], packed[2 * T:3 * T]
        o = 3 * T
        cu = packed[o:o + B + 1]; o += B + 1
        seq_slots = packed[o:o + B]; o += B
        seq_pos0 = packed[o:o + B]; o += B
        seq_lens = packed[o:o + B]; o += B
        rows = packed[o:o + R]
        t = r = 0
        cu[0] = 0
        for i, e in enumerate(entries):
            n = lens[i]
            tokens[t:t + n] = np.asarray(e.tokens, dtype=np.int32)
            positions[t:t + n] = np.arange(pos0[i], pos0[i] + n, dtype=np.int32)
            token_slots[t:t + n] = e.slot
            for w in e.want:
                rows[r] = t + int(w)
                r += 1
            t += n
            cu[i + 1] = t
            seq_slots[i] = e.slot
            seq_pos0[i] = pos0[i]
            seq_lens[i] = pos0[i] + n
        if self._staging is not None:
            dev = self._staging.upload(packed)
        else:
            dev = torch.from_numpy(packed.copy()).to(self.device)
        self.bytes_h2d = packed.nbytes
        ctx = StepContext()
        ctx.n_tokens, ctx.n_seqs = T, B
        ctx.max_q_len = max(lens)
        ctx.max_kv_len = max(p + n for p, n in zip(pos0, lens))
        ctx.is_decode = ctx.max_q_len == 1
        ctx.tokens, ctx.positions, ctx.token_slots = dev[0:T], dev[T:2 * T], dev[2 * T:3 * T]
        o = 3 * T
        ctx.cu_seqlens = dev[o:o + B + 1]; o += B + 1
        ctx.seq_slots = dev[o:o + B]; o += B
        ctx.seq_pos0 = dev[o:o + B]; o += B
        ctx.seq_lens = dev[o:o + B]; o += B
        ctx.logit_rows = dev[o:o + R] if R else None
        ctx.empty_f32 = self._empty_f32
        ctx.sm_count = self._sm_count
        ctx._host_q_lens, ctx._host_slots, ctx._host_pos0 = lens, [e.slot for e in entries], pos0
        return ctx

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The model over the tokens of `ctx`: embedding, the scheduled layers, then final norm and head on
        the wanted rows only (src/model.rs:1173-1188)."""
        from ..kernels import ops
        model = self.model
        # the residual stream: a tensor that a deferred product may leave partial sums for (they travel with it)
        x = ops.as_carrier(model.embedding.forward(ctx.tokens))
        for i, e in enumerate(model.spec.schedule):
            model.layers[e.layer].block.forward(x, ctx, self.cache.memory(i))
        if ctx.logit_rows is None:
            ops.drop_pending(x)
            return None
        if not getattr(model.final_norm, "settles_pending", False):
            ops.settle(x)
        h = model.final_norm.forward(x, rows=ctx.logit_rows)
        ops.drop_pending(x)
        return model.head.forward(h)

    def decode_plans(self, n_seqs: int, max_kv_len: int, kv_lens=None) -> Dict[int, Any]:
        """What every mixer plans for one-token steps of this shape: id(mixer) -> plan.  A recorded step is keyed
        by these plans, so a mixer decides itself how its work is cut and when a new recording is needed."""
        return {id(m): m.decode_plan(n_seqs, max_kv_len, self._sm_count, kv_lens) for m in self._mixers}

    def decoder(self, slots: Sequence[int], use_graph: bool = True):
        """A runner of one-token steps for these slots (see engine.decode.DecodeRunner)."""
        from .decode import DecodeRunner
        return DecodeRunner(self, slots, use_graph=use_graph)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the entries' tokens after what their slots hold.  Returns float32 logits
        [wanted places, vocab] on the device, in the order of the entries and of their `want`, or None."""
        self._validate(entries)
        new_lens = [(e.slot, self.cache.length(e.slot) + len(e.tokens)) for e in entries]
        self.cache.reserve(new_lens)          # raises before any launch if the cache cannot hold the step
        self.cache.sync_tables()
        ctx = self.build_context(entries)
        logits = self.forward(ctx)
        for slot, n in new_lens:
            self.cache.commit(slot, n)
        return logits
