"""The cache of a batch: a slot per sequence, keys and values per layer, fixed-size state beside them.

What the reference keeps per conversation (src/model.rs:686-728, src/cuda.rs:9826-9870) is kept
here per slot.  Layers with different needs are grouped: every mixer states what it wants
(`CacheRequest`: all keys, or a window of them; row geometry), equal requests share a group, and
each group has its own pages, page tables and storage.  This mirrors the reference sizing
its caches by attention layers only and its state buffers by the other layers
(src/model.rs:240-253, src/model.rs:738-741).  Fixed-size per-sequence state (the reference's
`conv_state`/`ssm_state`, zeroed on reset, src/model.rs:692-695, src/model.rs:772-777) lives in a
`[slot, ...]` tensor per schedule entry that asks for one (with one more row at the end, where the padding
rows of fixed-size launches land); the Llama decoder asks for none.

Storage of a group: K and V, each `[entry, page, kv_head, PAGE_TOKENS, head_dim]`.  One page of
one kv head is a contiguous block, which is what the decode kernel streams.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .pages import PAGE_TOKENS, CacheFullError, PagePool, SlotAllocator, pages_for


@dataclass(frozen=True)
class CacheRequest:
    """What a mixer wants kept per token.  kind "full": every position stays visible;
    kind "window": only the last `window` positions are ever read again."""
    kind: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def __post_init__(self):
        if self.kind not in ("full", "window"):
            raise ValueError(f"unknown cache kind {self.kind!r}")
        if self.kind == "window" and (self.window is None or self.window < 1):
            raise ValueError("a window cache needs a positive window")


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size memory per sequence, zero when the sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerMemory:
    """What one schedule entry sees of the cache during a step."""
    k: Optional[torch.Tensor]             # [page, kv_head, PAGE_TOKENS, head_dim] of this entry, or None
    v: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]   # device int32 [max_slots, max_pages_per_seq] of the entry's group
    window: Optional[int]
    writes: bool                          # False when the entry reads another entry's memory
    state: Optional[torch.Tensor]         # [max_slots + 1, *shape] or None; the last row (slot -1) is for padding rows


class _Group:
    def __init__(self, request: CacheRequest, n_pages: int, max_slots: int, max_pages_per_seq: int,
                 dtype: torch.dtype, device: torch.device):
        self.request = request
        self.entries: List[int] = []
        self.pool = PagePool(n_pages)
        self.pages: Dict[int, List[int]] = {}          # slot -> page numbers by page index (0 = released)
        self.first_live: Dict[int, int] = {}           # slot -> first page index still held
        self.table_host = np.zeros((max_slots, max_pages_per_seq), dtype=np.int32)
        self.table_dev: Optional[torch.Tensor] = None
        self.dirty: Dict[int, Tuple[int, int]] = {}    # slot -> [first, end) page indices not yet on the device
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.dtype = dtype
        self.device = device
        self.n_pages = n_pages

    def allocate(self) -> None:
        r = self.request
        shape = (len(self.entries), self.n_pages + 1, r.num_kv_heads, PAGE_TOKENS, r.head_dim)
        # zero-filled once: rows past a sequence's length are never read, but the padding rows of
        # fixed-size launches read the trash page, which must hold finite numbers
        self.k = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.v = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.table_dev = torch.zeros(self.table_host.shape, dtype=torch.int32, device=self.device)


class SequenceCache:
    def __init__(self, requests: Sequence[Tuple[int, Optional[CacheRequest], Optional[StateRequest], Optional[int]]],
                 *, max_tokens: int, max_slots: int, max_seq_len: int, dtype: torch.dtype,
                 device: torch.device | str = "cpu"):
        """`requests`: one tuple per schedule entry: (entry index, cache request or None,
        state request or None, memory_of or None)."""
        if max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_tokens = int(max_tokens)
        self.n_pages = pages_for(max_tokens)
        # a sequence whose every position stays cached cannot be longer than the pool; one that only keeps windows can
        keeps_all = any(creq is not None and creq.kind == "full" and memory_of is None for _, creq, _, memory_of in requests)
        self.max_seq_len = int(min(max_seq_len, self.n_pages * PAGE_TOKENS)) if keeps_all else int(max_seq_len)
        self.max_pages_per_seq = pages_for(self.max_seq_len)
        self.slots = SlotAllocator(max_slots)
        self.max_slots = max_slots
        self.lengths = [0] * max_slots
        self._groups: List[_Group] = []
        self._group_of_entry: Dict[int, Tuple[_Group, int]] = {}
        self._reads_from: Dict[int, int] = {}
        self._state: Dict[int, torch.Tensor] = {}
        by_request: Dict[CacheRequest, _Group] = {}
        for entry, creq, sreq, memory_of in requests:
            if memory_of is not None:
                self._reads_from[entry] = memory_of
                continue
            if creq is not None:
                g = by_request.get(creq)
                if g is None:
                    g = _Group(creq, self.n_pages, max_slots, self.max_pages_per_seq, dtype, self.device)
                    by_request[creq] = g
                    self._groups.append(g)
                self._group_of_entry[entry] = (g, len(g.entries))
                g.entries.append(entry)
            if sreq is not None:
                # one row more than there are slots: padding rows of a fixed-size launch carry slot -1, which
                # indexes this last row, as they write keys and values to the trash page
                self._state[entry] = torch.zeros((max_slots + 1,) + tuple(sreq.shape), dtype=sreq.dtype, device=self.device)
        for g in self._groups:
            g.allocate()

    # ---- sizes ------------------------------------------------------------------------------
    def bytes_per_token(self) -> int:
        total = 0
        esz = torch.empty((), dtype=self.dtype).element_size()
        for g in self._groups:
            total += 2 * len(g.entries) * g.request.num_kv_heads * g.request.head_dim * esz
        return total

    def state_bytes_per_sequence(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self._state.values())

    @property
    def free_pages(self) -> int:
        return min((g.pool.free_pages for g in self._groups), default=self.n_pages)

    @property
    def groups(self) -> List[_Group]:
        return self._groups

    # ---- slots ------------------------------------------------------------------------------
    def open_slot(self) -> int:
        s = self.slots.take()
        self.lengths[s] = 0
        for g in self._groups:
            g.pages[s] = []
            g.first_live[s] = 0
        for t in self._state.values():
            t[s].zero_()
        return s

    def close_slot(self, slot: int) -> None:
        if not self.slots.live(slot):
            raise RuntimeError(f"slot {slot} is closed but not open")
        for g in self._groups:
            held = [p for p in g.pages.pop(slot) if p != PagePool.TRASH_PAGE]
            g.pool.give_back(held)
            g.first_live.pop(slot, None)
            g.table_host[slot, :] = 0
            g.dirty.pop(slot, None)      # a closed slot's row is never read; it is rewritten when pages come
        self.lengths[slot] = 0
        self.slots.give_back(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    def reserve(self, wanted: Sequence[Tuple[int, int]]) -> None:
        """Pages for every (slot, new length) pair, in every group; all or nothing."""
        for slot, new_len in wanted:
            if not self.slots.live(slot):
                raise RuntimeError(f"slot {slot} is not open")
            if new_len > self.max_seq_len:
                raise CacheFullError(f"context full ({self.max_seq_len} tokens): slot {slot} would hold {new_len}")
        for g in self._groups:
            need = sum(max(0, pages_for(n) - len(g.pages[s])) for s, n in wanted)
            if need > g.pool.free_pages:
                raise CacheFullError(
                    f"the cache is full: {need} more pages of {PAGE_TOKENS} tokens wanted, {g.pool.free_pages} of {g.pool.n_pages} free")
        for g in self._groups:
            for s, n in wanted:
                have = len(g.pages[s])
                more = pages_for(n) - have
                if more > 0:
                    new = g.pool.take(more)
                    g.pages[s].extend(new)
                    g.table_host[s, have:have + more] = new
                    lo, hi = g.dirty.get(s, (have, have))
                    g.dirty[s] = (min(lo, have), max(hi, have + more))

    def commit(self, slot: int, new_len: int) -> None:
        """The slot now holds `new_len` tokens.  Window groups give back pages no later query can see."""
        self.lengths[slot] = new_len
        for g in self._groups:
            if g.request.kind != "window":
                continue
            # a query at position p >= new_len reads keys > p - window >= new_len - window
            dead_before = max(0, new_len - g.request.window + 1) // PAGE_TOKENS
            first = g.first_live[slot]
            if dead_before > first:
                pages = g.pages[slot]
                g.pool.give_back([pages[i] for i in range(first, dead_before)])
                for i in range(first, dead_before):
                    pages[i] = PagePool.TRASH_PAGE
                g.table_host[slot, first:dead_before] = 0    # never read again: the device copy may keep them
                g.first_live[slot] = dead_before

    def reset(self, slot: int) -> None:
        """The slot starts over: no tokens, pages given back, fixed-size state zero (src/model.rs:772-777)."""
        if not self.slots.live(slot):
            raise RuntimeError(f"slot {slot} is not open")
        for g in self._groups:
            held = [p for p in g.pages[slot] if p != PagePool.TRASH_PAGE]
            g.pool.give_back(held)
            g.pages[slot] = []
            g.first_live[slot] = 0
            g.table_host[slot, :] = 0
            g.dirty.pop(slot, None)
        for t in self._state.values():
            t[slot].zero_()
        self.lengths[slot] = 0

    def truncate(self, slot: int, pos: int) -> int:
        """Rewinds a slot to `pos` tokens (src/model.rs:799-821: lowering the position is enough for
        attention caches).  Returns the length actually reached: fixed-size state and released window
        pages cannot be rewound, so with those the slot stays where it is."""
        cur = self.lengths[slot]
        if pos >= cur:
            return cur
        if self._state or any(g.request.kind == "window" and g.first_live[slot] * PAGE_TOKENS > 0 for g in self._groups):
            return cur
        for g in self._groups:
            keep = pages_for(pos)
            pages = g.pages[slot]
            if len(pages) > keep:
                g.pool.give_back(pages[keep:])
                g.table_host[slot, keep:len(pages)] = 0
                del pages[keep:]
        self.lengths[slot] = pos
        return pos

    # ---- device side ------------------------------------------------------------------------
    def sync_tables(self) -> None:
        """Copies the changed stretches of the page tables to the device, on the stream of the kernels
        that read them.  Only rows that gained pages since the last call are touched.

        The host does not wait: the stretches are first copied into page-locked staging memory of this call's own
        (a copy from ordinary memory would hold the host until everything queued on the stream has run, one whole step
        in a decode loop that otherwise runs ahead of the device), and go to the device from there in stream order.
        The staging memory is handed back to torch's allocator, which reuses it only after those copies ran; the
        host's own table may change again at once (a slot closed, a page taken) without touching what is under way."""
        on_gpu = self.device.type == "cuda"
        for g in self._groups:
            if not g.dirty:
                continue
            if not on_gpu:
                for slot, (lo, hi) in g.dirty.items():
                    g.table_dev[slot, lo:hi].copy_(torch.from_numpy(g.table_host[slot, lo:hi]))
                g.dirty.clear()
                continue
            stretches = [(slot, lo, hi) for slot, (lo, hi) in g.dirty.items() if hi > lo]
            total = sum(hi - lo for _, lo, hi in stretches)
            if total:
                stage = torch.empty((total,), dtype=torch.int32, pin_memory=True)
                view = stage.numpy()
                at = 0
                for slot, lo, hi in stretches:
                    view[at:at + hi - lo] = g.table_host[slot, lo:hi]
                    g.table_dev[slot, lo:hi].copy_(stage[at:at + hi - lo], non_blocking=True)
                    at += hi - lo
            g.dirty.clear()

    def memory(self, entry: int) -> LayerMemory:
        src = self._reads_from.get(entry, entry)
        writes = entry not in self._reads_from
        gi = self._group_of_entry.get(src)
        state = self._state.get(src)
        if gi is None:
            return LayerMemory(None, None, None, None, writes, state)
        g, idx = gi
        return LayerMemory(g.k[idx], g.v[idx], g.table_dev, g.request.window if g.request.kind == "window" else None,
                           writes, state)
