"""The generation loop above the step function.

One sequence in the reference (src/main.rs:702-786): the prompt must be non-empty and leave room; it is
read in one go; then, while fewer than max_new tokens were generated and the context has room: sample
from the current logits, count the token, stop if it is a stop token (which is neither kept nor fed),
else keep it and feed it.  Here the same happens for batches: requests are taken in order, as many as
`batch_size` and the cache allow; all prompts of a batch run in one step; each following step carries
one token for every sequence still alive; a sequence that ends leaves the batch at once and its slot
goes back when the batch ends, to be used by the next batch.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.pages import PAGE_TOKENS, CacheFullError, pages_for
from .step import StepEntry


@dataclass
class GenerationResult:
    prompt_tokens: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""            # "stop", "length" or "capacity"
    stopped_on: Optional[int] = None


@dataclass
class GenerationStats:
    """The reference's Stats (src/main.rs:587-598), summed over batches."""
    prompt_tokens: int = 0
    prompt_secs: float = 0.0
    gen_tokens: int = 0
    gen_secs: float = 0.0
    batches: int = 0
    steps: int = 0
    # with `time_steps_every` = n: device time per decode step over each stretch of n steps, in milliseconds
    # (CUDA events on the launching stream, read when a batch ends)
    step_ms: List[float] = field(default_factory=list)


class GenerationLoop:
    """`engine` needs `.cache` (open_slot, close_slot, length, free_pages, max_seq_len) and
    `.step(entries) -> logits`; `sampler` needs `.start(n)` and `.pick(logits, request_ids) -> tokens`.
    With `engine.decoder(slots)` (a runner of one-token steps) and `sampler.pick_device` the loop keeps the
    sampled tokens on the device and looks at them one step late; it takes the same decisions either way."""

    def __init__(self, engine, sampler, stop_token_ids: Sequence[int] = (), batch_size: int = 8,
                 on_token: Optional[Callable[[int, int], None]] = None, max_step_tokens: Optional[int] = None,
                 time_steps_every: Optional[int] = None):
        """`max_step_tokens`: the most prompt tokens one step carries; longer batches of prompts are read in
        several steps that attend to the cache (the reference reads prompts in passes of 1024 tokens,
        src/cuda.rs:8550).  None: all prompts of a batch in one step."""
        if batch_size < 1:
            raise ValueError("batch_size must be at least 1")
        if max_step_tokens is not None and max_step_tokens < 1:
            raise ValueError("max_step_tokens must be at least 1")
        self.max_step_tokens = max_step_tokens
        self.time_steps_every = time_steps_every
        self.engine = engine
        self.sampler = sampler
        self.stop = frozenset(int(t) for t in stop_token_ids)
        self.batch_size = batch_size
        self.on_token = on_token
        self.stats = GenerationStats()

    # ---- which requests form the next batch -------------------------------------------------------
    def _admit(self, prompts: Sequence[Sequence[int]], first: int) -> int:
        """How many requests starting at `first` go into the next batch."""
        cache = self.engine.cache
        free = cache.free_pages
        free_slots = cache.slots.free_slots
        n = 0
        for i in range(first, min(len(prompts), first + self.batch_size)):
            need = pages_for(len(prompts[i]) + 1)
            if need > free or n >= free_slots:
                break
            free -= need
            n += 1
        if n == 0:
            raise CacheFullError(
                f"request {first} does not fit: its prompt of {len(prompts[first])} tokens needs "
                f"{pages_for(len(prompts[first]) + 1)} pages of {PAGE_TOKENS} tokens, {cache.free_pages} are free")
        return n

    def run(self, prompts: Sequence[Sequence[int]], max_new: int) -> List[GenerationResult]:
        cache = self.engine.cache
        for i, p in enumerate(prompts):
            if len(p) == 0:
                raise ValueError(f"request {i}: empty prompt")          # src/main.rs:703
            if len(p) >= cache.max_seq_len:
                raise ValueError(f"request {i}: prompt does not fit: {len(p)} tokens >= context {cache.max_seq_len}")  # :706
        results = [GenerationResult(prompt_tokens=len(p)) for p in prompts]
        self.sampler.start(len(prompts))
        first = 0
        while first < len(prompts):
            n = self._admit(prompts, first)
            self._run_batch(prompts, results, list(range(first, first + n)), max_new)
            first += n
        return results

    def _read_prompts(self, prompts, slots, live: List[int]):
        """All prompts of the batch, in one step or in steps of at most `max_step_tokens` tokens; returns the
        logits after each prompt's last token, in the order of `live`."""
        limit = self.max_step_tokens
        if limit is None or sum(len(prompts[i]) for i in live) <= limit:
            self.stats.steps += 1
            return self.engine.step([StepEntry(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live])
        import torch
        fed = {i: 0 for i in live}
        rows = {}
        while any(fed[i] < len(prompts[i]) for i in live):
            budget, entries, owners = limit, [], []
            for i in live:
                left = len(prompts[i]) - fed[i]
                if left == 0 or budget == 0:
                    continue
                n = min(left, budget)
                last = fed[i] + n == len(prompts[i])
                entries.append(StepEntry(slots[i], prompts[i][fed[i]:fed[i] + n], [n - 1] if last else []))
                if last:
                    owners.append(i)
                fed[i] += n
                budget -= n
            out = self.engine.step(entries)
            self.stats.steps += 1
            for r, i in enumerate(owners):
                rows[i] = out[r].clone()
        return torch.stack([rows[i] for i in live])

    def _run_batch(self, prompts, results, ids: List[int], max_new: int) -> None:
        if hasattr(self.engine, "decoder") and hasattr(self.sampler, "pick_device"):
            return self._run_batch_pipelined(prompts, results, ids, max_new)
        return self._run_batch_simple(prompts, results, ids, max_new)

    # ---- tokens stay on the device; the host looks at them one step late ---------------------------------
    def _run_batch_pipelined(self, prompts, results, ids: List[int], max_new: int) -> None:
        """The same decisions as `_run_batch_simple`, but the host is off the critical path: the step that feeds
        token k is launched from the device copy of the sampled tokens, and token k is examined on the host
        (stop tokens, callbacks) while that step runs.  A sequence that turns out to have ended on token k has
        then been stepped once too often: its extra token is dropped and its slot is given back with the batch."""
        import torch
        cache = self.engine.cache
        slots = {i: cache.open_slot() for i in ids}
        self.stats.batches += 1
        finished = {i: False for i in ids}
        n_sampled = {i: 0 for i in ids}
        on_gpu = getattr(self.engine, "device", torch.device("cpu")).type == "cuda"
        pinned = [torch.empty(len(ids), dtype=torch.int32, pin_memory=on_gpu) for _ in range(2)]
        flip = 0

        def to_host(dev_tokens, order):
            nonlocal flip
            buf = pinned[flip][:len(order)]
            flip ^= 1
            buf.copy_(dev_tokens[:len(order)], non_blocking=True)
            ev = None
            if on_gpu:
                ev = torch.cuda.Event()
                ev.record()
            # a token sampled when its sequence already fills the context is not taken: the reference's loop ends
            # on `pos < ctx` before it samples again (src/main.rs:770)
            at_end = {i for i in order if cache.length(slots[i]) >= cache.max_seq_len}
            return buf, ev, list(order), at_end

        def resolve(flight):
            """Host-side decisions on tokens sampled one step ago."""
            buf, ev, order, at_end = flight
            if ev is not None:
                ev.synchronize()
            for i, tok in zip(order, buf.tolist()):
                if finished[i]:
                    continue                                  # ended earlier; this token came from the extra step
                res = results[i]
                if i in at_end:
                    res.finish_reason, finished[i] = "capacity", True
                    continue
                self.stats.gen_tokens += 1
                if tok in self.stop:                          # counted, not kept, not fed (src/main.rs:772-776)
                    res.finish_reason, res.stopped_on, finished[i] = "stop", tok, True
                    continue
                res.tokens.append(tok)
                if self.on_token is not None:
                    self.on_token(i, tok)
                if len(res.tokens) >= max_new:
                    res.finish_reason, finished[i] = "length", True

        def eligible(order):
            return [i for i in order if not finished[i] and n_sampled[i] < max_new
                    and cache.length(slots[i]) + 1 <= cache.max_seq_len]

        runner = None
        marks, n_decode = [], [0]

        def launch(feed, order, cur):
            """One more token for every sequence of `feed`, taken from the device copy of the last picks."""
            nonlocal runner
            if len(feed) == len(order):
                tok_in = cur
            else:
                pos = {i: r for r, i in enumerate(order)}
                # from page-locked memory: a copy from ordinary memory would hold the host until the device has caught up
                rows = torch.tensor([pos[i] for i in feed], dtype=torch.int64, pin_memory=on_gpu).to(cur.device, non_blocking=True)
                tok_in = cur.index_select(0, rows)
            want = [slots[i] for i in feed]
            if runner is None or runner.slots != want:
                runner = self.engine.decoder(want)
            if on_gpu and self.time_steps_every and n_decode[0] % self.time_steps_every == 0:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((n_decode[0], ev))
            n_decode[0] += 1
            logits = runner.forward(dev_tokens=tok_in)
            self.stats.steps += 1
            nxt = self.sampler.pick_device(logits, feed)
            for i in feed:
                n_sampled[i] += 1
            return nxt, to_host(nxt, feed)

        try:
            t0 = time.perf_counter()
            if max_new <= 0:
                for i in ids:
                    results[i].finish_reason = "length"
                return
            order = list(ids)
            logits = self._read_prompts(prompts, slots, order)
            cur = self.sampler.pick_device(logits, order)
            for i in order:
                n_sampled[i] = 1
            flight = to_host(cur, order)
            self.stats.prompt_tokens += sum(len(prompts[i]) for i in order)
            if on_gpu:
                torch.cuda.current_stream().synchronize()
            t1 = time.perf_counter()
            self.stats.prompt_secs += t1 - t0
            while True:
                feed = eligible(order)
                nxt = nxt_flight = None
                resolved = False
                if feed:
                    try:
                        nxt, nxt_flight = launch(feed, order, cur)
                    except CacheFullError:
                        # The pool is full.  The host learns of a sequence's end one step late: learn it now, and try once
                        # more without those that have ended (the loop that decides at once would not have fed them).
                        resolve(flight)
                        resolved = True
                        again = eligible(feed)
                        feed = []
                        if again:
                            try:
                                nxt, nxt_flight = launch(again, order, cur)
                                feed = again
                            except CacheFullError:
                                pass
                if not resolved:
                    resolve(flight)
                for i in order:
                    if not finished[i] and i not in feed:
                        results[i].finish_reason, finished[i] = "capacity", True     # no room to go on (src/main.rs:770)
                if not feed:
                    break
                order, cur, flight = feed, nxt, nxt_flight
            self.stats.gen_secs += time.perf_counter() - t1
            if len(marks) > 1:
                torch.cuda.current_stream().synchronize()
                for (a, ea), (b, eb) in zip(marks, marks[1:]):
                    self.stats.step_ms.append(ea.elapsed_time(eb) / (b - a))
        finally:
            for s in slots.values():
                cache.close_slot(s)

    def _run_batch_simple(self, prompts, results, ids: List[int], max_new: int) -> None:
        cache = self.engine.cache
        slots = {i: cache.open_slot() for i in ids}
        self.stats.batches += 1
        try:
            t0 = time.perf_counter()
            live = list(ids)
            runner = None
            if max_new <= 0:
                for i in live:
                    results[i].finish_reason = "length"
                return
            logits = self._read_prompts(prompts, slots, live)
            picked = self.sampler.pick(logits, live)
            self.stats.prompt_tokens += sum(len(prompts[i]) for i in live)
            t1 = time.perf_counter()
            self.stats.prompt_secs += t1 - t0
            while True:
                feed = []
                for i, tok in zip(live, picked):
                    res = results[i]
                    if cache.length(slots[i]) >= cache.max_seq_len:
                        res.finish_reason = "capacity"        # the reference's `pos < ctx` ends its loop before it samples again (src/main.rs:770)
                        continue
                    self.stats.gen_tokens += 1
                    if tok in self.stop:                      # counted, not kept, not fed (src/main.rs:772-776)
                        res.finish_reason, res.stopped_on = "stop", tok
                        continue
                    res.tokens.append(tok)
                    if self.on_token is not None:
                        self.on_token(i, tok)
                    if len(res.tokens) >= max_new:
                        res.finish_reason = "length"
                    else:
                        feed.append((i, tok))                 # the context has room: checked above
                if not feed:
                    break
                try:
                    if hasattr(self.engine, "decoder"):
                        want = [slots[i] for i, _ in feed]
                        if runner is None or runner.slots != want:
                            runner = self.engine.decoder(want)
                        logits = runner.forward(tokens=[tok for _, tok in feed])
                    else:
                        logits = self.engine.step([StepEntry(slots[i], [tok], [0]) for i, tok in feed])
                except CacheFullError:
                    for i, _ in feed:
                        results[i].finish_reason = "capacity"
                    break
                self.stats.steps += 1
                live = [i for i, _ in feed]
                picked = self.sampler.pick(logits, live)
            self.stats.gen_secs += time.perf_counter() - t1
        finally:
            for s in slots.values():
                cache.close_slot(s)
