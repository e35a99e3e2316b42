"""Next-token selection: greedy, or temperature with top-k and top-p, one generator stream per request.

Options and defaults are the reference's (src/main.rs:57-61, src/sampler.rs:40-42): temperature 0.7
(0 = greedy), top_k 40 (0 = all), top_p 0.9, a seed.  The reference has one xorshift64* stream because
it runs one sequence; here request i of a call draws from its own stream, started at
max(seed + i * 0x9E3779B97F4A7C15 mod 2^64, 1), so that what a request samples does not depend on which
requests share its batch.  Request 0 of a call has exactly the reference's stream for that seed.
The selection itself runs on the device (`kernels.ops.sample`).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..kernels import ops

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    seed: Optional[int] = None     # None: taken from the clock, as the reference does (src/main.rs:128)

    def validate(self) -> None:
        if self.top_k < 0:
            raise ValueError("top_k must not be negative (0 = all tokens)")
        if not (0.0 < self.top_p):
            raise ValueError("top_p must be positive")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


def stream_seed(seed: int, request_index: int) -> int:
    s = (int(seed) + request_index * _GOLDEN) & _MASK
    return max(s, 1)


def _as_i64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


class DeviceSampler:
    """Keeps the generator states of a call's requests on the device and picks tokens there."""

    def __init__(self, params: SamplingParams, device):
        params.validate()
        self.params = params
        self.device = torch.device(device)
        self.seed = params.seed if params.seed is not None else time.time_ns()
        self.states: Optional[torch.Tensor] = None
        self._rows_of: Optional[tuple] = None          # the request ids whose device copy `_rows` holds
        self._rows: Optional[torch.Tensor] = None

    def start(self, n_requests: int) -> None:
        if self.params.greedy:
            self.states = None
            return
        host = torch.tensor([_as_i64(stream_seed(self.seed, i)) for i in range(n_requests)], dtype=torch.int64)
        self.states = host.to(self.device)

    def pick_device(self, logits: torch.Tensor, request_ids: Sequence[int]) -> torch.Tensor:
        """One token for each row of `logits` (row r belongs to request `request_ids[r]`), left on the device
        as int32, so that the next step can be launched before the host has looked at the tokens."""
        p = self.params
        with ops.bucket("sampling"):
            if p.greedy:
                return ops.sample(logits, 0.0, 0, 1.0)
            ids = tuple(request_ids)
            if self._rows_of != ids:        # the same rows step after step until a sequence leaves
                pinned = self.device.type == "cuda"
                self._rows = torch.tensor(ids, dtype=torch.int32, pin_memory=pinned).to(self.device, non_blocking=True)
                self._rows_of = ids
            idx = self._rows
            return ops.sample(logits, p.temperature, p.top_k, p.top_p, self.states, idx)

    def pick(self, logits: torch.Tensor, request_ids: Sequence[int]) -> List[int]:
        """The same, brought to the host."""
        return self.pick_device(logits, request_ids).cpu().tolist()
