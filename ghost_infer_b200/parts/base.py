"""What every part is: a class built from its constants, which names its tensors, takes them, and runs.

Interfaces (a new kind of part implements one of them and registers under a name):

* `Norm.forward(x, rows=None) -> h`: x is the float32 residual stream [tokens, width]; h has the
  step's activation dtype.  `rows` (int32, optional) picks the rows to norm.
* `PositionEncoding.encode_and_store(qkv, step, memory, n_heads, n_kv_heads, head_dim)`: changes the
  q and k parts of the packed rows as the encoding wants and writes k and v to the cache.
* `Mixer.forward(h, residual, step, memory)`: adds the mixer's output to `residual` in place.
  `Mixer.cache_request()` / `Mixer.state_request()` say what memory it wants per sequence.
  `Mixer.decode_plan(n_seqs, max_kv_len, sm_count, kv_lens=None)` says how it cuts the work of one-token steps of that shape
  (anything hashable, or None); a recorded step keeps the plan it was recorded with (`step.plan_of(self)`).
* `FeedForward.forward(h, residual, step)`: adds its output to `residual` in place.
* `Block.forward(x, step, memory)`: runs one layer's parts in its arrangement.  A block is built from the usual
  four parts (norm, mixer, norm, feed-forward; any may be None) and the extra parts its specification names.

No part knows which model it is in: sizes, constants and tensor names arrive as parameters (a part's
tensor names are its prefix plus sub-names that `params["tensor_names"]` may replace).

The arrays of a step live on the device; a part that works from them alone can be recorded once and
replayed (generation's one-token steps are).  A part whose `forward` plans in Python from the step's
host-side lists (`step.host_slots`, `step.host_q_lens`, `step.host_pos0`) sets `plans_on_host = True`:
a model with such a part decodes launch by launch instead.  Rows of a recorded step beyond the live
sequences carry slot -1; for them the cache's page table gives the trash page and `memory.state[-1]` is a
trash row, so indexing by the slot arrays needs no special case.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, NamedTuple, Optional, Tuple

import torch

from ..cache.sequence_cache import CacheRequest, LayerMemory, StateRequest


class WeightSpec(NamedTuple):
    name: str                  # full tensor name in the weights file
    shape: Tuple[int, ...]
    init: str = "normal"       # how the random-weights mode fills it: "normal" or "ones"


@dataclass
class Runtime:
    """Where and in which precision a model runs.  `dtype` is the dtype of activations and of the
    cache: torch.bfloat16 (the serving path) or torch.float32 (everything in true 32-bit)."""
    device: torch.device
    dtype: torch.dtype

    def place(self, t: torch.Tensor) -> torch.Tensor:
        """A weight on the device.  32-bit path: everything becomes float32.  bfloat16 path:
        bfloat16 stays, half becomes bfloat16, a tensor stored in 32-bit stays 32-bit."""
        if t.is_floating_point():
            if self.dtype == torch.float32:
                want = torch.float32
            elif t.dtype in (torch.float32, torch.float64):
                want = torch.float32
            else:
                want = torch.bfloat16
        else:
            want = torch.int32
        return t.to(device=self.device, dtype=want).contiguous()


class Part:
    plans_on_host = False      # True: forward() reads the step's host-side lists, so it must run in Python every step

    def __init__(self, params: Mapping[str, Any], prefix: str = ""):
        self.params = params
        self.prefix = prefix

    def tensor_name(self, key: str, default: str) -> str:
        """Full name of the tensor this part calls `key`: the prefix plus `params["tensor_names"][key]`, or plus
        `default` when the specification does not rename it."""
        names = self.params.get("tensor_names") if hasattr(self.params, "get") else None
        return self.prefix + (names.get(key, default) if names else default)

    def weights(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv: torch.Tensor, step, memory: LayerMemory, n_heads: int, n_kv_heads: int,
                         head_dim: int) -> None:
        raise NotImplementedError

    def project_and_store(self, h: torch.Tensor, w_qkv: torch.Tensor, step, memory: LayerMemory, n_heads: int,
                          n_kv_heads: int, head_dim: int) -> Optional[torch.Tensor]:
        """An encoding that can ride in the epilogue of the q/k/v product itself returns the packed rows of
        `h @ w_qkv^T` with its work and the cache write done (queries encoded in place; the keys' and values' columns
        need not hold anything afterwards), and neither the product nor `encode_and_store` is then run for the
        step.  None (the default): product and encoding run as steps of their own."""
        return None

    def left_to_attention(self, qkv: torch.Tensor, step, memory: LayerMemory, n_heads: int, n_kv_heads: int,
                          head_dim: int):
        """An encoding whose work for this step the attention kernel can do on the way (a rotation by a table of
        angles) returns what `ops.attention(..., rope=)` takes, and `encode_and_store` is then not called for the
        step.  None (the default): the encoding runs as a step of its own."""
        return None


class Mixer(Part):
    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None) -> Any:
        """How this mixer cuts the work of a step of `n_seqs` one-token rows over contexts of up to `max_kv_len`
        positions; hashable.  `kv_lens`: the live sequences' lengths where the caller knows them on the host (a plan
        must stay right for any lengths up to `max_kv_len`; the lengths only help to make it a good one).
        None: nothing about it depends on the shape."""
        return None

    def forward(self, h: torch.Tensor, residual: torch.Tensor, step, memory: LayerMemory) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, residual: torch.Tensor, step) -> None:
        raise NotImplementedError


class Block:
    """An arrangement of one layer's parts: the usual four (any of which an arrangement may lack: None) and whatever
    else the layer's specification names (`self.extra[name]`)."""

    def __init__(self, mixer_norm: Optional[Norm] = None, mixer: Optional[Mixer] = None, ffn_norm: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None, **extra: Part):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn
        self.extra = dict(extra)

    def parts(self):
        usual = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None)
        return usual + tuple(self.extra.values())

    def forward(self, x: torch.Tensor, step, memory: LayerMemory) -> None:
        raise NotImplementedError
