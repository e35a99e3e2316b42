"""What every part is: a class built from its constants, which names its tensors, takes them, and runs.

Interfaces (a new kind of part implements one of them and registers under a name):

* `Norm.forward(x, rows=None) -> h`: x is the float32 residual stream [tokens, width]; h has the
  step's activation dtype.  `rows` (int32, optional) picks the rows to norm.
* `PositionEncoding.encode_and_store(qkv, step, memory, n_heads, n_kv_heads, head_dim)`: changes the
  q and k parts of the packed rows as the encoding wants and writes k and v to the cache.
* `Mixer.forward(h, residual, step, memory)`: adds the mixer's output to `residual` in place.
  `Mixer.cache_request()` / `Mixer.state_request()` say what memory it wants per sequence.
* `FeedForward.forward(h, residual, step)`: adds its output to `residual` in place.
* `Block.forward(x, layer, step, memory)`: runs one layer's parts in its arrangement.

No part knows which model it is in: sizes, constants and tensor names arrive as parameters.
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
    def __init__(self, params: Mapping[str, Any], prefix: str = ""):
        self.params = params
        self.prefix = prefix

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


class Mixer(Part):
    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, h: torch.Tensor, residual: torch.Tensor, step, memory: LayerMemory) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, residual: torch.Tensor, step) -> None:
        raise NotImplementedError


class Block:
    """An arrangement of one layer's parts."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def forward(self, x: torch.Tensor, step, memory: LayerMemory) -> None:
        raise NotImplementedError
