"""The data a model is made of: parts with their constants, layers, and the order layers run in.

A model is not a class with a hard-wired layer: it is a `ModelSpec`, and the
engine walks it.  The reference walks its layers with a `match` on per-layer
enum variants inside one loop (src/model.rs:1007-1053, src/model.rs:1113-1170);
here the variants are names in registries (`parts.registry`), so another mixer,
feed-forward, norm or position encoding is a new registered class, and another
architecture is a new function from its configuration to a `ModelSpec`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: the registry name of its kind and its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class ExtraPart:
    """A part of a layer beyond the usual four (a norm after the mixer, a second feed-forward, ...): the block finds it
    as `self.extra[name]`.  `family` is the registry it comes from ("norm", "feed_forward", "position", "mixer": an
    extra mixer gets no cache or state of its own); `prefix` is where its tensors live under the layer's prefix."""
    name: str
    family: str
    spec: PartSpec
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (`block`) and which parts they are.

    `prefix` is where the layer's tensors live in the weights file
    (e.g. "model.layers.3.").  The usual arrangement has a norm before the mixer, the mixer, a norm before the
    feed-forward and the feed-forward; an arrangement that lacks one of them leaves it None, and one that has more
    names them in `extra`.  The registered block class decides what it does with them.
    """
    prefix: str
    block: str
    mixer_norm: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    mixer_norm_prefix: str = "input_layernorm."            # under `prefix`
    ffn_norm_prefix: str = "post_attention_layernorm."     # under `prefix`
    extra: Tuple[ExtraPart, ...] = ()


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers` (a layer may be named by several
    entries: same weights, run again).  Each entry keeps memory of its own (cache rows, state)
    unless `memory_of` names an earlier entry, whose cache it then reads without writing."""
    layer: int
    memory_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    embedding_prefix: str = "model.embed_tokens."
    final_norm_prefix: str = "model.norm."
    head_prefix: str = "lm_head."

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, but there are {len(self.layers)} layers")
            if e.memory_of is not None:
                if not (0 <= e.memory_of < i):
                    raise ValueError(f"schedule entry {i} reads the memory of entry {e.memory_of}, which does not run before it")
                if self.schedule[e.memory_of].memory_of is not None:
                    raise ValueError(f"schedule entry {i} reads the memory of entry {e.memory_of}, which has none of its own")
