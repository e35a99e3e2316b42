"""A model: parts built from a `ModelSpec`, bound to weights, walked by the step function.

The reference's `Model` holds the embedding, a vector of layers, the final norm and the output matrix,
bound by tensor name at load (src/model.rs:372-380, :588-644).  Here the same things are built from
data: each layer's parts come out of the registries by the kinds its `LayerSpec` names, and the
order of running is `spec.schedule`.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..cache.sequence_cache import SequenceCache
from ..config import registry as arch_registry
from ..parts import Runtime, WeightSpec, lookup
from ..parts.spec import ModelSpec
from ..weights.loader import load_model_tensors


def _dtype_of(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype {name} is not supported (bfloat16 or float32)")
        return name
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
             "f32": torch.float32}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype \"{name}\" is not supported (bfloat16 or float32)") from None


class Layer:
    def __init__(self, spec, index: int):
        self.spec = spec
        self.index = index
        p = spec.prefix

        def build(family, part, prefix):
            return None if part is None else lookup(family, part.kind)(part.params, prefix)

        mixer_norm = build("norm", spec.mixer_norm, p + spec.mixer_norm_prefix)
        mixer = build("mixer", spec.mixer, p)
        ffn_norm = build("norm", spec.ffn_norm, p + spec.ffn_norm_prefix)
        ffn = build("feed_forward", spec.ffn, p)
        extra = {e.name: build(e.family, e.spec, p + e.prefix) for e in getattr(spec, "extra", ())}
        if mixer_norm is None and mixer is None and ffn_norm is None and ffn is None and not extra:
            raise ValueError(f"layer {index} has no parts")
        self.block = lookup("block", spec.block)(mixer_norm, mixer, ffn_norm, ffn, **extra)

    def weights(self) -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.block.parts():
            out.extend(part.weights())
        return out

    def bind(self, tensors, rt) -> None:
        for part in self.block.parts():
            part.bind(tensors, rt)


class Model:
    """Parts of one model, not yet or already bound to weights."""

    def __init__(self, spec: ModelSpec, config: Any = None):
        spec.validate()
        self.spec = spec
        self.config = config
        self.embedding = lookup("embedding", spec.embedding.kind)(spec.embedding.params, spec.embedding_prefix)
        self.layers = [Layer(ls, i) for i, ls in enumerate(spec.layers)]
        self.final_norm = lookup("norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm_prefix)
        self.head = lookup("head", spec.head.kind)(spec.head.params, spec.head_prefix)
        self.rt: Optional[Runtime] = None

    # ---- weights ------------------------------------------------------------------------------
    def weight_manifest(self) -> List[WeightSpec]:
        out = list(self.embedding.weights())
        for layer in self.layers:
            out.extend(layer.weights())
        out.extend(self.final_norm.weights())
        out.extend(self.head.weights())
        seen = set()
        for w in out:
            if w.name in seen:
                raise ValueError(f"two parts claim the tensor \"{w.name}\"")
            seen.add(w.name)
        return out

    def ignorable_tensors(self) -> List[str]:
        return list(self.head.ignorable()) if hasattr(self.head, "ignorable") else []

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device="cuda") -> "Model":
        self.rt = Runtime(torch.device(device), _dtype_of(dtype))
        self.embedding.bind(tensors, self.rt)
        for layer in self.layers:
            layer.bind(tensors, self.rt)
        self.final_norm.bind(tensors, self.rt)
        self.head.bind(tensors, self.rt, self.embedding)
        return self

    # ---- memory -------------------------------------------------------------------------------
    def memory_requests(self):
        out = []
        for i, e in enumerate(self.spec.schedule):
            mixer = self.layers[e.layer].block.mixer
            if mixer is None:                                  # a layer without a mixer keeps nothing per sequence
                out.append((i, None, None, e.memory_of))
            else:
                out.append((i, mixer.cache_request(), mixer.state_request(), e.memory_of))
        return out

    def new_cache(self, max_tokens: int, max_slots: Optional[int] = None, max_seq_len: Optional[int] = None,
                  beyond_trained_positions: bool = False) -> SequenceCache:
        """A cache for at most `max_tokens` live tokens (each sequence's count rounded up to whole pages).
        A sequence holds at most `max_seq_len` tokens, and never more than the model's own `max_positions`:
        a larger value is lowered to it with a warning, as the reference clamps its context to the model's
        (`ctx.min(max_ctx)`, src/model.rs:732), unless `beyond_trained_positions` asks to run past them."""
        if self.rt is None:
            raise RuntimeError("the model has no weights yet: bind it first")
        from ..cache.pages import pages_for
        n_pages = pages_for(max_tokens)
        if max_slots is None:
            max_slots = max(1, min(n_pages, 4096))
        if max_seq_len is None:
            max_seq_len = self.spec.max_positions
        elif max_seq_len > self.spec.max_positions and not beyond_trained_positions:
            import warnings
            warnings.warn(f"max_seq_len {max_seq_len} is beyond the model's {self.spec.max_positions} positions and is "
                          f"lowered to them (beyond_trained_positions=True runs past them)", stacklevel=2)
            max_seq_len = self.spec.max_positions
        return SequenceCache(self.memory_requests(), max_tokens=max_tokens, max_slots=max_slots,
                             max_seq_len=max_seq_len, dtype=self.rt.dtype, device=self.rt.device)

    # ---- construction ---------------------------------------------------------------------------
    @classmethod
    def from_config_dict(cls, raw: Mapping[str, Any]) -> "Model":
        arch = arch_registry.get_architecture(arch_registry.architecture_of(raw))
        cfg = arch.parse_config(raw)
        return cls(arch.build_spec(cfg), cfg)

    @classmethod
    def from_pretrained(cls, model_dir: str, dtype="bfloat16", device="cuda") -> "Model":
        """Reads config.json and the safetensors weights of `model_dir`; the model class follows
        config.json's `architectures`."""
        raw = arch_registry.read_config_json(model_dir)
        model = cls.from_config_dict(raw)
        tensors = load_model_tensors(model_dir, model.weight_manifest(), model.ignorable_tensors())
        return model.bind(tensors, dtype, device)

    @classmethod
    def random(cls, raw_config: Mapping[str, Any], seed: int = 0, dtype="bfloat16", device="cuda",
               std: float = 0.02) -> "Model":
        """Random weights made directly on the device (for sizes not worth writing to disk)."""
        model = cls.from_config_dict(raw_config)
        rt_dtype = _dtype_of(dtype)
        gen = torch.Generator(device=device)
        gen.manual_seed(int(seed))
        tensors: Dict[str, torch.Tensor] = {}
        for w in model.weight_manifest():
            if w.init == "ones":
                tensors[w.name] = torch.ones(w.shape, dtype=rt_dtype, device=device)
            else:
                t = torch.empty(w.shape, dtype=rt_dtype, device=device)
                t.normal_(0.0, std, generator=gen)
                tensors[w.name] = t
        return model.bind(tensors, dtype, device)
