"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.

The reference has no such mode (its unit tests build small synthetic matrices from index arithmetic,
src/quant.rs:1424-1435).  Weights are N(0, std) drawn in 32-bit from one seeded CPU generator in
sorted-name order, then rounded to the stored dtype; norm weights are 1 unless `norm_jitter` spreads
them around 1 (tests do that, so that a forgotten norm weight shows).  The folder is the only carrier
of the numbers: whoever wants the same model reads the file.
"""
from __future__ import annotations

import json
import os
from typing import Any, Mapping

import torch

from .safetensors_io import save_safetensors


def random_tensors(manifest, seed: int, dtype: torch.dtype = torch.bfloat16, std: float = 0.02,
                   norm_jitter: float = 0.0):
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out = {}
    for w in sorted(manifest, key=lambda w: w.name):
        if w.init == "ones":
            t = torch.ones(w.shape, dtype=torch.float32)
            if norm_jitter:
                t = t + norm_jitter * torch.randn(w.shape, generator=gen, dtype=torch.float32)
        else:
            t = torch.randn(w.shape, generator=gen, dtype=torch.float32) * std
        out[w.name] = t.to(dtype)
    return out


def write_random_model(model_dir: str, raw_config: Mapping[str, Any], seed: int = 0, dtype: str = "bfloat16",
                       std: float = 0.02, norm_jitter: float = 0.0) -> str:
    from ..engine.model import Model, _dtype_of
    model = Model.from_config_dict(raw_config)
    t_dtype = _dtype_of(dtype)
    os.makedirs(model_dir, exist_ok=True)
    cfg = dict(raw_config)
    cfg["torch_dtype"] = "bfloat16" if t_dtype == torch.bfloat16 else "float32"
    if hasattr(model.config, "model_type"):
        cfg.setdefault("model_type", model.config.model_type)     # other readers of such folders look for it
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    tensors = random_tensors(model.weight_manifest(), seed, t_dtype, std, norm_jitter)
    save_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                     metadata={"format": "pt", "seed": str(seed), "std": str(std)})
    return model_dir
