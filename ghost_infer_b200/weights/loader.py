"""Binding weights by tensor name, with one error that says everything that is wrong.

The reference fetches each tensor by name and stops at the first problem ("missing tensor X",
src/model.rs:471-473; "not 2-D", :480-482; a head whose rows do not match the vocabulary,
src/cuda.rs:8015-8017).  Here the whole manifest is checked against the file first, and a single
`WeightsError` lists every missing tensor, every tensor nobody asked for, and every wrong shape.
Floating tensors keep their stored precision here; the runtime decides what they become on the device.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable, List, Mapping, Sequence

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightsError(ValueError):
    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str], wrong: Sequence[str]):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = [f"{where}: the weights do not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shapes or types ({len(self.wrong)}): " + "; ".join(self.wrong))
        super().__init__("\n".join(lines))


def _open_files(model_dir: str) -> List[SafetensorsFile]:
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            shards = sorted(set(json.load(f).get("weight_map", {}).values()))
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json is there")


def load_model_tensors(model_dir: str, manifest: Iterable, ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """CPU tensors (views of the mapped files) for every name in `manifest` (name, shape, init)."""
    files = _open_files(model_dir)
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for n in f.names():
            where[n] = f
    wanted = {w.name: tuple(w.shape) for w in manifest}
    ignorable = set(ignorable)
    missing = [n for n in wanted if n not in where]
    unexpected = sorted(n for n in where if n not in wanted and n not in ignorable)
    wrong = []
    for n, shape in wanted.items():
        if n in where:
            ent = where[n].entries[n]
            if tuple(ent.shape) != shape:
                wrong.append(f"{n} is {list(ent.shape)}, the configuration wants {list(shape)}")
            elif ent.dtype not in ("F32", "BF16", "F16", "F64"):
                wrong.append(f"{n} is stored as {ent.dtype}, not a floating type")
    if missing or unexpected or wrong:
        raise WeightsError(model_dir, missing, unexpected, wrong)
    return {n: where[n].get(n) for n in wanted}
