"""Reading and writing safetensors files, by tensor name.

File layout: an 8-byte little-endian header length, a JSON header mapping each
tensor name to {dtype, shape, data_offsets}, then the raw little-endian data.
The reference reads GGUF the same way: a header and a tensor table over a
memory map, tensors fetched by name (src/gguf.rs:303-367); only the container
differs.  This reader maps the file and hands out views, so a 16 GB file costs
no host copy until a tensor is moved to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Optional, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# name -> (numpy dtype used to view the bytes, torch dtype of the result, bytes per element)
_DTYPES = {
    "F64": (np.float64, torch.float64, 8),
    "F32": (np.float32, torch.float32, 4),
    "F16": (np.float16, torch.float16, 2),
    "BF16": (np.uint16, torch.bfloat16, 2),
    "I64": (np.int64, torch.int64, 8),
    "I32": (np.int32, torch.int32, 4),
    "I16": (np.int16, torch.int16, 2),
    "I8": (np.int8, torch.int8, 1),
    "U8": (np.uint8, torch.uint8, 1),
    "BOOL": (np.bool_, torch.bool, 1),
}
_TORCH_TO_NAME = {
    torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
    torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
    torch.bool: "BOOL",
}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; `get(name)` returns a CPU tensor viewing the map."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except FileNotFoundError:
            raise SafetensorsError(f"{path}: no such file") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: the header must be a JSON object")
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for \"{name}\"") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor \"{name}\" has unsupported dtype {dtype}")
            n = 1
            for s in shape:
                n *= s
            if e - b != n * _DTYPES[dtype][2]:
                raise SafetensorsError(f"{path}: tensor \"{name}\" spans {e - b} bytes but {dtype}{list(shape)} needs {n * _DTYPES[dtype][2]}")
            if b < 0 or e > data_len:
                raise SafetensorsError(f"{path}: tensor \"{name}\" runs past the end of the file")
            self.entries[name] = TensorEntry(name, dtype, shape, b, e)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def get(self, name: str) -> torch.Tensor:
        ent = self.entries[name]
        np_dtype, t_dtype, _ = _DTYPES[ent.dtype]
        n = 1
        for s in ent.shape:
            n *= s
        if n == 0:
            return torch.empty(ent.shape, dtype=t_dtype)
        arr = np.frombuffer(self._map, dtype=np_dtype, count=n, offset=self._data_start + ent.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; nobody writes through these views
            t = torch.from_numpy(arr)
        if ent.dtype == "BF16":
            t = t.view(torch.bfloat16)
        return t.reshape(ent.shape)

    def close(self) -> None:
        # views handed out keep the map alive through numpy's buffer reference
        try:
            self._f.close()
        except Exception:
            pass


def save_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Writes `tensors` (CPU, any supported dtype) in sorted-name order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot store tensor \"{name}\" of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)
