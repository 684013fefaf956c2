"""Reading and writing safetensors files.

The format: an 8-byte little-endian header length, a JSON header
{name: {"dtype", "shape", "data_offsets": [begin, end]}} and the raw little-endian data.
Shards are resolved as the reference does (vllm-oxide, crates/vllm-oxide/src/loader.rs:124-193):
`model.safetensors.index.json` (every file of its weight_map must exist), else
`model.safetensors`, else all `*.safetensors` sorted by name.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Dict, Tuple

import torch

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def resolve_shards(folder: str):
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            files = sorted(set(json.load(f).get("weight_map", {}).values()))
        paths = [os.path.join(folder, n) for n in files]
        missing = [p for p in paths if not os.path.isfile(p)]
        if missing:
            raise SafetensorsError(f"{index} names shards that do not exist (partial copy?): {missing}")
        if not paths:
            raise SafetensorsError(f"{index} has an empty weight_map")
        return paths
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    paths = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not paths:
        raise SafetensorsError(
            f"{folder}: no weights found (looked for model.safetensors.index.json, model.safetensors, *.safetensors)")
    return paths


class SafetensorsFile:
    """One memory-mapped file; tensors are views of the map until copied."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size} (truncated?)")
        try:
            header = json.loads(self._f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        header.pop("__metadata__", None)
        self._base = 8 + n
        self.entries: Dict[str, Tuple[str, tuple, int, int]] = {}
        for name, meta in header.items():
            if meta["dtype"] not in DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
            a, b = meta["data_offsets"]
            if self._base + b > size or a > b:
                raise SafetensorsError(f"{path}: tensor {name} lies outside the file (truncated?)")
            self.entries[name] = (meta["dtype"], tuple(meta["shape"]), a, b)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self):
        return self.entries.keys()

    def shape(self, name: str) -> tuple:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return DTYPES[self.entries[name][0]]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, a, b = self.entries[name]
        n = 1
        for s in shape:
            n *= s
        if n == 0:
            return torch.empty(shape, dtype=DTYPES[dt])
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the map is read-only; the view is only ever copied from
            t = torch.frombuffer(self._map, dtype=DTYPES[dt], count=n, offset=self._base + a)
        return t.reshape(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of tensor {name}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * ((8 - len(head) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
