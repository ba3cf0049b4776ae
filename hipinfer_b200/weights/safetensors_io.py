"""A reader and a writer for the safetensors container, by tensor name.

Layout: 8 bytes little-endian header length N, N bytes of JSON
`{name: {"dtype": "BF16", "shape": [...], "data_offsets": [begin, end]}, "__metadata__": {...}}`,
then the tensors' bytes. The reader maps the file and hands out views, so a tensor that is
never asked for is never read. A folder may hold one `model.safetensors` or several shards with
a `model.safetensors.index.json` (`weight_map`: name -> file).

The reference reads a positional flat file instead (src/api.cu:1317-1399): no names, a fixed
order, 256-byte alignment.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped .safetensors file: `names()`, `info(name)` -> (dtype, shape), `get(name)`."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too small to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            head = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = head.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in head.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {e.get('dtype')!r}")
            dt, shape = _DTYPES[e["dtype"]], tuple(int(s) for s in e["shape"])
            b, en = (int(v) for v in e["data_offsets"])
            numel = 1
            for s in shape:
                numel *= s
            if en - b != numel * torch.empty((), dtype=dt).element_size() or self._base + en > size or b < 0:
                raise SafetensorsError(f"{path}: tensor {name!r}: data_offsets {b}..{en} do not match shape "
                                       f"{list(shape)} of {e['dtype']} in a file of {size} bytes")
            self._entries[name] = (dt, shape, b, en)
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > self._base else None

    def names(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str):
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the mapping)."""
        dt, shape, b, e = self._entries[name]
        if e == b:
            return torch.empty(shape, dtype=dt)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=e - b, offset=self._base + b).copy()
        return torch.from_numpy(raw).view(dt).reshape(shape)

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()


class ModelFiles:
    """All tensors of a model folder, whether in one file or in shards."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            with open(index) as f:
                wm = json.load(f).get("weight_map", {})
            paths = [os.path.join(folder, p) for p in sorted(set(wm.values()))]
        else:
            raise SafetensorsError(f"{folder}: no model.safetensors and no model.safetensors.index.json")
        for p in paths:
            if not os.path.isfile(p):
                raise SafetensorsError(f"{folder}: shard {os.path.basename(p)} named by the index is missing")
            sf = SafetensorsFile(p)
            self._files[p] = sf
            for n in sf.names():
                if n in self._where:
                    raise SafetensorsError(f"{folder}: tensor {n!r} is in two files")
                self._where[n] = p

    def names(self) -> List[str]:
        return list(self._where)

    def info(self, name: str):
        return self._files[self._where[name]].info(name)

    def get(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].get(name)

    def close(self):
        for f in self._files.values():
            f.close()


def save_safetensors(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] | None = None) -> None:
    """Write `tensors` (any device; written from CPU copies, one at a time) to `path`."""
    head, off = {}, 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        nb = t.numel() * t.element_size()
        head[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nb]}
        off += nb
    if metadata:
        head["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(head, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
