"""Reading and writing safetensors files without any library.

Layout: 8 bytes little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor bytes; offsets count from the end of the header.
The reference memory-maps such files and fetches tensors by name
(backends/vllm/src/models/llama.rs:86-93); a folder may hold one file or several
listed by ``model.safetensors.index.json`` (backends/vllm/src/models/mod.rs:9-37).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A memory-mapped file; ``tensor(name)`` returns a CPU view without copying."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n))
        except Exception as e:  # noqa: BLE001
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY)
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {e['dtype']!r}")
            dt = _DTYPES[e["dtype"]]
            shape = tuple(int(s) for s in e["shape"])
            b, en = e["data_offsets"]
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=dt).element_size()
            if en - b != want or self._base + en > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans {en - b} bytes, its shape {shape} needs {want}"
                )
            self.entries[name] = (dt, shape, b, en)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, en = self.entries[name]
        if en == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._base + b:self._base + en]
        return torch.frombuffer(buf, dtype=dt).reshape(shape)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((-(8 + len(blob))) % 8)  # data starts 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                t.reshape(-1).view(torch.uint8).numpy().tofile(f)


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The safetensors files of a model folder: the index's shards, else every ``*.safetensors``."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        paths = [os.path.join(model_dir, s) for s in shards]
    else:
        paths = sorted(
            os.path.join(model_dir, p) for p in os.listdir(model_dir) if p.endswith(".safetensors")
        )
    if not paths:
        raise SafetensorsError(f"{model_dir!r} holds no .safetensors file")
    for p in paths:
        if not os.path.isfile(p):
            raise SafetensorsError(f"{p} is listed by the index but does not exist")
    return [SafetensorsFile(p) for p in paths]
