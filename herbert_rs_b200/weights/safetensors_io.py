"""A small reader and writer for the safetensors container.

Layout: 8 bytes little-endian header length n, n bytes of JSON
({name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}),
then the tensor bytes.  The reference reads the same container through the safetensors
crate, one memory-mapped shard at a time, and finds shards through
`model.safetensors.index.json` (crates/backends/backend_common/src/loader_common.rs:1131-1149,
1182-1193).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

from ..errors import SafeTensorsError

# name -> (torch dtype, numpy carrier dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4"), 4),
    "BF16": (torch.bfloat16, np.dtype("<u2"), 2),
    "F16": (torch.float16, np.dtype("<f2"), 2),
    "F64": (torch.float64, np.dtype("<f8"), 8),
    "I64": (torch.int64, np.dtype("<i8"), 8),
    "I32": (torch.int32, np.dtype("<i4"), 4),
    "I16": (torch.int16, np.dtype("<i2"), 2),
    "I8": (torch.int8, np.dtype("i1"), 1),
    "U8": (torch.uint8, np.dtype("u1"), 1),
    "BOOL": (torch.bool, np.dtype("u1"), 1),
}
_TORCH_TO_NAME = {v[0]: k for k, v in _DTYPES.items()}

MAX_HEADER_BYTES = 100 * 1024 * 1024


class SafeTensorsFile:
    """One memory-mapped safetensors file; tensors are read by name."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._f = open(path, "rb")
        except OSError as e:
            raise SafeTensorsError(f"cannot open {path}: {e}") from e
        if size < 8:
            raise SafeTensorsError(f"{path}: truncated file ({size} bytes, no header length)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafeTensorsError(f"{path}: truncated file or bad header length {n} (file has {size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafeTensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafeTensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + n
        self._data_len = size - self._data_start
        self.entries: Dict[str, Tuple[str, tuple, int, int]] = {}
        for name, info in header.items():
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(v) for v in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafeTensorsError(f"{path}: malformed header entry for '{name}'") from e
            if dtype not in _DTYPES:
                raise SafeTensorsError(f"{path}: tensor '{name}' has unsupported dtype {dtype}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][2] if shape else _DTYPES[dtype][2]
            if begin < 0 or end < begin or end - begin != want:
                raise SafeTensorsError(
                    f"{path}: tensor '{name}' ({dtype} {list(shape)}) needs {want} bytes, header gives {end - begin}")
            if end > self._data_len:
                raise SafeTensorsError(
                    f"{path}: truncated file: tensor '{name}' ends at byte {end} of a {self._data_len}-byte data section")
            self.entries[name] = (dtype, shape, begin, end)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> Tuple[torch.dtype, tuple]:
        dtype, shape, _, _ = self.entries[name]
        return _DTYPES[dtype][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor holding a copy of the named tensor's bytes."""
        dtype, shape, begin, end = self.entries[name]
        tdt, ndt, _ = _DTYPES[dtype]
        count = (end - begin) // ndt.itemsize
        arr = np.frombuffer(self._mm, dtype=ndt, count=count, offset=self._data_start + begin).copy()
        t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.int16).view(torch.bfloat16)
        elif tdt == torch.bool:
            t = t.to(torch.bool)
        return t.reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


def _raw_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().tobytes()
    if t.dtype == torch.bool:
        return t.to(torch.uint8).numpy().tobytes()
    return t.numpy().tobytes()


def save_stream(entries, path: str, metadata: dict | None = None) -> None:
    """Write one safetensors file from `entries`: (name, dtype, shape, make) with `make()` returning
    the tensor.  Tensors are made and written one at a time, sorted by name, so a model larger
    than the host's free memory can still be written."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    entries = sorted(entries, key=lambda e: e[0])
    offset = 0
    for name, dtype, shape, _ in entries:
        if dtype not in _TORCH_TO_NAME:
            raise SafeTensorsError(f"cannot store dtype {dtype} for '{name}'")
        key = _TORCH_TO_NAME[dtype]
        n = int(np.prod(shape, dtype=np.int64)) * _DTYPES[key][2] if len(shape) else _DTYPES[key][2]
        header[name] = {"dtype": key, "shape": [int(d) for d in shape], "data_offsets": [offset, offset + n]}
        offset += n
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for name, dtype, shape, make in entries:
            t = make()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise SafeTensorsError(f"'{name}' was announced as {dtype} {list(shape)} and made as {t.dtype} {list(t.shape)}")
            f.write(_raw_bytes(t))


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: dict | None = None) -> None:
    """Write tensors (sorted by name) to one safetensors file."""
    save_stream([(n, t.dtype, tuple(t.shape), (lambda t=t: t)) for n, t in tensors.items()], path, metadata)


class ModelFiles:
    """All safetensors shards of a model folder, addressed by tensor name."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.files: Dict[str, SafeTensorsFile] = {}
        self.where: Dict[str, str] = {}
        if os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
            except (OSError, KeyError, json.JSONDecodeError) as e:
                raise SafeTensorsError(f"{index}: cannot read weight_map: {e}") from e
            for shard in sorted(set(weight_map.values())):
                self.files[shard] = SafeTensorsFile(os.path.join(model_dir, shard))
            for name, shard in weight_map.items():
                if name not in self.files[shard].entries:
                    raise SafeTensorsError(f"tensor '{name}' is listed in the index but missing from shard {shard}")
                self.where[name] = shard
        elif os.path.exists(single):
            self.files["model.safetensors"] = SafeTensorsFile(single)
            for name in self.files["model.safetensors"].names():
                self.where[name] = "model.safetensors"
        else:
            raise SafeTensorsError(f"{model_dir}: no model.safetensors or model.safetensors.index.json")

    def names(self):
        return self.where.keys()

    def info(self, name: str):
        return self.files[self.where[name]].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.files[self.where[name]].tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()
