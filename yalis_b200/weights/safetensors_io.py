"""Reading and writing the safetensors container.

The format: 8 bytes (little-endian u64) = length n of a JSON header, n bytes of
JSON ``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the raw little-endian tensor bytes; offsets are relative to the end of the
header.  Files are memory-mapped and a tensor is materialised only when it is
asked for, as the reference's lazy dictionary does (yalis/model_loading.py:13-181).
A folder may hold one ``model.safetensors`` or shards listed by
``model.safetensors.index.json`` (``weight_map``: name -> file).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise RuntimeError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise RuntimeError(f"{path}: not a safetensors file (header length {n})")
        try:
            header = json.loads(self._f.read(n))
        except ValueError as e:
            raise RuntimeError(f"{path}: unreadable safetensors header: {e}") from None
        header.pop("__metadata__", None)
        self._data_start = 8 + n
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise RuntimeError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            b, e = info["data_offsets"]
            self.entries[name] = (_DTYPES[info["dtype"]], tuple(info["shape"]), b, e)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if size > 0 else None

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (clone or move it before the file is closed).
        The mapping is private (copy-on-write), so nothing written through the view reaches the file."""
        dtype, shape, b, e = self.entries[name]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        if (e - b) != count * torch.empty((), dtype=dtype).element_size():
            raise RuntimeError(f"{self.path}: tensor {name} has {e - b} bytes for shape {shape} {dtype}")
        t = torch.frombuffer(self._mm, dtype=dtype, count=count, offset=self._data_start + b)
        return t.view(shape)

    def close(self) -> None:
        self.entries = {}
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass  # a tensor still views the map; the map goes with the last view
        self._f.close()


class Checkpoint:
    """All tensors of a model folder by name, whichever shard holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if not os.path.isdir(model_dir):
            raise FileNotFoundError(f"model folder {model_dir} does not exist")
        if os.path.isfile(index):
            with open(index) as f:
                idx = json.load(f)
            if "weight_map" not in idx:
                raise RuntimeError(f"{index} has no `weight_map`")
            for name, shard in idx["weight_map"].items():
                self._where[name] = shard
            for shard in sorted(set(self._where.values())):
                path = os.path.join(model_dir, shard)
                if not os.path.isfile(path):
                    raise FileNotFoundError(f"shard {path} named by the index is missing")
                self._files[shard] = SafetensorsFile(path)
            for name, shard in self._where.items():
                if name not in self._files[shard].entries:
                    raise RuntimeError(f"{index} places {name} in {shard}, which does not hold it")
        elif os.path.isfile(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].entries:
                self._where[name] = "model.safetensors"
        else:
            raise FileNotFoundError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> Iterable[str]:
        return self._where.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self._files[self._where[name]].entries[name]
        return dtype, shape

    def get(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].get(name)

    def close(self) -> None:
        for f in self._files.values():
            f.close()
        self._files = {}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write CPU tensors in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise RuntimeError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().data)
    os.replace(tmp, path)
