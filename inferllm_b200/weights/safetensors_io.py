"""Reading and writing the safetensors container (one file, or shards with an index).

Layout of a file: an unsigned 64-bit little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}` (offsets relative to the end
of the header), then the raw little-endian row-major data.  The reference has its own
container with the same idea, a per-tensor record of dims, name and type followed by
the raw data (src/core/graph.cpp:285-309); there the bytes are read at first use, here
a file is memory-mapped and each tensor is copied to the device once at load.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass
class TensorRecord:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int
    end: int
    file: "SafetensorsFile"


class SafetensorsFile:
    """A memory-mapped safetensors file; `tensor(name)` gives a CPU tensor that views the
    mapping (copy it before the file is closed)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file size {size}")
        try:
            header = json.loads(self._f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        self.records: Dict[str, TensorRecord] = {}
        for name, rec in header.items():
            if rec["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {rec['dtype']}")
            dtype = _DTYPES[rec["dtype"]]
            shape = tuple(int(s) for s in rec["shape"])
            b, e = rec["data_offsets"]
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=dtype).element_size()
            if e - b != want or b < 0 or self._base + e > size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' {list(shape)} {rec['dtype']} needs {want} bytes, "
                    f"its record gives [{b}, {e}) in a data section of {size - self._base} bytes "
                    "(truncated or corrupt file)")
            self.records[name] = TensorRecord(name, dtype, shape, b, e, self)

    def tensor(self, name: str) -> torch.Tensor:
        r = self.records[name]
        if r.end == r.begin:
            return torch.empty(r.shape, dtype=r.dtype)
        buf = memoryview(self._map)[self._base + r.begin:self._base + r.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # read-only buffer: the tensor is only copied from
            t = torch.frombuffer(buf, dtype=r.dtype)
        return t.view(r.shape)

    def close(self):
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass  # tensors still view the mapping; it goes with them
            self._map = None
        self._f.close()


def open_model_files(folder: str) -> Tuple[Dict[str, TensorRecord], List[SafetensorsFile]]:
    """All tensor records of a model folder: `model.safetensors`, or the shards named by
    `model.safetensors.index.json`."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    files: List[SafetensorsFile] = []
    records: Dict[str, TensorRecord] = {}
    if os.path.isfile(single):
        files.append(SafetensorsFile(single))
    elif os.path.isfile(index):
        with open(index) as f:
            weight_map = json.load(f).get("weight_map", {})
        for shard in sorted(set(weight_map.values())):
            p = os.path.join(folder, shard)
            if not os.path.isfile(p):
                raise SafetensorsError(f"{index} names shard '{shard}', which is not in {folder}")
            files.append(SafetensorsFile(p))
    else:
        raise SafetensorsError(f"{folder}: neither model.safetensors nor "
                               "model.safetensors.index.json found")
    for f in files:
        for name, rec in f.records.items():
            if name in records:
                raise SafetensorsError(f"tensor '{name}' appears in both {records[name].file.path} "
                                       f"and {f.path}")
            records[name] = rec
    return records, files


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None):
    """Write tensors to `path`.  `tensors` is a list of (name, tensor) or a callable-free
    iterable that can be walked twice (the header needs all shapes before the data)."""
    tensors = list(tensors)
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in tensors:
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy())
