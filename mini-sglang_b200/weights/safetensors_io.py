"""Reader and writer of the safetensors container, by tensor name (the reference reads the same files
with the safetensors package, mini_sglang/utils/loader.py:17-23).

File layout: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the raw
little-endian tensor data.  The reader maps the file and hands out one tensor at a time, so a
16 GB checkpoint is never held twice in host memory.
"""

from __future__ import annotations

import glob
import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I8": torch.int8, "U8": torch.uint8, "I16": torch.int16, "I32": torch.int32, "I64": torch.int64,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name, dtype, shape, begin, end, file):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, tuple(shape), begin, end, file


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file")
        try:
            header = json.loads(self._f.read(n))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self._data_start = 8 + n
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dt = _DTYPES.get(info.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor {name!r} has dtype {info.get('dtype')!r}, which is not handled")
            b, e = info["data_offsets"]
            numel = 1
            for s in info["shape"]:
                numel *= s
            if e - b != numel * torch.empty((), dtype=dt).element_size() or self._data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has offsets that do not match its shape")
            self.entries[name] = TensorEntry(name, dt, info["shape"], b, e, self)

    def read(self, name: str) -> torch.Tensor:
        """CPU tensor that views the mapped file (copy before the file is closed)."""
        e = self.entries[name]
        if e.end == e.begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._mm)[self._data_start + e.begin: self._data_start + e.end]
        with warnings.catch_warnings():      # the map is read-only; callers copy, never write
            warnings.simplefilter("ignore", UserWarning)
            return torch.frombuffer(buf, dtype=e.dtype).reshape(e.shape)

    def close(self):
        # tensors handed out by read() may still view the map; let the garbage collector unmap
        self._mm = None
        self._f.close()


def open_model_dir(model_dir: str) -> Tuple[List[SafetensorsFile], Dict[str, TensorEntry]]:
    """All *.safetensors of a folder, sorted, and the union of their tensors."""
    paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not paths:
        raise SafetensorsError(f"{model_dir}: no *.safetensors file")
    files, index = [], {}
    for p in paths:
        f = SafetensorsFile(p)
        files.append(f)
        for name, e in f.entries.items():
            if name in index:
                raise SafetensorsError(f"tensor {name!r} is in both {index[name].file.path} and {p}")
            index[name] = e
    return files, index


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: Dict[str, str] = None) -> None:
    """Write tensors (an iterable of (name, tensor), consumed twice if it is a list, once if the
    caller passes a list of already materialised tensors)."""
    items = list(tensors)
    header, off = {}, 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"{name}: dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for _, t in items:
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)
