"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header {name: {dtype, shape, data_offsets}}, then the raw tensors.

The reader maps the file and hands out tensors that alias the mapping, so a tensor is
copied once, by whoever moves it to its device.  (The reference reads GGUF through
Candle, src/weights.rs:300-331; the container is the only thing replaced here.)
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Callable, Dict, List, Tuple

import torch

DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsFile:
    """One mapped file; `entries` maps a name to (dtype, shape, begin, end)."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise ValueError(f"{path}: too short to be a safetensors file")
            (n,) = struct.unpack("<Q", head)
            size = os.path.getsize(path)
            if n > size - 8:
                raise ValueError(f"{path}: header length {n} exceeds the file")
            try:
                header = json.loads(f.read(n))
            except json.JSONDecodeError as e:
                raise ValueError(f"{path}: header is not JSON ({e})") from None
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        self._base = 8 + n
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, meta in header.items():
            if meta["dtype"] not in DTYPES:
                raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
            a, b = meta["data_offsets"]
            if not (0 <= a <= b <= size - self._base):
                raise ValueError(f"{path}: tensor {name!r} lies outside the file")
            self.entries[name] = (DTYPES[meta["dtype"]], tuple(meta["shape"]), a, b)

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only tensor aliasing the mapped file."""
        dtype, shape, a, b = self.entries[name]
        if a == b:
            return torch.empty(shape, dtype=dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            raw = torch.frombuffer(self._map, dtype=torch.uint8, count=b - a,
                                   offset=self._base + a)
        return raw.view(dtype).reshape(shape)


def write_streamed(path: str, layout: List[Tuple[str, Tuple[int, ...], torch.dtype]],
                   produce: Callable[[str], torch.Tensor],
                   metadata: Dict[str, str] = None) -> None:
    """Write the tensors named in `layout` (name, shape, dtype), asking `produce` for
    each one in turn so that only one is in memory at a time."""
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    for name, shape, dtype in layout:
        numel = 1
        for d in shape:
            numel *= d
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": NAMES[dtype], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-(8 + len(blob)) % 64)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype in layout:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise ValueError(f"tensor {name!r}: produced {tuple(t.shape)} {t.dtype}, "
                                 f"layout says {tuple(shape)} {dtype}")
            if t.numel():
                f.write(t.contiguous().view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor],
                      metadata: Dict[str, str] = None) -> None:
    """Write a dictionary of tensors."""
    layout = [(n, tuple(t.shape), t.dtype) for n, t in tensors.items()]
    write_streamed(path, layout, lambda n: tensors[n], metadata)
