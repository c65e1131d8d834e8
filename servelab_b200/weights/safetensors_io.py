"""Minimal safetensors reader and writer (no third-party package needed).

File layout: an unsigned 64-bit little-endian header length, a JSON header
mapping each tensor name to {"dtype", "shape", "data_offsets": [begin, end]}
(offsets relative to the end of the header), then the raw little-endian data.
Tensors are read lazily by name through a copy-on-write memory map, so only the
pages of requested tensors are touched.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Callable, Dict, Iterable, List, Tuple

import torch

DTYPE_CODES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
CODE_OF_DTYPE = {v: k for k, v in DTYPE_CODES.items()}


class SafetensorsFile:
    """One open .safetensors file: header parsed eagerly, data mapped lazily."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise ValueError(f"{path}: too short to be a safetensors file")
            (hlen,) = struct.unpack("<Q", head)
            if hlen <= 0 or 8 + hlen > size:
                raise ValueError(f"{path}: corrupt safetensors header length {hlen}")
            try:
                header = json.loads(f.read(hlen).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise ValueError(f"{path}: corrupt safetensors header: {e}") from None
        self._base = 8 + hlen
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, dict] = header
        for name, info in header.items():
            lo, hi = info["data_offsets"]
            if info["dtype"] not in DTYPE_CODES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            if lo < 0 or lo > hi or self._base + hi > size:
                raise ValueError(f"{path}: tensor {name} points outside the file")
            count = 1
            for d in info["shape"]:
                count *= int(d)
            itemsize = torch.empty((), dtype=DTYPE_CODES[info["dtype"]]).element_size()
            if hi - lo != count * itemsize:
                # a shorter range would make read() return a neighbour's bytes
                raise ValueError(f"{path}: tensor {name} spans {hi - lo} bytes, its shape "
                                 f"{list(info['shape'])} and dtype need {count * itemsize}")
        self._map = None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return DTYPE_CODES[self.entries[name]["dtype"]]

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped file (copy-on-write)."""
        info = self.entries[name]
        dt = DTYPE_CODES[info["dtype"]]
        shape = tuple(info["shape"])
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dt)
        if self._map is None:
            with open(self.path, "rb") as f:
                self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
        lo, _ = info["data_offsets"]
        t = torch.frombuffer(self._map, dtype=dt, count=count, offset=self._base + lo)
        return t.reshape(shape)


def write_safetensors(path: str, decls: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      produce: Callable[[str], torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write tensors one at a time: ``decls`` fixes names, shapes and dtypes (so
    the header can be written first), ``produce(name)`` returns each tensor."""
    decls = list(decls)
    header, offset = {}, 0
    for name, shape, dt in decls:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dt).element_size()
        header[name] = {"dtype": CODE_OF_DTYPE[dt], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dt in decls:
            t = produce(name).detach().to("cpu").contiguous()
            if tuple(t.shape) != tuple(shape) or t.dtype != dt:
                raise ValueError(f"tensor {name}: produced {tuple(t.shape)} {t.dtype}, "
                                 f"declared {tuple(shape)} {dt}")
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
