"""Reading and writing the safetensors container, without any model library.

Format: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}},
then the raw little-endian tensor data.  Tensors are memory-mapped and returned
in the dtype they were stored in.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """A memory-mapped safetensors file: `names()`, `info(name)`, `tensor(name)`."""

    def __init__(self, path: str) -> None:
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (too short)")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise ValueError(f"{path}: not a safetensors file (bad header length {n})")
        self._header = json.loads(self._f.read(n).decode("utf-8"))
        self._header.pop("__metadata__", None)
        self._base = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def names(self) -> list[str]:
        return list(self._header)

    def info(self, name: str) -> tuple[torch.dtype, tuple[int, ...]]:
        e = self._header[name]
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {e['dtype']}")
        return _DTYPES[e["dtype"]], tuple(e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape = self.info(name)
        begin, end = self._header[name]["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # read-only mapping: never written to
            t = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + begin)
        if (end - begin) != count * t.element_size():
            raise ValueError(f"{self.path}: tensor {name!r} has {end - begin} bytes, "
                             f"its shape needs {count * t.element_size()}")
        return t.view(shape)


def save_safetensors(tensors: dict[str, torch.Tensor], path: str) -> None:
    header: dict[str, object] = {}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)
