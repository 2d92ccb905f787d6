"""safetensors files: a reader and a writer of our own.

Format (include/ai/Safetensors.hpp:389-485): an unsigned 64-bit little-endian
header length, a JSON header ``{name: {dtype, shape, data_offsets: [b, e]}}``
(``__metadata__`` is skipped), then the payload.  The reader checks what the
reference checks: header length in range, offsets a pair with ``e >= b`` and
``e`` inside the payload, a known dtype, and bytes == elements x width.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# dtype name -> (bytes per element, torch dtype)
DTYPES = {
    "F64": (8, torch.float64), "F32": (4, torch.float32), "F16": (2, torch.float16),
    "BF16": (2, torch.bfloat16), "I64": (8, torch.int64), "I32": (4, torch.int32),
    "I16": (2, torch.int16), "I8": (1, torch.int8), "U8": (1, torch.uint8),
    "BOOL": (1, torch.bool),
}
_NAME_OF = {v[1]: k for k, v in DTYPES.items()}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read by name."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise SafetensorsError(f"{path}: no such file") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a header length")
        self._file = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len < 2 or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self._base = 8 + header_len
        payload = size - self._base
        self.tensors: Dict[str, TensorInfo] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            self.tensors[name] = self._entry(name, meta, payload)
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def _entry(self, name: str, meta, payload: int) -> TensorInfo:
        where = f"{self.path}: tensor '{name}'"
        if not isinstance(meta, dict):
            raise SafetensorsError(f"{where}: entry is not an object")
        dtype, shape, offsets = meta.get("dtype"), meta.get("shape"), meta.get("data_offsets")
        if dtype not in DTYPES:
            raise SafetensorsError(f"{where}: unknown dtype {dtype!r}")
        if not isinstance(shape, list) or not all(isinstance(s, int) and s >= 0 for s in shape):
            raise SafetensorsError(f"{where}: bad shape {shape!r}")
        if (not isinstance(offsets, list) or len(offsets) != 2
                or not all(isinstance(o, int) and o >= 0 for o in offsets)):
            raise SafetensorsError(f"{where}: data_offsets must be a pair of byte offsets")
        begin, end = offsets
        if end < begin or end > payload:
            raise SafetensorsError(f"{where}: data_offsets [{begin}, {end}] outside the payload ({payload} bytes)")
        info = TensorInfo(name, dtype, tuple(shape), begin, end)
        if info.numel * DTYPES[dtype][0] != end - begin:
            raise SafetensorsError(
                f"{where}: {end - begin} bytes for shape {list(shape)} of {dtype} "
                f"(needs {info.numel * DTYPES[dtype][0]})")
        return info

    def names(self) -> Iterable[str]:
        return self.tensors.keys()

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor of the stored dtype that owns its memory."""
        info = self.tensors[name]
        width, dtype = DTYPES[info.dtype]
        if info.numel == 0:
            return torch.empty(info.shape, dtype=dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=info.end - info.begin,
                            offset=self._base + info.begin).copy()
        return torch.from_numpy(raw).view(dtype).reshape(info.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Writes CPU tensors in name order, each starting on an 8-byte boundary of
    the payload."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAME_OF:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAME_OF[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
