"""Reading and writing the safetensors container, without a library.

Layout (the same one the reference's converter parses, tools/convert.py:41-50): an
8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the raw little-endian data.  BF16, F16, F32 and the integer types
I32 / I64 are understood; anything else is an error (tools/convert.py:85-92 accepts
BF16, F32 and F16 only).
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
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int  # absolute byte offsets in the file
    end: int
    path: str


class SafetensorsFile:
    """One ``.safetensors`` file, memory-mapped; tensors are views until copied."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > size - 8:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: Dict[str, TensorEntry] = {}
        base = 8 + hlen
        for name, info in header.items():
            dt = info.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {dt}")
            shape = tuple(int(s) for s in info["shape"])
            b, e = info["data_offsets"]
            numel = 1
            for s in shape:
                numel *= s
            if e - b != numel * _DTYPES[dt][1]:
                raise SafetensorsError(
                    f"{path}: tensor {name}: {e - b} bytes do not match shape {list(shape)} {dt}")
            if b < 0 or base + e > size:
                raise SafetensorsError(f"{path}: tensor {name} is truncated (offsets beyond the file)")
            self.entries[name] = TensorEntry(name, dt, shape, base + b, base + e, path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor sharing the mapping's memory (read-only; copy before writing)."""
        e = self.entries[name]
        dtype, _ = _DTYPES[e.dtype]
        numel = 1
        for s in e.shape:
            numel *= s
        if numel == 0:
            return torch.empty(e.shape, dtype=dtype)
        buf = memoryview(self._mm)[e.begin:e.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch notes that the buffer is not writable
            t = torch.frombuffer(buf, dtype=dtype, count=numel)
        return t.reshape(e.shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through their buffer
        self._f.close()


def open_model_shards(folder: str) -> List[SafetensorsFile]:
    """All ``*.safetensors`` of a model folder in sorted order (tools/convert.py:83)."""
    files = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"no .safetensors file in {folder}")
    return [SafetensorsFile(os.path.join(folder, f)) for f in files]


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Write CPU tensors in the given order; offsets are packed without padding."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    offset = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name} of dtype {t.dtype}")
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
