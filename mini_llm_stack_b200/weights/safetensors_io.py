"""Reading and writing ``.safetensors`` files by tensor name.

The reference keeps a checkpoint as one ``torch.save`` dict (serve/api.py:47-48)
and loads it with a strict ``load_state_dict`` (serve/api.py:60).  A model
folder here holds ``model.safetensors`` instead: an 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw
little-endian tensor bytes.  The file is memory-mapped, so a tensor's bytes are
touched only when that tensor is copied to the device.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
    "F64": torch.float64, "I32": torch.int32, "I64": torch.int64,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFormatError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read one at a time."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        if not self.path.is_file():
            raise FileNotFoundError(f"no weight file at {str(self.path)!r}")
        self._fh = open(self.path, "rb")
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsFormatError(f"{self.path}: too short for a header")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsFormatError(f"{self.path}: bad header length {hlen}")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsFormatError(f"{self.path}: header is not JSON") from exc
        self.metadata = header.pop("__metadata__", {}) or {}
        self._data_start = 8 + hlen
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsFormatError(
                    f"{self.path}: tensor {name!r} has unsupported dtype "
                    f"{info['dtype']}")
            b, e = info["data_offsets"]
            ent = TensorEntry(name, _DTYPES[info["dtype"]], tuple(info["shape"]),
                              int(b), int(e))
            n = 1
            for s in ent.shape:
                n *= s
            if e - b != n * ent.dtype.itemsize or self._data_start + e > size:
                raise SafetensorsFormatError(
                    f"{self.path}: tensor {name!r} has inconsistent offsets")
            self.entries[name] = ent
        self._mm = (mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
                    if size > 0 else None)

    def names(self) -> list:
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU tensor that owns its memory."""
        ent = self.entries[name]
        n = 1
        for s in ent.shape:
            n *= s
        if n == 0:
            return torch.empty(ent.shape, dtype=ent.dtype)
        buf = memoryview(self._mm)[self._data_start + ent.begin:
                                   self._data_start + ent.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # read-only map; cloned at once
            t = torch.frombuffer(buf, dtype=ent.dtype, count=n).reshape(ent.shape)
        return t.clone()

    def close(self) -> None:
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str | Path, specs: list, produce, metadata=None) -> None:
    """Write tensors one by one.

    ``specs`` is a list of ``(name, dtype, shape)`` in file order; ``produce(name)``
    returns that tensor (CPU, right dtype and shape) when its turn comes, so a
    large model never exists twice in memory.
    """
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, dtype, shape in specs:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * dtype.itemsize
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name, dtype, shape in specs:
            t = produce(name)
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise ValueError(f"tensor {name!r}: produced {t.dtype} "
                                 f"{tuple(t.shape)}, declared {dtype} {tuple(shape)}")
            t = t.contiguous().cpu()
            if t.numel():
                fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
