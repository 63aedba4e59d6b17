"""Reading and writing .safetensors files, by tensor name, through mmap.

File layout: 8 bytes little-endian header length, a JSON header
`{name: {"dtype", "shape", "data_offsets": [begin, end]}}`, then the data.  This
takes the place of QStream's mmap file access (src/file_access.c:21-172) and of
its converter's name index (tools/convert_hf.py:576-598).  Every offset is checked
against the file before anything is read.
"""
from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

from ..errors import QsError, QStreamError

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 << 20


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    begin: int          # offsets into the file
    end: int


class SafetensorsFile:
    """One mapped file; `read(name)` returns a CPU tensor that views the mapping."""

    def __init__(self, path, allow_mmap: bool = True):
        self.path = Path(path)
        if not self.path.is_file():
            raise QStreamError(QsError.FILE_NOT_FOUND, str(self.path))
        size = self.path.stat().st_size
        if size < 8:
            raise QStreamError(QsError.FILE_CORRUPTED, f"{self.path}: shorter than its length field")
        self._fh = open(self.path, "rb")
        if allow_mmap:
            self._buf = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        else:                               # QStream's --no-mmap: plain read
            self._buf = self._fh.read()
        (hlen,) = struct.unpack("<Q", self._buf[:8])
        if hlen > _MAX_HEADER or 8 + hlen > size:
            raise QStreamError(QsError.FILE_CORRUPTED,
                               f"{self.path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(bytes(self._buf[8:8 + hlen]))
        except (ValueError, UnicodeDecodeError) as e:
            raise QStreamError(QsError.FILE_CORRUPTED, f"{self.path}: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise QStreamError(QsError.FILE_CORRUPTED, f"{self.path}: header is not a JSON object")
        base = 8 + hlen
        self.entries: dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = _DTYPES[meta["dtype"]]
                shape = tuple(int(s) for s in meta["shape"])
                a, b = (int(x) for x in meta["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise QStreamError(QsError.FILE_CORRUPTED,
                                   f"{self.path}: bad header entry for '{name}': {meta!r}") from None
            n = 1
            for s in shape:
                n *= s
            want = n * torch.empty((), dtype=dtype).element_size()
            if a < 0 or b < a or base + b > size or b - a != want:
                raise QStreamError(
                    QsError.FILE_CORRUPTED,
                    f"{self.path}: tensor '{name}' {meta['dtype']}{list(shape)} needs {want} bytes, "
                    f"its offsets [{a}, {b}) give {b - a}, data section holds {size - base}")
            self.entries[name] = TensorEntry(name, dtype, shape, base + a, base + b)

    def names(self):
        return list(self.entries)

    def read(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        if n == 0:
            return torch.empty(e.shape, dtype=e.dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the mapping is read-only; nothing writes to it
            t = torch.frombuffer(self._buf, dtype=e.dtype, count=n, offset=e.begin)
        return t.reshape(e.shape)

    def close(self):
        buf, self._buf = self._buf, None
        if isinstance(buf, mmap.mmap):
            try:
                buf.close()
            except BufferError:
                pass                            # a tensor still views the mapping
        self._fh.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors in the order given, each 8-byte aligned."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise QStreamError(QsError.INVALID_INPUT, f"cannot store dtype {t.dtype} ('{name}')")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)
