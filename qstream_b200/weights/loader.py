"""Binding a checkpoint's tensors to the tensors the parts declare.

The model says which tensors it wants (checkpoint name, shape, kind); the files say
which they hold.  Everything that does not fit is reported in ONE error that lists
missing tensors, unexpected tensors and wrong shapes, in the place of QStream's
late "missing Q projection tensor" at run time (src/engine.c:842-845) and its
converter's silent skips (tools/convert_hf.py:1142-1144).

Precision rule: floating tensors are kept in bfloat16 in a bfloat16 engine and
widened to float32 in a float32 engine; a tensor that the file stores in 32-bit
stays in 32-bit; integer tables become int32.  A bfloat16 engine that is given
matrices stored in 32-bit therefore runs them on the CUDA cores in true 32-bit, far
from the tensor-core path: the loader says so once, and `narrow_fp32_matrices=True`
rounds such matrices (not norms or biases) to bfloat16 instead.

A checkpoint in several files is read through `model.safetensors.index.json`
(`weight_map`: tensor name -> file) when the folder has one, as the converter's
TensorLoader reads it (tools/convert_hf.py:576-598); without it every *.safetensors
file of the folder is opened.  On a CUDA device the stored bytes are uploaded as they
are and converted there (csrc/utility.cu).
"""
from __future__ import annotations

import json
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping

import torch

from ..errors import QsError, QStreamError
from .safetensors_io import SafetensorsFile


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part wants.  `role` tells the random initialiser what it is:
    "matrix" (projection or table), "norm_weight", "bias" or "int_table"."""
    shape: tuple
    role: str = "matrix"

    @property
    def is_int(self) -> bool:
        return self.role == "int_table"


def target_dtype(stored: torch.dtype, engine_dtype: torch.dtype, is_int: bool, narrow: bool = False) -> torch.dtype:
    if is_int:
        return torch.int32
    if stored in (torch.float32, torch.float64) and not narrow:
        return torch.float32
    return engine_dtype                     # 16-bit floats follow the engine


INDEX_NAME = "model.safetensors.index.json"


def open_checkpoint(folder, allow_mmap: bool = True) -> list[SafetensorsFile]:
    """The folder's safetensors files: those its index names, else all of them."""
    folder = Path(folder)
    index = folder / INDEX_NAME
    if index.is_file():
        try:
            weight_map = json.loads(index.read_text())["weight_map"]
            names = sorted(set(weight_map.values()))
            if not names or not all(isinstance(n, str) for n in names):
                raise ValueError("empty or malformed weight_map")
        except (ValueError, KeyError, TypeError, AttributeError) as e:
            raise QStreamError(QsError.FILE_CORRUPTED, f"{index}: {e!r}") from None
        files = []
        for n in names:
            if Path(n).name != n or not (folder / n).is_file():
                raise QStreamError(QsError.FILE_NOT_FOUND, f"{index} names '{n}', which is not a file of {folder}")
            files.append(SafetensorsFile(folder / n, allow_mmap))
        misplaced = [f"{t} (index: {fn})" for t, fn in weight_map.items()
                     if t not in next(f for f in files if f.path.name == fn).entries]
        if misplaced:
            raise QStreamError(QsError.INVALID_MODEL, f"{index}: tensors not in the file it names: " + ", ".join(sorted(misplaced)))
        return files
    paths = sorted(folder.glob("*.safetensors"))
    if not paths:
        raise QStreamError(QsError.FILE_NOT_FOUND, f"no .safetensors file in {folder}")
    return [SafetensorsFile(p, allow_mmap) for p in paths]


_ON_DEVICE = (torch.float32, torch.bfloat16, torch.float16)


def _place(src: torch.Tensor, dtype: torch.dtype, device) -> torch.Tensor:
    device = torch.device(device)
    if device.type == "cuda" and src.dtype in _ON_DEVICE and dtype in (torch.float32, torch.bfloat16):
        raw = src.contiguous().to(device)               # the stored bytes; converted on the device
        if raw.dtype == dtype:
            return raw
        from ..csrc import ops
        return ops.convert(raw, dtype)
    return src.to(device=device, dtype=dtype).contiguous()


def bind_tensors(files: list[SafetensorsFile], wanted: Mapping[str, TensorDecl],
                 engine_dtype: torch.dtype, device, ignored_suffixes: Iterable[str] = (),
                 progress=None, narrow_fp32_matrices: bool = False) -> dict[str, torch.Tensor]:
    """Load every wanted tensor onto `device`; raise one INVALID_MODEL error that
    lists all that is missing, unexpected or misshapen."""
    where: dict[str, SafetensorsFile] = {}
    duplicate = []
    for f in files:
        for name in f.names():
            if name in where:
                duplicate.append(name)
            where[name] = f
    ignored = tuple(ignored_suffixes)
    missing = [n for n in wanted if n not in where]
    unexpected = [n for n in where if n not in wanted and not (ignored and n.endswith(ignored))]
    wrong = []
    for name, decl in wanted.items():
        if name not in where:
            continue
        e = where[name].entries[name]
        if tuple(e.shape) != tuple(decl.shape):
            wrong.append(f"{name}: file has {list(e.shape)}, model wants {list(decl.shape)}")
        elif decl.is_int == e.dtype.is_floating_point:
            wrong.append(f"{name}: file stores {e.dtype}, model wants "
                         f"{'an integer table' if decl.is_int else 'a floating tensor'}")
    if missing or unexpected or wrong or duplicate:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: " + ", ".join(sorted(missing)))
        if unexpected:
            parts.append(f"{len(unexpected)} unexpected: " + ", ".join(sorted(unexpected)))
        if wrong:
            parts.append(f"{len(wrong)} wrong shape or type: " + "; ".join(wrong))
        if duplicate:
            parts.append(f"{len(duplicate)} stored twice: " + ", ".join(sorted(duplicate)))
        raise QStreamError(QsError.INVALID_MODEL, "checkpoint does not fit the model - " + " | ".join(parts))

    out = {}
    wide = []
    for i, (name, decl) in enumerate(wanted.items()):
        src = where[name].read(name)
        dt = target_dtype(src.dtype, engine_dtype, decl.is_int, narrow_fp32_matrices and decl.role == "matrix")
        if decl.role == "matrix" and dt == torch.float32 and engine_dtype == torch.bfloat16:
            wide.append(name)
        out[name] = _place(src, dt, device)
        if progress:
            progress(i + 1, len(wanted), name)
    if wide:
        print(f"[qstream] {len(wide)} matrices are stored in 32-bit (first: {wide[0]}) and stay so in this bfloat16 "
              "engine: their products run on the CUDA cores in true 32-bit, not on the tensor cores; "
              "narrow_fp32_matrices=True (--narrow-fp32) rounds them to bfloat16", file=sys.stderr)
    return out
