"""Binding a checkpoint's tensors to the tensors the parts declare.

The model says which tensors it wants (checkpoint name, shape, kind); the files say
which they hold.  Everything that does not fit is reported in ONE error that lists
missing tensors, unexpected tensors and wrong shapes, in the place of QStream's
late "missing Q projection tensor" at run time (src/engine.c:842-845) and its
converter's silent skips (tools/convert_hf.py:1142-1144).

Precision rule: floating tensors are kept in bfloat16 in a bfloat16 engine and
widened to float32 in a float32 engine; a tensor that the file stores in 32-bit
stays in 32-bit; integer tables become int32.
"""
from __future__ import annotations

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


def target_dtype(stored: torch.dtype, engine_dtype: torch.dtype, is_int: bool) -> torch.dtype:
    if is_int:
        return torch.int32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return engine_dtype                     # 16-bit floats follow the engine


def open_checkpoint(folder, allow_mmap: bool = True) -> list[SafetensorsFile]:
    folder = Path(folder)
    paths = sorted(folder.glob("*.safetensors"))
    if not paths:
        raise QStreamError(QsError.FILE_NOT_FOUND, f"no .safetensors file in {folder}")
    return [SafetensorsFile(p, allow_mmap) for p in paths]


def bind_tensors(files: list[SafetensorsFile], wanted: Mapping[str, TensorDecl],
                 engine_dtype: torch.dtype, device, ignored_suffixes: Iterable[str] = (),
                 progress=None) -> dict[str, torch.Tensor]:
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
    for i, (name, decl) in enumerate(wanted.items()):
        src = where[name].read(name)
        dt = target_dtype(src.dtype, engine_dtype, decl.is_int)
        out[name] = src.to(device=device, dtype=dt).contiguous()
        if progress:
            progress(i + 1, len(wanted), name)
    return out
