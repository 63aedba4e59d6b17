"""Random weights from a configuration and a seed, and the model folder they make.

QStream has no such mode; it exists so that every path (loader included) can be run
without a checkpoint.  The distributions are those the benchmark configurations name:
matrices and tables N(0, sigma_w); norm weights 1 + U(-a, a); biases N(0, sigma_b).
Each tensor draws from its own generator, seeded by the seed and the tensor's place in
the model's declaration order, so a tensor does not depend on which others exist
before it only through that index.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Mapping

import torch

from ..errors import QsError, QStreamError
from .loader import TensorDecl
from .safetensors_io import write_safetensors


@dataclass(frozen=True)
class InitScales:
    matrix_std: float = 0.02
    norm_spread: float = 0.1
    bias_std: float = 0.02


def random_tensors(wanted: Mapping[str, TensorDecl], seed: int, dtype: torch.dtype,
                   device="cpu", scales: InitScales = InitScales(),
                   int_high: int = 2) -> dict[str, torch.Tensor]:
    """Tensors for every declaration.  Values are drawn in float32 and rounded once
    to `dtype`."""
    out = {}
    dev = torch.device(device)
    for i, (name, decl) in enumerate(wanted.items()):
        g = torch.Generator(device=dev)
        g.manual_seed((int(seed) * 1_000_003 + i) & 0x7FFF_FFFF_FFFF_FFFF)
        shape = tuple(decl.shape)
        if decl.role == "int_table":
            t = torch.randint(0, int_high, shape, generator=g, device=dev, dtype=torch.int32)
        elif decl.role == "norm_weight":
            t = torch.rand(shape, generator=g, device=dev, dtype=torch.float32)
            t = (1.0 + (2.0 * t - 1.0) * scales.norm_spread).to(dtype)
        elif decl.role == "bias":
            t = (torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
                 * scales.bias_std).to(dtype)
        elif decl.role == "matrix":
            t = torch.empty(shape, device=dev, dtype=dtype)
            flat = t.view(-1)
            step = 1 << 26                  # bounded 32-bit staging for very large tables
            for a in range(0, flat.numel(), step):
                n = min(step, flat.numel() - a)
                flat[a:a + n] = (torch.randn(n, generator=g, device=dev, dtype=torch.float32)
                                 * scales.matrix_std).to(dtype)
        else:
            raise QStreamError(QsError.INTERNAL, f"unknown tensor role '{decl.role}' for {name}")
        out[name] = t
    return out


def write_model_folder(folder, config, seed: int, dtype="bfloat16",
                       scales: InitScales = InitScales()) -> Path:
    """Write `config.json` and `model.safetensors` for `config` with random weights."""
    from ..engine.model import declared_tensors      # the model says what it holds
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32,
                   torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}.get(dtype)
    if torch_dtype is None:
        raise QStreamError(QsError.INVALID_INPUT, f"dtype {dtype!r}: want bfloat16 or float32")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    wanted = declared_tensors(config.model_spec())
    tensors = random_tensors(wanted, seed, torch_dtype, "cpu", scales)
    d = config.to_dict()
    d["torch_dtype"] = "bfloat16" if torch_dtype == torch.bfloat16 else "float32"
    (folder / "config.json").write_text(json.dumps(d, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": seed})
    return folder
