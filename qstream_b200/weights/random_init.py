"""Random weights from a configuration and a seed, and the model folder they make.

QStream has no such mode; it exists so that every path (loader included) can be run
without a checkpoint.  The distributions are those the benchmark configurations name:
matrices and tables N(0, sigma_w); norm weights 1 + U(-a, a); biases N(0, sigma_b).

The generator is counter-based: element i of a tensor is a pure function of the seed,
the tensor's checkpoint name and i, so a tensor does not depend on which others exist,
any slice can be made alone, and the device kernel (csrc/utility.cu, `qs_random_fill`)
and the numpy code below give the same bits: a model made on the device
(`CausalLM.random`) and a folder written by the host (`write_model_folder`) hold the
same weights for the same seed.  Both compute Box-Muller's logarithm and cosine from
additions, multiplications, one division and one square root in double precision, in
the same order, instead of calling a library whose last bit differs between machines.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path
from typing import Mapping

import numpy as np
import torch

from ..errors import QsError, QStreamError
from .loader import TensorDecl
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


@dataclass(frozen=True)
class InitScales:
    matrix_std: float = 0.02
    norm_spread: float = 0.1
    bias_std: float = 0.02


# --------------------------------------------------------------------------- the stream

def _mix64_int(z: int) -> int:
    z &= _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream: the seed mixed with the FNV-1a hash of its name."""
    h = 0xCBF29CE484222325
    for byte in name.encode():
        h = ((h ^ byte) * 0x100000001B3) & _M64
    return _mix64_int(_mix64_int(int(seed) + _GOLDEN) ^ h)


def _bits(key: int, first: int, n: int) -> np.ndarray:
    """Elements first .. first + n of the SplitMix64 stream of seed `key`, as uint64."""
    with np.errstate(over="ignore"):
        z = np.uint64(key) + (np.arange(first + 1, first + n + 1, dtype=np.uint64) * np.uint64(_GOLDEN))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _horner(x2: np.ndarray, coefficients) -> np.ndarray:
    p = np.full_like(x2, coefficients[0])
    for c in coefficients[1:]:
        p = p * x2 + c              # two roundings, as the device's unfused multiply and add
    return p


_LN_COEFFS = [1.0 / 15.0, 1.0 / 13.0, 1.0 / 11.0, 1.0 / 9.0, 1.0 / 7.0, 1.0 / 5.0, 1.0 / 3.0, 1.0]
_COS_COEFFS = [1.0 / 20922789888000.0, -1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0,
               1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -0.5, 1.0]
_SIN_COEFFS = [-1.0 / 1307674368000.0, 1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0,
               -1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0, 1.0]


def _ln_of_fraction(m: np.ndarray) -> np.ndarray:
    """ln(m / 2^24) for integers m in 1 .. 2^24 (float64, the device's operations)."""
    raw = m.astype(np.float64).view(np.uint64)
    e = (raw >> np.uint64(52)).astype(np.int64) - 1023
    f = ((raw & np.uint64(0x000FFFFFFFFFFFFF)) | np.uint64(0x3FF0000000000000)).view(np.float64)
    big = f > 1.4142135623730951
    f = np.where(big, f * 0.5, f)
    e = e + big
    s = (f + -1.0) / (f + 1.0)
    p = _horner(s * s, _LN_COEFFS)
    return ((2.0 * s) * p) + (e - 24).astype(np.float64) * 0.6931471805599453


def _cos_of_turn(k: np.ndarray) -> np.ndarray:
    """cos(2 pi k / 2^24) for integers k in 0 .. 2^24 - 1."""
    quadrant = k >> np.uint64(22)
    j = (k & np.uint64(0x3FFFFF)).astype(np.int64)
    swap = j > 0x200000
    jj = np.where(swap, 0x400000 - j, j)
    x = jj.astype(np.float64) * (3.141592653589793 / 2.0 / 4194304.0)
    x2 = x * x
    c = _horner(x2, _COS_COEFFS)
    s = _horner(x2, _SIN_COEFFS) * x
    cos_t = np.where(swap, s, c)
    sin_t = np.where(swap, c, s)
    return np.select([quadrant == 0, quadrant == 1, quadrant == 2], [cos_t, -sin_t, -cos_t], sin_t)


def host_values(key: int, kind: str, a: float, first: int, n: int) -> np.ndarray:
    """Elements first .. first + n of a tensor's stream: float32 ("normal": N(0, a);
    "around_one": 1 + U(-a, a)) or int32 ("int": integers in [0, a))."""
    bits = _bits(key, first, n)
    if kind == "int":
        return (bits % np.uint64(int(a))).astype(np.int32)
    if kind == "normal":
        m1 = (bits >> np.uint64(40)) + np.uint64(1)
        k2 = (bits >> np.uint64(16)) & np.uint64(0xFFFFFF)
        r = np.sqrt(-2.0 * _ln_of_fraction(m1))
        v = (r * _cos_of_turn(k2)) * float(a)
    elif kind == "around_one":
        u = (bits >> np.uint64(40)).astype(np.float64) * (1.0 / 16777216.0)
        v = 1.0 + ((2.0 * u) + -1.0) * float(a)
    else:
        raise QStreamError(QsError.INTERNAL, f"unknown random kind '{kind}'")
    return v.astype(np.float32)


_KINDS = {"normal": 0, "around_one": 1, "int": 2}
_HOST_CHUNK = 1 << 22


def _fill(name, decl, seed, dtype, device, scales, int_high) -> torch.Tensor:
    if decl.role == "int_table":
        kind, a, dt = "int", float(int_high), torch.int32
    elif decl.role == "norm_weight":
        kind, a, dt = "around_one", scales.norm_spread, dtype
    elif decl.role == "bias":
        kind, a, dt = "normal", scales.bias_std, dtype
    elif decl.role == "matrix":
        kind, a, dt = "normal", scales.matrix_std, dtype
    else:
        raise QStreamError(QsError.INTERNAL, f"unknown tensor role '{decl.role}' for {name}")
    key = tensor_key(seed, name)
    shape = tuple(decl.shape)
    n = math.prod(shape)
    if device.type == "cuda":
        from ..csrc import ops
        out = torch.empty(shape, dtype=dt, device=device)
        ops.random_fill(out, key, _KINDS[kind], a)
        return out
    out = torch.empty(n, dtype=dt)
    for first in range(0, n, _HOST_CHUNK):          # bounded staging for very large tables
        m = min(_HOST_CHUNK, n - first)
        out[first:first + m] = torch.from_numpy(host_values(key, kind, a, first, m)).to(dt)
    return out.reshape(shape)


def random_tensors(wanted: Mapping[str, TensorDecl], seed: int, dtype: torch.dtype,
                   device="cpu", scales: InitScales = InitScales(),
                   int_high: int = 2) -> dict[str, torch.Tensor]:
    """Tensors for every declaration, made where they are to live (the device kernel or
    its host twin).  Values are drawn in float32 and rounded once to `dtype`."""
    dev = torch.device(device)
    return {name: _fill(name, decl, seed, dtype, dev, scales, int_high) for name, decl in wanted.items()}


def write_model_folder(folder, config, seed: int, dtype="bfloat16",
                       scales: InitScales = InitScales(), device="cpu") -> Path:
    """Write `config.json` and `model.safetensors` for `config` with random weights.
    `device`: where the values are made ("cuda": by the kernel, which is much faster for a
    large model; the file is the same bit for bit)."""
    from ..engine.model import declared_tensors      # the model says what it holds
    torch_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32,
                   torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}.get(dtype)
    if torch_dtype is None:
        raise QStreamError(QsError.INVALID_INPUT, f"dtype {dtype!r}: want bfloat16 or float32")
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    wanted = declared_tensors(config.model_spec())
    tensors = random_tensors(wanted, seed, torch_dtype, device, scales)
    if torch.device(device).type != "cpu":
        tensors = {k: v.cpu() for k, v in tensors.items()}
    d = config.to_dict()
    d["torch_dtype"] = "bfloat16" if torch_dtype == torch.bfloat16 else "float32"
    (folder / "config.json").write_text(json.dumps(d, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": seed})
    return folder
