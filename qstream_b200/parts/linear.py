"""The matrix product y = act(x W^T + b) + residuals, and the choice of its kernel.

bfloat16 activations with a bfloat16 matrix run on the tensor cores (tcgen05, fed by
TMA, 32-bit accumulation); everything else (the float32 engine, a matrix stored in
32-bit) runs on the CUDA cores in true 32-bit.  Both kernels sum a row's products in
an order that does not depend on the other rows of the batch.
"""
from __future__ import annotations

import torch

from ..csrc import ops


def linear(x, weight, bias=None, activation=None, residuals=(), out_dtype=None, out=None) -> torch.Tensor:
    """`out`: an optional view [M, N] with contiguous rows (any row stride) to write into."""
    residuals = tuple(r for r in residuals if r is not None)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        from ..csrc import gemm_tc
        if gemm_tc.takes(x, weight):
            return gemm_tc.linear(x, weight, bias, activation, residuals, out_dtype, out)
    return ops.linear_simt(x, weight, bias, activation, residuals, out_dtype, out)
