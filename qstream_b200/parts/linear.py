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


def shared_sms():
    """A context in which the tensor-core products of few tokens leave half of each SM to another product."""
    from ..csrc import gemm_tc
    return gemm_tc.shared_sms()


class beside_main_stream:
    """Enter a second CUDA stream that has waited for everything the current stream holds so far; products
    inside use a scratch of their own.  `join()` afterwards makes the current stream wait for the second."""

    def __init__(self, side: "torch.cuda.Stream", device):
        self.side, self.device = side, device

    def __enter__(self):
        from ..csrc import gemm_tc
        self.main = torch.cuda.current_stream(self.device)
        forked = torch.cuda.Event()
        forked.record(self.main)
        self.ctx = torch.cuda.stream(self.side)
        self.ctx.__enter__()
        self.side.wait_event(forked)
        self.scratch = gemm_tc.second_scratch()
        self.scratch.__enter__()
        return self

    def __exit__(self, *exc):
        self.scratch.__exit__(*exc)
        self.done = torch.cuda.Event()
        self.done.record(self.side)
        self.ctx.__exit__(*exc)

    def join(self):
        self.main.wait_event(self.done)
