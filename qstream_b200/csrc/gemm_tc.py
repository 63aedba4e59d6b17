"""The tensor-core matrix product (tcgen05 + TMA) for bfloat16 operands."""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_void_p

import torch

from ..errors import QsError, QStreamError
from . import ops

_fn = None
_status = {}


def _entry():
    global _fn
    if _fn is None:
        _fn = ops.bind("qs_gemm_tc", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                                      c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p])
    return _fn


def status_word(device) -> torch.Tensor:
    """A device int32 that the kernel sets if one of its bounded waits runs out."""
    key = (device.type, device.index)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


WS_FLOATS = 16 << 20            # split-K partial tiles: 64 MiB of float32
N_COUNTERS = 1 << 16
_scratch = {}


scratch_slot = 0                # which set of scratch the next products use (see `second_scratch`)


class second_scratch:
    """Products launched inside this context use a second set of scratch: for a stream that runs
    beside the main one (products on one stream run in order and may share a set; two streams may not)."""

    def __enter__(self):
        global scratch_slot
        self.before, scratch_slot = scratch_slot, 1

    def __exit__(self, *exc):
        global scratch_slot
        scratch_slot = self.before


smem_limit_kb = 0               # what a CTA of the weight-streaming product may take of its SM's shared memory (0 = all)


class shared_sms:
    """Products of few tokens launched inside this context take half of an SM's shared memory each, so that the
    CTAs of two of them - one on each of two streams - sit on the same SMs and stream their weights together
    instead of taking turns."""

    def __enter__(self):
        global smem_limit_kb
        self.before, smem_limit_kb = smem_limit_kb, 111

    def __exit__(self, *exc):
        global smem_limit_kb
        smem_limit_kb = self.before


def scratch(device):
    """Per-device scratch of the split-K reduction: partial tiles and zeroed arrival counters."""
    key = (device.type, device.index, scratch_slot)
    if key not in _scratch:
        _scratch[key] = (torch.empty(WS_FLOATS, dtype=torch.float32, device=device),
                         torch.zeros(N_COUNTERS, dtype=torch.int32, device=device))
    return _scratch[key]


def check_status(device) -> None:
    code = int(status_word(torch.device(device)).item())
    if code:
        status_word(torch.device(device)).zero_()
        raise QStreamError(QsError.INTERNAL, f"tensor-core matrix product: a wait inside the kernel ran out (code {code})")


def takes(x, weight) -> bool:
    """Whether the tensor-core kernel takes these operands: bfloat16, rows of 16-byte pitch (the matrix may
    be a range of columns of a wider one)."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and weight.dim() == 2 and weight.stride(1) == 1 and weight.stride(0) % 8 == 0
            and weight.stride(0) >= weight.shape[1] and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def linear(x, weight, bias=None, activation=None, residuals=(), out_dtype=None, out=None) -> torch.Tensor:
    M, K = x.shape
    N, K2 = weight.shape
    if K2 != K:
        raise QStreamError(QsError.INVALID_INPUT, f"linear: x is [{M}, {K}] but weight is {tuple(weight.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=x.device)
    elif out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise QStreamError(QsError.INVALID_INPUT, "linear: the output view does not fit")
    res = [r for r in residuals if r is not None]
    if len(res) > 2:
        raise QStreamError(QsError.INVALID_INPUT, "linear: at most two residuals")
    ldr = N
    for r in res:
        if r.shape != (M, N) or r.dtype != torch.bfloat16 or r.stride(1) != 1:
            raise QStreamError(QsError.INVALID_INPUT, "linear: residual differs in shape or type")
        ldr = r.stride(0)
    if len(res) == 2 and res[0].stride(0) != res[1].stride(0):
        raise QStreamError(QsError.INVALID_INPUT, "linear: residuals of two layouts")
    res += [None, None]
    ws, counters = scratch(x.device)
    ops.check(_entry()(ops.ptr(out), ops.dtype_code(out), ops.ptr(x), ops.ptr(weight), ops.ptr(bias),
                       ops.dtype_code(bias) if bias is not None else 0, ops.ACTIVATIONS[activation],
                       ops.ptr(res[0]), ops.ptr(res[1]), M, N, K, x.stride(0), weight.stride(0), out.stride(0), ldr,
                       ops.ptr(ws), ws.numel(), ops.ptr(counters), counters.numel(),
                       ops.ptr(status_word(x.device)), int(smem_limit_kb), ops.stream()))
    return out
