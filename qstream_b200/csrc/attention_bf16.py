"""bfloat16 attention kernels specialised for decode and for prefill."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import ops

_decode = None
_scratch_size = None


def _bind():
    global _decode, _scratch_size
    if _decode is None:
        _scratch_size = ops.bind("qs_attention_decode_scratch", [c_int, c_int, c_int, c_int], c_longlong)
        _decode = ops.bind("qs_attention_decode", [
            c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
            c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])


def decode(q, n_heads, n_kv_heads, head_dim, scale, window, tok_slot, tok_pos, page_table, page_tokens,
           k_cache, v_cache, max_context, status) -> torch.Tensor:
    """One query token per row against the paged cache, split over the keys and merged."""
    _bind()
    T = q.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    n = _scratch_size(T, n_heads, head_dim, max_context)
    scratch = torch.empty((n,), dtype=torch.float32, device=q.device)
    ops.check(_decode(ops.ptr(out), out.stride(0), ops.ptr(q), q.stride(0), ops.ptr(k_cache), ops.ptr(v_cache),
                      ops.ptr(page_table), page_table.shape[1], page_tokens, ops.ptr(tok_slot), ops.ptr(tok_pos),
                      T, n_heads, n_kv_heads, head_dim, float(scale), int(window), int(max_context),
                      ops.ptr(scratch), ops.ptr(status), ops.stream()))
    ops.count_launches(1)                                   # split kernel + merge kernel
    return out


def attend(q, spec, step, view):
    """The specialised kernel's output, or None if the generic kernel is to run."""
    b = step.batch
    if (b.decode and view.page_tokens == 64 and spec.head_dim % 8 == 0 and spec.head_dim <= 512
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
        return decode(q, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.scale, spec.window, b.tok_slot,
                      b.tok_pos, view.page_table, view.page_tokens, view.k, view.v, step.cache.max_context,
                      step.status)
    return None
