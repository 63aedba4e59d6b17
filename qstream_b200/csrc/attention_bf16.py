"""bfloat16 attention kernels specialised for decode and for prefill."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import ops

_decode = None
_scratch_size = None
_prefill = None


def _bind():
    global _decode, _scratch_size
    if _decode is None:
        _scratch_size = ops.bind("qs_attention_decode_scratch", [c_int, c_int, c_int, c_int], c_longlong)
        _decode = ops.bind("qs_attention_decode", [
            c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p,
            c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p])


def decode(q, n_heads, n_kv_heads, head_dim, scale, window, tok_slot, tok_pos, page_table, page_tokens,
           k_cache, v_cache, max_context, status, out=None) -> torch.Tensor:
    """One query token per row against the paged cache, split over the keys and merged."""
    _bind()
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    n = _scratch_size(T, n_heads, head_dim, max_context)
    scratch = torch.empty((n,), dtype=torch.float32, device=q.device)
    ops.check(_decode(ops.ptr(out), out.stride(0), ops.ptr(q), q.stride(0), ops.ptr(k_cache), ops.ptr(v_cache),
                      ops.ptr(page_table), page_table.shape[1], page_tokens, ops.ptr(tok_slot), ops.ptr(tok_pos),
                      T, n_heads, n_kv_heads, head_dim, float(scale), int(window), int(max_context),
                      ops.ptr(scratch), ops.ptr(status), ops.stream()))
    ops.count_launches(1)                                   # split kernel + merge kernel
    return out


def prefill_tiles(batch, device) -> torch.Tensor:
    """The step's query rows cut into pieces of at most 128 rows of one sequence:
    int32 [n, 4] = (first packed row, rows, position of the first row, slot), longest context first."""
    cached = getattr(batch, "_prefill_tiles", None)
    if cached is not None:
        return cached
    tiles, row = [], 0
    for slot, n, p0 in zip(batch.slots, batch.new_tokens, batch.p0):
        for a in range(0, n, 128):
            tiles.append((row + a, min(128, n - a), p0 + a, slot))
        row += n
    tiles.sort(key=lambda t: -(t[2] + t[1]))
    t = torch.tensor(tiles, dtype=torch.int32).reshape(-1, 4)
    t = t.pin_memory().to(device, non_blocking=True) if device.type == "cuda" else t
    batch._prefill_tiles = t
    return t


def prefill(q, n_heads, n_kv_heads, head_dim, scale, window, tiles, page_table, page_tokens, k_cache, v_cache,
            status, padded=False, out=None) -> torch.Tensor:
    """Many query rows per sequence against the paged cache on the tensor cores (tcgen05)."""
    global _prefill
    if _prefill is None:
        _prefill = ops.bind("qs_attention_prefill", [
            c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
            c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
    T = q.shape[0]
    # rows that belong to no sequence (padding) are covered by no tile: give them a defined value
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    if padded:
        out.zero_()
    ops.check(_prefill(ops.ptr(out), out.stride(0), ops.ptr(q), q.stride(0), T, ops.ptr(k_cache), ops.ptr(v_cache),
                       k_cache.shape[0], ops.ptr(page_table), page_table.shape[1], page_tokens, ops.ptr(tiles),
                       tiles.shape[0], n_heads, n_kv_heads, head_dim, float(scale), int(window), ops.ptr(status),
                       ops.stream()))
    return out


def attend(q, spec, step, view, out=None):
    """The specialised kernel's output, or None if the generic kernel is to run."""
    b = step.batch
    if (b.decode and view.page_tokens == 64 and spec.head_dim % 8 == 0 and spec.head_dim <= 512
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
        # the grid covers the longest sequence of the step (a captured step: the bound it was captured for),
        # not the longest the cache allows: splits beyond it would be CTAs that start only to leave
        reach = min(b.max_total or step.cache.max_context, step.cache.max_context)
        return decode(q, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.scale, spec.window, b.tok_slot,
                      b.tok_pos, view.page_table, view.page_tokens, view.k, view.v, reach,
                      step.status, out=out)
    if (not b.decode and b.slots and view.page_tokens == 64 and spec.head_dim % 16 == 0 and spec.head_dim <= 256
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
        tiles = prefill_tiles(b, q.device)
        return prefill(q, spec.n_heads, spec.n_kv_heads, spec.head_dim, spec.scale, spec.window, tiles,
                       view.page_table, view.page_tokens, view.k, view.v, step.status,
                       padded=b.n_tokens != sum(b.new_tokens), out=out)
    return None
