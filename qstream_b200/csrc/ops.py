"""Python face of the kernel library: one function per `extern "C"` entry point.

Tensors are torch CUDA tensors used as typed device buffers; every launch goes on
torch's current stream, so the calls can be captured in a CUDA graph.  There is no
other implementation behind these functions: if the library cannot be built or
loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from ..errors import QsError, QStreamError
from . import build as _build

F32, BF16 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACTIVATIONS = {None: ACT_NONE, "none": ACT_NONE, "gelu_new": ACT_GELU_TANH, "gelu": ACT_GELU_ERF}

_lib = None

_SIGNATURES = {
    "qs_abi_version": ([], c_int),
    "qs_embedding": ([c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p], c_int),
    "qs_layernorm": ([c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                      c_longlong, c_longlong, c_int, c_void_p], c_int),
    "qs_gather_rows": ([c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p], c_int),
    "qs_add": ([c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p], c_int),
    "qs_linear_simt": ([c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                        c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p], c_int),
    "qs_rope_store": ([c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_longlong,
                       c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                       c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p], c_int),
    "qs_attention": ([c_void_p, c_void_p, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p,
                      c_void_p], c_int),
    "qs_argmax": ([c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p], c_int),
    "qs_repeat_penalty": ([c_void_p, c_int, c_int, c_longlong, c_void_p, c_int, c_void_p, c_float, c_void_p], c_int),
    "qs_sample": ([c_void_p, c_void_p, c_int, c_int, c_longlong, c_float, c_int, c_float, c_void_p, c_void_p], c_int),
    "qs_random_fill": ([c_void_p, c_int, c_longlong, c_ulonglong, c_int, c_double, c_longlong, c_void_p], c_int),
    "qs_convert": ([c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p], c_int),
    "qs_check_finite": ([c_void_p, c_int, c_int, c_int, c_longlong, c_int, c_void_p, c_void_p, c_void_p], c_int),
    "qs_canary_fill": ([c_void_p, c_longlong, c_uint, c_void_p], c_int),
    "qs_canary_check": ([c_void_p, c_longlong, c_uint, c_void_p, c_void_p], c_int),
    "qs_selftest_bounded_wait": ([c_void_p, c_int, c_void_p], c_int),
    "qs_take_tokens": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p], c_int),
    "qs_zero_pages": ([c_void_p, c_longlong, c_longlong, c_int, c_void_p, c_int, c_int, c_void_p], c_int),
}


def library():
    """The loaded kernel library; built on first use."""
    global _lib
    if _lib is None:
        path = _build.build()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise QStreamError(QsError.INTERNAL, f"cannot load {path}: {e}") from None
        lib.qs_last_error.restype = ctypes.c_char_p
        lib.qs_last_error.argtypes = []
        for name, (argtypes, restype) in _SIGNATURES.items():
            if not hasattr(lib, name):
                continue                    # optional entry points are bound by their own modules
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib


def bind(name: str, argtypes, restype=c_int):
    """Bind one more entry point (used by modules that own further kernels)."""
    lib = library()
    try:
        fn = getattr(lib, name)
    except AttributeError:
        raise QStreamError(QsError.INTERNAL, f"the kernel library has no entry point '{name}'") from None
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


_launches = 0


def launch_count() -> int:
    """How many kernels of the library have been launched (replayed graph nodes included)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def check(rc: int) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        detail = library().qs_last_error().decode(errors="replace")
        try:
            code = QsError(rc)
        except ValueError:
            code = QsError.INTERNAL
        raise QStreamError(code, detail)


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise QStreamError(QsError.INVALID_INPUT, f"kernels take float32 or bfloat16, got {t.dtype}")


def ptr(t) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise QStreamError(QsError.INVALID_INPUT, "kernels run on CUDA tensors only; there is no CPU path")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """The current CUDA stream's handle (the capturing stream while a graph is captured)."""
    if _raw_stream is not None:                       # a plain C call: the Stream object costs ten times as much
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _rows(t: torch.Tensor):
    """(rows, width, row stride) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise QStreamError(QsError.INVALID_INPUT, f"need a 2-D tensor with contiguous rows, got "
                           f"shape {tuple(t.shape)} strides {t.stride()}")
    return t.shape[0], t.shape[1], t.stride(0)


def _int32(t: torch.Tensor, what: str):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, f"{what} must be a contiguous int32 tensor")
    return ptr(t)


# ------------------------------------------------------------------------------- wrappers

def embedding(table: torch.Tensor, tokens: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    V, D = table.shape
    T = tokens.numel()
    out = torch.empty((T, D), dtype=out_dtype, device=table.device)
    check(library().qs_embedding(ptr(out), dtype_code(out), ptr(table), dtype_code(table),
                                 _int32(tokens, "tokens"), T, D, V, stream()))
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias, eps: float, out=None, settled=False) -> torch.Tensor:
    """`settled`: weight and bias were complete before the previous kernel of the stream began (a model's
    are); the kernel then fetches them while that kernel still runs."""
    rows, D, ldx = _rows(x)
    if out is None:
        out = torch.empty((rows, D), dtype=x.dtype, device=x.device)
    _, _, ldo = _rows(out)
    if weight.numel() != D or (bias is not None and bias.numel() != D):
        raise QStreamError(QsError.INVALID_INPUT, f"layernorm: width {D} but weight {tuple(weight.shape)}")
    check(library().qs_layernorm(ptr(out), ptr(x), dtype_code(x), ptr(weight), dtype_code(weight),
                                 ptr(bias), dtype_code(bias) if bias is not None else 0, rows, D,
                                 float(eps), ldx, ldo, int(bool(settled)), stream()))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _, D, ldx = _rows(x)
    n = rows.numel()
    out = torch.empty((n, D), dtype=x.dtype, device=x.device)
    check(library().qs_gather_rows(ptr(out), ptr(x), dtype_code(x), _int32(rows, "rows"), n, D, ldx, stream()))
    return out


def add(a: torch.Tensor, b: torch.Tensor, c=None) -> torch.Tensor:
    for t in (b, c):
        if t is not None and (t.shape != a.shape or t.dtype != a.dtype or not t.is_contiguous()):
            raise QStreamError(QsError.INVALID_INPUT, "add: operands differ in shape, type or layout")
    if not a.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "add: operands must be contiguous")
    out = torch.empty_like(a)
    check(library().qs_add(ptr(out), ptr(a), ptr(b), ptr(c), dtype_code(a), a.numel(), stream()))
    return out


def linear_simt(x, weight, bias=None, activation=None, residuals=(), out_dtype=None, out=None) -> torch.Tensor:
    """act(x W^T + bias) + residuals, accumulated in true 32-bit on the CUDA cores."""
    M, K, lda = _rows(x)
    N, K2 = weight.shape
    if K2 != K or not weight.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, f"linear: x is [{M}, {K}] but weight is {tuple(weight.shape)}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    elif out.shape != (M, N) or out.stride(1) != 1:
        raise QStreamError(QsError.INVALID_INPUT, "linear: the output view does not fit")
    res = list(residuals) + [None, None]
    ldr = N
    for r in res[:2]:
        if r is not None:
            if r.shape != (M, N) or r.dtype != x.dtype or r.stride(1) != 1:
                raise QStreamError(QsError.INVALID_INPUT, "linear: residual differs in shape or type")
            ldr = r.stride(0)
    if len(residuals) > 2 or (len(residuals) == 2 and res[0].stride(0) != res[1].stride(0)):
        raise QStreamError(QsError.INVALID_INPUT, "linear: at most two residuals of one layout")
    check(library().qs_linear_simt(ptr(out), dtype_code(out), ptr(x), dtype_code(x), ptr(weight),
                                   dtype_code(weight), ptr(bias), dtype_code(bias) if bias is not None else 0,
                                   ACTIVATIONS[activation], ptr(res[0]), ptr(res[1]), M, N, K, lda, out.stride(0), ldr,
                                   stream()))
    return out


def rope_store(q, k, v, n_heads, n_kv_heads, head_dim, rotary_dim, cos_sin, tok_slot, tok_pos,
               page_table, page_tokens, k_cache, v_cache, status, settled=False) -> None:
    """Rotate q (in place) and k, and write k and v into the paged cache entry.
    k = v = None (n_kv_heads = 0): rotate q only (no page table is needed then).
    `settled`: slots, positions, page table and the table of angles were complete before the previous kernel
    of the stream began (a step's own are); the kernel then reads them early."""
    ref = k if k is not None else q
    T = ref.shape[0]
    max_pos = cos_sin.shape[0] if cos_sin is not None else 0
    check(library().qs_rope_store(
        ptr(q), ptr(k), ptr(v), dtype_code(ref), q.stride(0) if q is not None else 0,
        k.stride(0) if k is not None else 0, v.stride(0) if v is not None else 0,
        n_heads if q is not None else 0, n_kv_heads, head_dim, rotary_dim if cos_sin is not None else 0,
        ptr(cos_sin), max_pos, _int32(tok_slot, "tok_slot"), _int32(tok_pos, "tok_pos"),
        _int32(page_table, "page_table") if page_table is not None else None,
        page_table.shape[1] if page_table is not None else 0, page_tokens, ptr(k_cache), ptr(v_cache), T,
        ptr(status), int(bool(settled)), stream()))


def attention(q, n_heads, n_kv_heads, head_dim, scale, window, tok_slot, tok_pos, page_table,
              page_tokens, k_cache, v_cache, status, out=None) -> torch.Tensor:
    """Causal attention of every token over its sequence's cache (generic kernel)."""
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=q.dtype, device=q.device)
    check(library().qs_attention(
        ptr(out), ptr(q), dtype_code(q), out.stride(0), q.stride(0), ptr(k_cache), ptr(v_cache),
        _int32(page_table, "page_table"), page_table.shape[1], page_tokens, _int32(tok_slot, "tok_slot"),
        _int32(tok_pos, "tok_pos"), T, n_heads, n_kv_heads, head_dim, float(scale), int(window),
        ptr(status), stream()))
    return out


def argmax(logits: torch.Tensor, out=None) -> torch.Tensor:
    rows, V, ld = _rows(logits)
    if logits.dtype != torch.float32:
        raise QStreamError(QsError.INVALID_INPUT, "argmax: logits must be float32")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(library().qs_argmax(ptr(out), ptr(logits), rows, V, ld, stream()))
    return out


def repeat_penalty(logits, recent, n_recent, penalty: float) -> None:
    rows, V, ld = _rows(logits)
    check(library().qs_repeat_penalty(ptr(logits), rows, V, ld, _int32(recent, "recent"), recent.shape[1],
                                      _int32(n_recent, "n_recent"), float(penalty), stream()))


def sample(logits, temperature: float, top_k: int, top_p: float, draws, out=None) -> torch.Tensor:
    rows, V, ld = _rows(logits)
    if logits.dtype != torch.float32 or draws.dtype != torch.float32 or draws.numel() != rows:
        raise QStreamError(QsError.INVALID_INPUT, "sample: logits and draws must be float32, one draw per row")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(library().qs_sample(ptr(out), ptr(logits), rows, V, ld, float(temperature), int(top_k),
                              float(top_p), ptr(draws), stream()))
    return out


# ------------------------------------------------------------------------------- utility kernels

_FILL_TYPES = {torch.float32: 0, torch.bfloat16: 1, torch.int32: 2}
_CONVERT_IN = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def random_fill(out: torch.Tensor, key: int, kind: int, a: float, first: int = 0) -> torch.Tensor:
    """Fill `out` (contiguous; float32, bfloat16 or int32) with elements first.. of the stream `key`:
    kind 0 N(0, a), kind 1 1 + U(-a, a), kind 2 integers below a."""
    if not out.is_contiguous() or out.dtype not in _FILL_TYPES:
        raise QStreamError(QsError.INVALID_INPUT, "random fill: need a contiguous float32, bfloat16 or int32 tensor")
    check(library().qs_random_fill(ptr(out), _FILL_TYPES[out.dtype], out.numel(), int(key) & (2**64 - 1), int(kind),
                                   float(a), int(first), stream()))
    return out


def convert(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """A copy of `src` (float32, bfloat16 or float16, contiguous) in float32 or bfloat16, rounded to
    nearest even."""
    if not src.is_contiguous() or src.dtype not in _CONVERT_IN or dtype not in (torch.float32, torch.bfloat16):
        raise QStreamError(QsError.INVALID_INPUT, f"convert: {src.dtype} -> {dtype} is not offered")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    check(library().qs_convert(ptr(out), _FILL_TYPES[dtype], ptr(src), _CONVERT_IN[src.dtype], src.numel(), stream()))
    return out


def check_finite(x: torch.Tensor, tag: int, record: torch.Tensor, row_slot=None) -> None:
    """Scan x [rows, width]; the first value that is not finite sets record = (1, tag, row, column).
    Rows with a negative `row_slot` entry are skipped."""
    rows, width, ld = _rows(x)
    check(library().qs_check_finite(ptr(x), dtype_code(x), rows, width, ld, int(tag),
                                    _int32(row_slot, "row_slot") if row_slot is not None else None,
                                    _int32(record, "record"), stream()))


def canary_fill(words: torch.Tensor, pattern: int) -> None:
    check(library().qs_canary_fill(ptr(words), words.numel() * words.element_size() // 4, pattern & 0xFFFFFFFF, stream()))


def canary_check(words: torch.Tensor, pattern: int, damaged: torch.Tensor) -> None:
    """Adds the number of damaged guard words to damaged[0] (int32 [2] on the device)."""
    check(library().qs_canary_check(ptr(words), words.numel() * words.element_size() // 4, pattern & 0xFFFFFFFF,
                                    _int32(damaged, "damaged"), stream()))


def take_tokens(dst: torch.Tensor, src: torch.Tensor, idx: torch.Tensor, n: int) -> None:
    """dst[j] = src[idx[j]] for j < n where idx[j] >= 0 (all int32, on the device)."""
    check(library().qs_take_tokens(_int32(dst, "dst"), _int32(src, "src"), _int32(idx, "idx"), int(n),
                                   src.numel(), stream()))


def zero_pages(storage: torch.Tensor, pages: torch.Tensor) -> None:
    """Zero the listed pages (int32, device) of every entry of a cache tensor [entries, pages, ...]."""
    if not storage.is_contiguous():
        raise QStreamError(QsError.INVALID_INPUT, "zero pages: the cache tensor must be contiguous")
    page_bytes = storage.stride(1) * storage.element_size()
    check(library().qs_zero_pages(ptr(storage), storage.stride(0) * storage.element_size(), page_bytes,
                                  storage.shape[0], _int32(pages, "pages"), pages.numel(), storage.shape[1], stream()))


def selftest_bounded_wait(status: torch.Tensor, polls: int = 2000) -> None:
    """Launch a kernel that waits, with the library's polling loop, on a barrier nothing completes: after
    `polls` polls it records code 199 in `status` (int32 on the device) and returns."""
    check(library().qs_selftest_bounded_wait(_int32(status, "status"), int(polls), stream()))
