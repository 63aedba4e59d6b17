"""Error codes and the exception that carries them.

The codes and their order follow QStream's `QSFError` (include/qsf/error.h:14-32)
so that a caller who knows the reference finds the same names; the detail string
plays the part of its thread-local detail buffer (src/error.c:14-53).
"""
from __future__ import annotations

import enum


class QsError(enum.IntEnum):
    OK = 0
    FILE_NOT_FOUND = 1
    FILE_CORRUPTED = 2
    FILE_VERSION = 3
    OUT_OF_MEMORY = 4
    BUDGET_EXCEEDED = 5
    INVALID_MODEL = 6
    QUANT_MISMATCH = 7
    IO_FAILURE = 8
    DECOMPRESSION = 9
    NAN_DETECTED = 10
    INVALID_INPUT = 11
    SEQ_TOO_LONG = 12
    UNSUPPORTED_ARCH = 13
    THREAD_FAILURE = 14
    INTERNAL = 15


_STRINGS = {
    QsError.OK: "success",
    QsError.FILE_NOT_FOUND: "file not found",
    QsError.FILE_CORRUPTED: "file corrupted",
    QsError.FILE_VERSION: "unsupported file version",
    QsError.OUT_OF_MEMORY: "out of memory",
    QsError.BUDGET_EXCEEDED: "memory budget exceeded",
    QsError.INVALID_MODEL: "invalid model",
    QsError.QUANT_MISMATCH: "quantization mismatch",
    QsError.IO_FAILURE: "I/O failure",
    QsError.DECOMPRESSION: "decompression failure",
    QsError.NAN_DETECTED: "NaN or Inf detected",
    QsError.INVALID_INPUT: "invalid input",
    QsError.SEQ_TOO_LONG: "sequence too long",
    QsError.UNSUPPORTED_ARCH: "unsupported architecture",
    QsError.THREAD_FAILURE: "thread failure",
    QsError.INTERNAL: "internal error",
}


def error_string(code: QsError) -> str:
    return _STRINGS[QsError(code)]


class QStreamError(Exception):
    """Every failure of the library: a code of `QsError` and a detail string."""

    def __init__(self, code: QsError, detail: str = ""):
        self.code = QsError(code)
        self.detail = detail
        super().__init__(f"[qstream] {error_string(self.code)}: {detail}" if detail
                         else f"[qstream] {error_string(self.code)}")
