"""The tensor-core matrix product (tcgen05 + TMA) for bfloat16 operands."""
from __future__ import annotations


def takes(x, weight) -> bool:
    """Whether the tensor-core kernel takes these operands."""
    return False
