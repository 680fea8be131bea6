"""Small helpers shared by the ops (src/bastile/ops/utils.py:8-25)."""

from __future__ import annotations

_sm_count = 0


def get_sm_count() -> int:
    """Number of SMs of the current CUDA device (cached)."""
    global _sm_count
    if _sm_count == 0:
        from .._lib import get_lib

        _sm_count = int(get_lib().bt_sm_count())
    return _sm_count


def next_power_of_2(n: int) -> int:
    return 1 if n <= 0 else 1 << (n - 1).bit_length()


def ceildiv(a: int, b: int) -> int:
    return -(a // -b)
