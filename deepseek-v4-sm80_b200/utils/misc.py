"""Small arithmetic helpers (counterparts of python/minisgl/utils/misc.py:4-48 of the reference)."""
from __future__ import annotations


class _Unset:
    def __repr__(self):
        return "UNSET"

    def __bool__(self):
        return False


UNSET = _Unset()


def div_ceil(a: int, b: int) -> int:
    return (a + b - 1) // b


def align_ceil(a: int, b: int) -> int:
    return div_ceil(a, b) * b


def align_down(a: int, b: int) -> int:
    return a // b * b


def div_even(a: int, b: int, allow_replicate: bool = False) -> int:
    """a / b when it divides evenly; with allow_replicate a < b with b % a == 0 yields 1 (each of the a units is
    replicated on b / a ranks, e.g. one KV head shared by every tensor-parallel rank)."""
    if allow_replicate and a < b and b % a == 0:
        return 1
    if a % b != 0:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


def call_if_main(name: str):
    def deco(fn):
        if name == "__main__":
            fn()
        return fn

    return deco
