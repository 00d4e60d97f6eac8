"""Name -> factory registry with argparse-friendly errors (python/minisgl/utils/registry.py:6-38 of the reference)."""
from __future__ import annotations

from typing import Callable, Dict, Generic, List, TypeVar

T = TypeVar("T")


class Registry(Generic[T]):
    def __init__(self, kind: str):
        self.kind = kind
        self._items: Dict[str, T] = {}

    def register(self, name: str) -> Callable[[T], T]:
        def deco(obj: T) -> T:
            if name in self._items:
                raise KeyError(f"{self.kind} {name!r} is already registered")
            self._items[name] = obj
            return obj

        return deco

    def __getitem__(self, name: str) -> T:
        if name not in self._items:
            raise KeyError(f"unknown {self.kind} {name!r}; supported: {self.supported_names()}")
        return self._items[name]

    def __contains__(self, name: str) -> bool:
        return name in self._items

    def supported_names(self) -> List[str]:
        return sorted(self._items)

    def assert_supported(self, name: str) -> str:
        """argparse ``type=`` hook."""
        import argparse

        if name not in self._items:
            raise argparse.ArgumentTypeError(f"unknown {self.kind} {name!r}; choose from {self.supported_names()}")
        return name
