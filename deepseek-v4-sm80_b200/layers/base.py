"""Minimal parameter container: attribute-walking ``state_dict`` / ``load_state_dict`` without torch.nn.Module
(python/minisgl/layers/base.py:15-99 of the reference).  The model of this engine keeps its weights in a flat dict
(``models/weight.py``); this module exists for code that wants the reference's BaseOP-style objects, e.g. to export
the runtime tensors under the reference's parameter names."""
from __future__ import annotations

from typing import Any, Dict, Generic, Iterator, List, Tuple, TypeVar

import torch

T = TypeVar("T")


class BaseOP:
    def _walk(self, prefix: str = "") -> Iterator[Tuple[str, Any, str, Any]]:
        for name, value in vars(self).items():
            if name.startswith("_"):
                continue
            full = f"{prefix}.{name}" if prefix else name
            if isinstance(value, torch.Tensor):
                yield full, self, name, value
            elif isinstance(value, BaseOP):
                yield from value._walk(full)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {k: v for k, _, _, v in self._walk()}

    def load_state_dict(self, state: Dict[str, torch.Tensor], strict: bool = True) -> None:
        seen = set()
        for key, owner, attr, old in list(self._walk()):
            if key not in state:
                if strict:
                    raise KeyError(f"missing parameter {key}")
                continue
            new = state[key]
            if tuple(new.shape) != tuple(old.shape) or new.dtype != old.dtype:
                raise ValueError(f"{key}: expected {tuple(old.shape)} {old.dtype}, got {tuple(new.shape)} {new.dtype}")
            setattr(owner, attr, new)
            seen.add(key)
        extra = set(state) - seen
        if strict and extra:
            raise KeyError(f"unexpected parameters: {sorted(extra)[:5]}")


class OPList(BaseOP, Generic[T]):
    def __init__(self, ops: List[T]):
        self.op_list = list(ops)

    def _walk(self, prefix: str = ""):
        for i, op in enumerate(self.op_list):
            yield from op._walk(f"{prefix}.{i}" if prefix else str(i))

    def __getitem__(self, i: int) -> T:
        return self.op_list[i]

    def __len__(self) -> int:
        return len(self.op_list)

    def __iter__(self):
        return iter(self.op_list)
