"""Device capability probes.  This engine targets sm_100a only: its kernels use tcgen05 / TMEM / TMA instructions
that exist on no other architecture, so the gate is the mirror image of the reference's Ampere-only gate
(python/minisgl/utils/arch.py:6-35)."""
from __future__ import annotations

import functools

import torch

B200_CAPABILITIES = {(10, 0)}


@functools.lru_cache(maxsize=None)
def device_capability(index: int = 0):
    if not torch.cuda.is_available():
        return None
    return torch.cuda.get_device_capability(index)


def is_arch_supported(major: int, minor: int = 0) -> bool:
    cap = device_capability()
    return cap is not None and cap >= (major, minor)


def is_sm90_supported() -> bool:
    return is_arch_supported(9, 0)


def is_sm100_supported() -> bool:
    return is_arch_supported(10, 0)


def is_dsv4_blackwell_capability(index: int = 0) -> bool:
    return device_capability(index) in B200_CAPABILITIES


def require_blackwell(index: int = 0) -> None:
    """Called by the engine before it loads anything onto a CUDA device."""
    if not is_dsv4_blackwell_capability(index or 0):
        raise RuntimeError("the DSV4 kernels are compiled for sm_100a only; found capability "
                           f"{device_capability(index or 0)}")
