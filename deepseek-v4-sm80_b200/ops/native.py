"""ctypes bindings to the native libraries built by :mod:`minisgl.ops.build`.

The CUDA library exports ``extern "C"`` launchers that take raw device pointers,
sizes and a ``cudaStream_t``.  There is no Python fallback for them: when a CUDA
tensor reaches an op and the library cannot be loaded, the call raises.  The
reference guards its kernels the same way ("fail closed",
python/minisgl/kernel/deepseek_v4.py:141-143,384-385).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_CUDA_LIB = None
_HOST_LIB = None


class NativeError(RuntimeError):
    pass


def cuda_lib() -> ctypes.CDLL:
    """Loads (building first if it is missing and nvcc exists) the sm_100a kernel library."""
    global _CUDA_LIB
    if _CUDA_LIB is None:
        path = _HERE / "libdsv4_b200.so"
        if not path.exists() or os.environ.get("MINISGL_REBUILD_KERNELS") == "1":
            from . import build

            build.build_cuda(verbose=False)
        _CUDA_LIB = ctypes.CDLL(str(path))
        _CUDA_LIB.dsv4_abi_version.restype = ctypes.c_int
    return _CUDA_LIB


def host_lib() -> ctypes.CDLL:
    global _HOST_LIB
    if _HOST_LIB is None:
        path = _HERE / "libdsv4_host.so"
        if not path.exists():
            from . import build

            build.build_host(verbose=False)
        _HOST_LIB = ctypes.CDLL(str(path))
        _HOST_LIB.dsv4_first_mismatch.restype = ctypes.c_int64
        _HOST_LIB.dsv4_first_mismatch.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32]
        _HOST_LIB.dsv4_host_last_error.restype = ctypes.c_char_p
    return _HOST_LIB


def ptr(t) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(code: int, what: str) -> None:
    if code != 0:
        raise NativeError(f"{what} failed with code {code}")


_LAUNCHES = [0]


def launch_count() -> int:
    """Kernel launches issued through this module so far (graph replays add their captured launches)."""
    return _LAUNCHES[0]


def add_launches(n: int) -> None:
    _LAUNCHES[0] += n


_PROFILE = {"on": False, "events": []}


def enable_profile(on: bool = True) -> None:
    """Per-launcher device timing (CUDA events around every call); for kernel-share breakdowns, not for benchmarks."""
    _PROFILE["on"] = on
    _PROFILE["events"] = []


def profile_report() -> dict:
    """{launcher: (calls, total ms)} since enable_profile(); synchronises the device."""
    torch.cuda.synchronize()
    out = {}
    for name, a, b in _PROFILE["events"]:
        c, t = out.get(name, (0, 0.0))
        out[name] = (c + 1, t + a.elapsed_time(b))
    _PROFILE["events"] = []
    return dict(sorted(out.items(), key=lambda kv: -kv[1][1]))


_ARITY = {}


def _arity(name: str):
    """Number of parameters of the exported ``dsv4_<name>`` as written in the CUDA sources (None if not found).
    ctypes cannot check a call against the C prototype; a stale argument list would read garbage pointers, so
    :func:`call` compares the count before every first call of an entry point."""
    if not _ARITY:
        import glob
        import re

        src_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
        for path in glob.glob(os.path.join(src_dir, "*.cu")):
            src = open(path, encoding="utf-8").read()
            for m in re.finditer(r"DSV4_API\s+int\s+(dsv4_\w+)\s*\(([^)]*)\)", src):
                params = m.group(2).strip()
                _ARITY[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
        _ARITY["__loaded__"] = -1
    return _ARITY.get("dsv4_" + name)


_CHECKED = set()


def call(name: str, *args) -> None:
    """Calls ``dsv4_<name>(*args, stream)`` and raises on a non-zero return code."""
    fn = getattr(cuda_lib(), "dsv4_" + name)
    if name not in _CHECKED:
        want = _arity(name)
        if want is not None and want != len(args) + 1:
            raise NativeError(f"dsv4_{name} takes {want} arguments (stream included), the caller passed {len(args) + 1}")
        _CHECKED.add(name)
    _LAUNCHES[0] += 1
    if _PROFILE["on"]:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        code = fn(*args, stream())
        b.record()
        _PROFILE["events"].append((name, a, b))
    else:
        code = fn(*args, stream())
    if code != 0:
        raise NativeError(f"dsv4_{name} failed with code {code}")


def read_status(clear: bool = True) -> list:
    """Device status word: [code, detail_a, detail_b, count, ...]; code 0 means no kernel gave up a wait."""
    buf = (ctypes.c_int * 8)()
    check(cuda_lib().dsv4_read_status(buf, ctypes.c_int(1 if clear else 0)), "dsv4_read_status")
    return list(buf)


STATUS_NAMES = {1: "wait timeout inside a kernel", 2: "index out of range", 3: "peer GPU did not answer in time"}


class DeviceStatusError(NativeError):
    """A kernel gave up a bounded wait or refused an index; results computed since are not trustworthy."""


def _raise_status(st) -> None:
    raise DeviceStatusError(f"a kernel reported status {st[0]} ({STATUS_NAMES.get(st[0], 'unknown')}; detail "
                            f"{st[1]}, {st[2]}; {st[3]} occurrences)")


def assert_device_ok() -> None:
    st = read_status()
    if st[0] != 0:
        _raise_status(st)


class StatusProbe:
    """Per-step, non-blocking view of the device status word.  ``snapshot()`` queues an 8-int device-to-host copy
    into page-locked memory on the current stream; ``check()`` -- called after the caller has synchronised with that
    stream for its own reasons (the sampled tokens' copy event) -- raises :class:`DeviceStatusError` if a kernel
    recorded a timeout or a bad index.  The serving loop calls both once per step, so a peer that stopped answering
    ends the scheduler process (and with it the server's health) instead of producing garbage tokens."""

    def __init__(self):
        self.host = torch.zeros(8, dtype=torch.int32, pin_memory=True)
        self.armed = False

    def snapshot(self) -> None:
        check(cuda_lib().dsv4_status_snapshot(ctypes.c_void_p(self.host.data_ptr()), stream()),
              "dsv4_status_snapshot")
        self.armed = True

    def check(self) -> None:
        if self.armed and int(self.host[0]) != 0:
            _raise_status([int(v) for v in self.host])


def set_peer_wait_ms(ms: int) -> None:
    """Limit of the in-kernel waits on other GPUs' flags (default 2 000 ms)."""
    check(cuda_lib().dsv4_set_peer_wait_ms(ctypes.c_longlong(int(ms))), "dsv4_set_peer_wait_ms")


I = ctypes.c_int
F = ctypes.c_float
L = ctypes.c_int64
