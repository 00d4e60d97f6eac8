"""Per-rank heartbeat in host shared memory.

Every scheduler process stamps a slot of a small shared-memory board once per loop iteration (monotonic counter +
wall-clock time + a busy flag).  The frontend's health watcher reads the board: a rank whose stamp has not moved for
``timeout`` seconds *while it reports work in flight* is wedged (a hung collective, a stuck kernel wait that the
device-side limit has not yet ended, a dead-locked host thread), which process-exit polling alone cannot see.  An idle
rank blocks in its message receive and is not expected to beat.  The reference detects only exited children
(python/minisgl/server/supervisor.py:147-169); this adds liveness of running ones, on the host only.
"""
from __future__ import annotations

import struct
import time
from multiprocessing import shared_memory
from typing import List, Optional, Tuple

_SLOT = struct.Struct("<QdQ")  # beats, last wall time, busy flag


class HeartbeatBoard:
    def __init__(self, name: Optional[str], ranks: int, create: bool):
        self.ranks = ranks
        size = _SLOT.size * ranks
        if create:
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            self.shm.buf[:size] = bytes(size)
        else:
            self.shm = shared_memory.SharedMemory(name=name, create=False)
        self.name = self.shm.name
        self._owner = create

    def beat(self, rank: int, busy: bool, now: Optional[float] = None) -> None:
        off = rank * _SLOT.size
        beats, _, _ = _SLOT.unpack_from(self.shm.buf, off)
        _SLOT.pack_into(self.shm.buf, off, beats + 1, time.time() if now is None else now, 1 if busy else 0)

    def read(self, rank: int) -> Tuple[int, float, bool]:
        beats, t, busy = _SLOT.unpack_from(self.shm.buf, rank * _SLOT.size)
        return beats, t, bool(busy)

    def stale(self, timeout: float, now: Optional[float] = None) -> List[int]:
        """Ranks that reported work in flight and have not stamped for more than ``timeout`` seconds."""
        now = time.time() if now is None else now
        out = []
        for r in range(self.ranks):
            beats, t, busy = self.read(r)
            if beats and busy and now - t > timeout:
                out.append(r)
        return out

    def close(self) -> None:
        try:
            self.shm.close()
            if self._owner:
                self.shm.unlink()
        except FileNotFoundError:  # pragma: no cover
            pass
