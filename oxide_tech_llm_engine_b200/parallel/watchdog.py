"""Rank liveness over a host-side key/value store: heartbeats, a monitor, typed failures.

Every rank runs a `Heartbeat` thread that bumps `hb/<rank>` in a `torch.distributed.TCPStore`
(or any object with `set`/`get`); before launching a step that contains collectives, the engine asks
`RankMonitor.check()` — a peer whose counter has not moved for `timeout_s` raises `RankFailure`, so
the survivors stop BEFORE entering a kernel that would wait on the missing peer. Device-side waits
are bounded as a second line (they return a status code, see `ops.check_status`). A rank leaves only
between steps (`Heartbeat.leave()` publishes a tombstone first), never with work in flight.

The reference has no rank-failure detection (single process); its typed error for the case is
`EngineError::HardwareFault{recoverable}` (oxide-core/src/error.rs:56-88).
"""
from __future__ import annotations

import threading
import time
from typing import Optional, Sequence

from ..errors import EngineError


class RankFailure(EngineError):
    """A peer rank stopped answering (missed heartbeats) or announced that it left."""

    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} {reason}")
        self.rank, self.reason = rank, reason


class Heartbeat:
    def __init__(self, store, rank: int, period_s: float = 0.05):
        self.store, self.rank, self.period = store, rank, period_s
        self._stop = threading.Event()
        self._n = 0
        self._thread: Optional[threading.Thread] = None
        self.beat()

    def beat(self) -> None:
        self._n += 1
        self.store.set(f"hb/{self.rank}", str(self._n))

    def start(self) -> "Heartbeat":
        def loop():
            while not self._stop.wait(self.period):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, name=f"oxb-heartbeat-{self.rank}", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def leave(self) -> None:
        """Announce an orderly exit (between steps), then stop beating."""
        self.stop()
        self.store.set(f"hb/{self.rank}", "left")


class RankMonitor:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 1.0,
                 peers: Optional[Sequence[int]] = None, clock=time.monotonic):
        self.store, self.rank, self.world, self.timeout = store, rank, world, timeout_s
        self.peers = [p for p in (peers if peers is not None else range(world)) if p != rank]
        self.clock = clock
        now = clock()
        self._last = {p: (None, now) for p in self.peers}
        self.failed: dict[int, str] = {}

    def _read(self, peer: int) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"hb/{peer}"]):
                return None
            v = self.store.get(f"hb/{peer}")
            return v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
        except Exception:
            return None

    def poll(self) -> dict[int, str]:
        """Updates and returns {rank: reason} of peers considered gone."""
        now = self.clock()
        for p in self.peers:
            if p in self.failed:
                continue
            v = self._read(p)
            if v == "left":
                self.failed[p] = "left the job"
                continue
            last_v, last_t = self._last[p]
            if v is not None and v != last_v:
                self._last[p] = (v, now)
            elif now - last_t > self.timeout:
                self.failed[p] = f"missed heartbeats for {now - last_t:.2f}s"
        return dict(self.failed)

    def check(self) -> None:
        gone = self.poll()
        if gone:
            r = min(gone)
            raise RankFailure(r, gone[r])
