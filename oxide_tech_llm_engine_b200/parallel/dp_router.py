"""Data-parallel replicas behind one front: request routing by prefix affinity and free KV.

Each replica is a complete engine (itself possibly TP/EP over several GPUs). A request goes to
the replica that most recently served the same prompt prefix (so the radix cache hits), unless
that replica is much busier than the least loaded one. The reference only has a `dp_size` field
(oxide-engine/src/distributed.rs:17,66-67).
"""
from __future__ import annotations

import threading
from collections import OrderedDict
from typing import Sequence

from ..engine.kv_tiers import fnv1a_chain


class DpRouter:
    def __init__(self, replicas: Sequence, affinity_tokens: int = 64, max_tracked: int = 4096,
                 imbalance: int = 4):
        self.replicas = list(replicas)  # EngineHandle-like: submit(), active_slots(), engine.sched
        self.affinity_tokens, self.imbalance = affinity_tokens, imbalance
        self.seen: "OrderedDict[int, int]" = OrderedDict()
        self.max_tracked = max_tracked
        self._lock = threading.Lock()
        self.routed = [0] * len(self.replicas)

    def _load(self, i: int) -> int:
        return self.replicas[i].active_slots()

    def pick(self, prompt_tokens) -> int:
        key = fnv1a_chain(0, list(prompt_tokens[: self.affinity_tokens]))
        with self._lock:
            loads = [self._load(i) for i in range(len(self.replicas))]
            least = min(range(len(loads)), key=lambda i: (loads[i], i))
            choice = self.seen.get(key)
            if choice is None or loads[choice] - loads[least] > self.imbalance:
                choice = least
            self.seen[key] = choice
            self.seen.move_to_end(key)
            while len(self.seen) > self.max_tracked:
                self.seen.popitem(last=False)
            self.routed[choice] += 1
            return choice

    def submit(self, prompt_tokens, params, **kw):
        i = self.pick(prompt_tokens)
        return i, self.replicas[i].submit(prompt_tokens, params, **kw)


class DpHandle:
    """Several engine replicas behind the `EngineHandle` interface the HTTP server uses: `submit`
    routes by prefix affinity and load, `cancel` goes to the replica that owns the request, health and
    slot counts aggregate. Each replica is a full engine (its own GPU or TP group, its own thread)."""

    def __init__(self, handles: Sequence, **router_kw):
        if not handles:
            raise ValueError("DpHandle needs at least one replica")
        self.handles = list(handles)
        self.router = DpRouter(self.handles, **router_kw)
        self._owner: dict = {}
        self._lock = threading.Lock()

    # the server reads these
    @property
    def engine(self):
        return self.handles[0].engine

    @property
    def max_slots(self) -> int:
        return sum(h.max_slots for h in self.handles)

    @property
    def healthy(self) -> bool:
        return all(h.healthy for h in self.handles)

    def active_slots(self) -> int:
        return sum(h.active_slots() for h in self.handles)

    def submit(self, prompt_tokens, params, **kw):
        i = self.router.pick(prompt_tokens)
        st = self.handles[i].submit(prompt_tokens, params, **kw)
        with self._lock:
            self._owner[(i, st.req_id)] = i
        st.replica = i
        return st

    def cancel(self, req_id: int, replica: int = 0) -> None:
        self.handles[replica].cancel(req_id)

    def generate(self, prompt_tokens, params, timeout: float = 600.0):
        i = self.router.pick(prompt_tokens)
        return self.handles[i].generate(prompt_tokens, params, timeout=timeout)

    def shutdown(self, timeout: float = 10.0) -> None:
        for h in self.handles:
            h.shutdown(timeout)
