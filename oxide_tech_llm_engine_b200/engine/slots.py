"""Slot manager, request typestate and device/host arenas (thin API-parity layer).

Reference parity: ContinuousBatchingSlotManager with Idle/Prefill/Decode/Finished slots and
fixed-chunk scheduling (oxide-engine/src/slot_manager.rs:12-21,117-240; the server uses it as a
concurrency lease, oxide-server/src/lib.rs:203-250), the request typestate
Unallocated->Allocated->Prefilling->Decoding->Terminal (oxide-core/src/typestate.rs:5-114) as a
runtime state machine, DeviceMemoryArena slot binding with start-up budget calibration
(oxide-alloc/src/device_arena.rs:7-144) and the bump HostPinnedArena (host_arena.rs:6-106).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from enum import Enum
from typing import Optional

from ..errors import EngineError, OutOfMemory, SlotsExhausted


class SlotState(Enum):
    IDLE = "idle"
    PREFILL = "prefill"
    DECODE = "decode"
    FINISHED = "finished"


@dataclass
class Slot:
    index: int
    state: SlotState = SlotState.IDLE
    request_id: Optional[int] = None
    prompt_len: int = 0
    prefilled: int = 0
    generated: int = 0


class SlotManager:
    def __init__(self, max_slots: int, chunk_size: int = 512):
        self.slots = [Slot(i) for i in range(max_slots)]
        self.max_slots, self.chunk_size = max_slots, chunk_size
        self._lock = threading.Lock()

    def total_active_slots(self) -> int:
        return sum(1 for s in self.slots if s.state != SlotState.IDLE)

    def lease(self, request_id: int, prompt_len: int) -> Slot:
        with self._lock:
            for s in self.slots:
                if s.state == SlotState.IDLE:
                    s.state, s.request_id, s.prompt_len, s.prefilled, s.generated = \
                        SlotState.PREFILL, request_id, prompt_len, 0, 0
                    return s
        raise SlotsExhausted("All inference slots busy (concurrency limit reached)")

    def next_chunk(self, slot: Slot) -> int:
        """Tokens of the next fixed-size prefill chunk (0 once the prompt is done)."""
        n = min(self.chunk_size, slot.prompt_len - slot.prefilled)
        slot.prefilled += n
        if slot.prefilled >= slot.prompt_len:
            slot.state = SlotState.DECODE
        return n

    def on_token(self, slot: Slot, finished: bool) -> None:
        slot.generated += 1
        if finished:
            slot.state = SlotState.FINISHED

    def release(self, slot: Slot) -> None:
        with self._lock:
            slot.state, slot.request_id = SlotState.IDLE, None

    class Lease:
        """RAII-style lease: `with mgr.leased(rid, n) as slot:` always frees the slot."""

        def __init__(self, mgr, rid, n):
            self.mgr, self.slot = mgr, mgr.lease(rid, n)

        def __enter__(self):
            return self.slot

        def __exit__(self, *exc):
            self.mgr.release(self.slot)
            return False

    def leased(self, request_id: int, prompt_len: int) -> "SlotManager.Lease":
        return SlotManager.Lease(self, request_id, prompt_len)


class RequestPhase(Enum):
    UNALLOCATED = 0
    ALLOCATED = 1
    PREFILLING = 2
    DECODING = 3
    TERMINAL = 4


_ALLOWED = {
    RequestPhase.UNALLOCATED: {RequestPhase.ALLOCATED, RequestPhase.TERMINAL},
    RequestPhase.ALLOCATED: {RequestPhase.PREFILLING, RequestPhase.TERMINAL},
    RequestPhase.PREFILLING: {RequestPhase.PREFILLING, RequestPhase.DECODING, RequestPhase.TERMINAL},
    RequestPhase.DECODING: {RequestPhase.DECODING, RequestPhase.TERMINAL, RequestPhase.ALLOCATED},
    RequestPhase.TERMINAL: set(),
}


class RequestLifecycle:
    """Run-time version of the compile-time typestate: illegal transitions raise."""

    def __init__(self):
        self.phase = RequestPhase.UNALLOCATED

    def to(self, nxt: RequestPhase) -> "RequestLifecycle":
        if nxt not in _ALLOWED[self.phase]:
            raise EngineError(f"illegal request transition {self.phase.name} -> {nxt.name}")
        self.phase = nxt
        return self


class DeviceMemoryArena:
    """Carves a byte budget into equal slots; `calibrate` sizes the budget from free memory."""

    def __init__(self, budget_bytes: int, slot_bytes: int):
        self.slot_bytes = slot_bytes
        self.n_slots = budget_bytes // max(slot_bytes, 1)
        self.bound: dict[int, int] = {}

    @classmethod
    def calibrate(cls, free_bytes: int, reserve_bytes: int, slot_bytes: int, utilisation: float = 0.9):
        return cls(max(int(free_bytes * utilisation) - reserve_bytes, 0), slot_bytes)

    def bind(self, owner: int) -> int:
        for i in range(self.n_slots):
            if i not in self.bound.values():
                self.bound[owner] = i
                return i * self.slot_bytes
        raise OutOfMemory("device arena has no free slot")

    def unbind(self, owner: int) -> None:
        self.bound.pop(owner, None)


class HostPinnedArena:
    """Bump allocator over one pinned host buffer (staging for H2D copies)."""

    def __init__(self, nbytes: int, pin: bool = True):
        import torch

        self.buf = torch.empty(nbytes, dtype=torch.uint8, pin_memory=pin and torch.cuda.is_available())
        self.off = 0

    def alloc(self, nbytes: int, align: int = 64):
        start = (self.off + align - 1) // align * align
        if start + nbytes > self.buf.numel():
            raise OutOfMemory("host arena exhausted")
        self.off = start + nbytes
        return self.buf[start:start + nbytes]

    def reset(self) -> None:
        self.off = 0
