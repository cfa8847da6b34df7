"""Allocation-count guard: asserts that a region of code performs no device allocation.

On CUDA it reads the caching allocator's counters (`allocation.all.allocated` counts every block the
allocator handed out, `segment.all.allocated` every `cudaMalloc`); on CPU-only hosts any object with
a `memory_stats()` method can stand in. Steady-state decode steps run out of buffers made at engine
construction, so both counters must stay put.

Reference: the counting global allocator of oxide-core/src/zero_alloc_guard.rs:11-65 and its test
(tests/test_zero_alloc_forward_decode.rs:49-85), which measures a mock executor on the host.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class AllocDelta:
    blocks: int
    segments: int
    bytes_peak_growth: int


class AllocGuard:
    def __init__(self, device=None, stats_source=None, max_blocks: int = 0, max_segments: int = 0):
        self.device, self.src = device, stats_source
        self.max_blocks, self.max_segments = max_blocks, max_segments
        self.delta: Optional[AllocDelta] = None

    def _stats(self) -> dict:
        if self.src is not None:
            return self.src.memory_stats()
        import torch

        return torch.cuda.memory_stats(self.device)

    def __enter__(self) -> "AllocGuard":
        s = self._stats()
        self._b0 = s.get("allocation.all.allocated", 0)
        self._s0 = s.get("segment.all.allocated", 0)
        self._p0 = s.get("allocated_bytes.all.peak", 0)
        return self

    def __exit__(self, et, ev, tb) -> None:
        s = self._stats()
        self.delta = AllocDelta(blocks=s.get("allocation.all.allocated", 0) - self._b0,
                                segments=s.get("segment.all.allocated", 0) - self._s0,
                                bytes_peak_growth=s.get("allocated_bytes.all.peak", 0) - self._p0)
        if et is None and (self.delta.blocks > self.max_blocks or self.delta.segments > self.max_segments):
            raise AssertionError(f"device allocations inside a guarded region: {self.delta}")
