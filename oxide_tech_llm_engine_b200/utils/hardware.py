"""Device profiles, shared-device budget handle, energy sampler and allocation guard.

Reference parity: GpuDeviceProfile table and ComputeCapability::architecture (10..=12 ->
Blackwell) of oxide-core/src/hardware.rs:6-14,260-280,464-517,876-926; SharedDevice VRAM budget
handle with a hibernate flag (shared_device.rs:12-141); NVML energy sampler -- total-energy
counter or power integration, J / W / tokens per joule (oxide-backend-cuda/src/energy.rs:41-437);
CountingAlloc test hook (zero_alloc_guard.rs:11-65) as a CUDA caching-allocator counter.
Everything here only READS device state; no clock, power or mode setting is ever changed.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Optional

from ..errors import OutOfMemory
from .roofline import load_measured_peaks


@dataclass(frozen=True)
class GpuDeviceProfile:
    name: str
    arch: str
    sm_count: int
    hbm_gb: float
    hbm_gbs: float          # nominal
    bf16_tflops: float      # nominal dense
    fp8_tflops: float
    fp4_tflops: float
    tensor_core_gen: int
    nvlink_gbs_per_dir: float
    l2_mb: float
    smem_kb_per_cta: int


PROFILES = {
    "B200": GpuDeviceProfile("NVIDIA B200", "blackwell", 148, 180.0, 7700.0, 2250.0, 4500.0, 9000.0, 5, 900.0, 126.0, 227),
    "GB200": GpuDeviceProfile("NVIDIA GB200", "blackwell", 148, 186.0, 8000.0, 2500.0, 5000.0, 10000.0, 5, 900.0, 126.0, 227),
    "H100": GpuDeviceProfile("NVIDIA H100 SXM", "hopper", 132, 80.0, 3350.0, 989.0, 1979.0, 0.0, 4, 450.0, 50.0, 227),
    "A100": GpuDeviceProfile("NVIDIA A100 SXM", "ampere", 108, 80.0, 2039.0, 312.0, 0.0, 0.0, 3, 300.0, 40.0, 163),
    "RTX 4060": GpuDeviceProfile("NVIDIA RTX 4060 Laptop", "ada", 24, 8.0, 256.0, 60.0, 120.0, 0.0, 4, 0.0, 32.0, 99),
}


def architecture(major: int, minor: int = 0) -> str:
    if 10 <= major <= 12:
        return "blackwell"
    return {9: "hopper", 8: "ada" if minor == 9 else "ampere", 7: "volta" if minor == 0 else "turing"}.get(major, "unknown")


def lookup_profile(name: str) -> Optional[GpuDeviceProfile]:
    up = name.upper()
    for key, p in PROFILES.items():
        if key.upper() in up:
            return p
    return None


def current_profile(device: int = 0) -> dict:
    """Nominal profile of the visible GPU plus the measured peaks used as roofline denominators."""
    import torch

    out: dict = {"measured": load_measured_peaks()}
    if torch.cuda.is_available():
        pr = torch.cuda.get_device_properties(device)
        out.update(name=pr.name, sm_count=pr.multi_processor_count, hbm_gb=round(pr.total_memory / 1e9, 1),
                   arch=architecture(pr.major, pr.minor))
        p = lookup_profile(pr.name)
        if p is not None:
            out["nominal"] = p
    return out


class SharedDevice:
    """Byte budget shared by the components of one process (weights, KV pool, workspaces)."""

    def __init__(self, total_bytes: int):
        self.total, self.used = total_bytes, 0
        self.hibernating = False
        self._lock = threading.Lock()

    def reserve(self, nbytes: int, what: str = "") -> None:
        with self._lock:
            if self.used + nbytes > self.total:
                raise OutOfMemory(f"device budget exceeded by {what or 'allocation'}: "
                                  f"{self.used + nbytes} > {self.total}")
            self.used += nbytes

    def release(self, nbytes: int) -> None:
        with self._lock:
            self.used = max(0, self.used - nbytes)

    def free_bytes(self) -> int:
        return self.total - self.used

    def hibernate(self, flag: bool = True) -> None:
        self.hibernating = flag


class EnergySampler:
    """Reads the NVML total-energy counter (or integrates power draw) around a region."""

    def __init__(self, device: int = 0, nvml=None, period_s: float = 0.05):
        self.device, self.period = device, period_s
        self.nvml = nvml
        self._h = None
        self._t0 = self._e0 = None
        self._thread = None
        self._stop = threading.Event()
        self._joules = 0.0

    def _lib(self):
        if self.nvml is None:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
        if self._h is None:
            self._h = self.nvml.nvmlDeviceGetHandleByIndex(self.device)
        return self.nvml

    def start(self) -> None:
        n = self._lib()
        self._t0 = time.perf_counter()
        try:
            self._e0 = n.nvmlDeviceGetTotalEnergyConsumption(self._h)  # millijoules
        except Exception:
            self._e0 = None
            self._stop.clear()
            self._joules = 0.0

            def loop():
                last = time.perf_counter()
                while not self._stop.wait(self.period):
                    now = time.perf_counter()
                    self._joules += n.nvmlDeviceGetPowerUsage(self._h) / 1e3 * (now - last)
                    last = now
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()

    def stop(self, tokens: int = 0) -> dict:
        n = self._lib()
        dt = time.perf_counter() - self._t0
        if self._e0 is not None:
            joules = (n.nvmlDeviceGetTotalEnergyConsumption(self._h) - self._e0) / 1e3
        else:
            self._stop.set()
            if self._thread:
                self._thread.join()
            joules = self._joules
        return {"joules": joules, "seconds": dt, "watts": joules / dt if dt > 0 else 0.0,
                "tokens_per_joule": tokens / joules if joules > 0 else 0.0}


class AllocationGuard:
    """Counts device allocations made by the caching allocator inside a region (the decode loop
    is expected to make none once its graphs are captured)."""

    def __enter__(self):
        import torch

        self.torch = torch
        torch.cuda.synchronize()
        self.before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        return self

    def __exit__(self, *exc):
        self.torch.cuda.synchronize()
        self.count = self.torch.cuda.memory_stats().get("allocation.all.allocated", 0) - self.before
        return False
