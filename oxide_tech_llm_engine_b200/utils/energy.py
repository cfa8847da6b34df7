"""Energy accounting around a generation: joules, average watts, tokens per joule.

Reads NVML (read-only queries: the total-energy counter when the GPU has one, else power samples
integrated over time by a sampling thread). Nothing here changes a GPU setting. The NVML module is
injectable so the logic is tested on CPU against a fake.

Reference: the energy sampler of oxide-backend-cuda/src/energy.rs:41-437 (dlopen of
libnvidia-ml.so.1, total-energy counter or power integration thread -> J, W, tok/J).
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Optional


@dataclass
class EnergyReport:
    joules: float
    seconds: float
    tokens: int
    source: str  # "counter" | "integrated" | "unavailable"

    @property
    def watts(self) -> float:
        return self.joules / self.seconds if self.seconds > 0 else 0.0

    @property
    def tokens_per_joule(self) -> float:
        return self.tokens / self.joules if self.joules > 0 else 0.0

    def to_dict(self) -> dict:
        return {"joules": round(self.joules, 3), "seconds": round(self.seconds, 4), "watts": round(self.watts, 2),
                "tokens": self.tokens, "tokens_per_joule": round(self.tokens_per_joule, 4), "source": self.source}


class EnergySampler:
    def __init__(self, gpu_index: int = 0, nvml=None, period_s: float = 0.05, clock=time.monotonic):
        self.clock, self.period = clock, period_s
        self.source = "unavailable"
        self._h = None
        self._nvml = nvml
        if nvml is None:
            try:
                import pynvml as nvml_mod  # provided by nvidia-ml-py
                self._nvml = nvml_mod
            except Exception:
                self._nvml = None
        if self._nvml is not None:
            try:
                self._nvml.nvmlInit()
                self._h = self._nvml.nvmlDeviceGetHandleByIndex(gpu_index)
                try:
                    self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._h)  # millijoules
                    self.source = "counter"
                except Exception:
                    self._nvml.nvmlDeviceGetPowerUsage(self._h)              # milliwatts
                    self.source = "integrated"
            except Exception:
                self._h, self.source = None, "unavailable"
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._acc_j = 0.0
        self._e0 = 0.0
        self._t0 = 0.0

    def _power_w(self) -> float:
        return self._nvml.nvmlDeviceGetPowerUsage(self._h) / 1e3

    def sample_once(self, dt: float) -> None:
        """One integration step of `dt` seconds (the thread calls this; tests call it directly)."""
        self._acc_j += self._power_w() * dt

    def start(self) -> "EnergySampler":
        self._t0 = self.clock()
        self._acc_j = 0.0
        if self.source == "counter":
            self._e0 = self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._h) / 1e3
        elif self.source == "integrated":
            def loop():
                last = self.clock()
                while not self._stop.wait(self.period):
                    now = self.clock()
                    self.sample_once(now - last)
                    last = now
            self._stop.clear()
            self._thread = threading.Thread(target=loop, name="oxb-energy", daemon=True)
            self._thread.start()
        return self

    def stop(self, tokens: int = 0) -> EnergyReport:
        dt = self.clock() - self._t0
        if self.source == "counter":
            j = self._nvml.nvmlDeviceGetTotalEnergyConsumption(self._h) / 1e3 - self._e0
        elif self.source == "integrated":
            self._stop.set()
            if self._thread is not None:
                self._thread.join(timeout=2.0)
            j = self._acc_j
        else:
            j = 0.0
        return EnergyReport(joules=j, seconds=dt, tokens=tokens, source=self.source)
