"""Roofline receipt: memory-bandwidth and model-FLOP utilisation of a decode run.

MBU = (bytes read per token * tokens/s) / measured copy bandwidth, MFU = (2 * active params *
tokens/s) / measured GEMM peak; a receipt above 1.05 is rejected as physically impossible.
Reference parity: RooflineReceipt (oxide-core/src/roofline.rs:15-71, sanity check :52-58). The
denominators are the measured peaks of this machine (`MEASURED_PEAKS.json` at the repo root when
present, else the stated fallback of 6.65 TB/s and 1.59 PFLOP/s).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass

from ..errors import BenchmarkIntegrityViolation

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def load_measured_peaks(path: str | None = None) -> dict:
    cands = [path] if path else []
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cands.append(os.path.join(here, "MEASURED_PEAKS.json"))
    for c in cands:
        if c and os.path.exists(c):
            d = json.load(open(c))
            d["source"] = "measured"
            return d
    return dict(FALLBACK_PEAKS)


@dataclass
class RooflineReceipt:
    model: str
    tokens_per_s: float
    batch: int
    bytes_per_step: float
    flops_per_token: float
    hbm_gbs: float
    peak_tflops: float
    mbu: float
    mfu: float
    peaks_source: str

    @classmethod
    def from_run(cls, mc, *, tokens_per_s: float, batch: int, peaks: dict, weight_bytes_per_param: float = 2.0,
                 context: int = 0, tp: int = 1) -> "RooflineReceipt":
        weight_bytes = mc.active_params() * weight_bytes_per_param / tp
        kv_bytes = batch * context * mc.kv_bytes_per_token() / tp
        bytes_per_step = weight_bytes + kv_bytes
        steps_per_s = tokens_per_s / max(batch, 1)
        mbu = bytes_per_step * steps_per_s / (peaks["hbm_gbs"] * 1e9)
        flops = 2.0 * mc.active_params()
        mfu = flops * tokens_per_s / tp / (peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]) * 1e12)
        r = cls(mc.name, tokens_per_s, batch, bytes_per_step, flops, peaks["hbm_gbs"],
                peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]), mbu, mfu, peaks.get("source", "measured"))
        r.validate()
        return r

    def validate(self) -> None:
        if self.mbu > 1.05 or self.mfu > 1.05:
            raise BenchmarkIntegrityViolation(
                f"roofline receipt is physically impossible: MBU={self.mbu:.3f} MFU={self.mfu:.3f} (> 1.05)")

    def to_dict(self) -> dict:
        return asdict(self)
