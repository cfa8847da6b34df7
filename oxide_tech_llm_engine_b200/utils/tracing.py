"""Logging, step traces, NVTX ranges and tensor dumps.

* `get_logger()` - stderr logger filtered by OXB_LOG / RUST_LOG style levels (default info).
* `StepTrace` - one JSON line per engine step (tokens, batch, wall ms) when OXB_TRACE_FILE is set.
* `nvtx_range` - NVTX ranges around layers / kernels when a profiler is attached.
* `debug_tensor` - first values of an intermediate tensor when OXIDE_DEBUG_LAYER / OXB_DEBUG_LAYER
  is set, for diffing the device path against the oracle.

Reference parity: tracing_subscriber fmt + EnvFilter("info") (oxide-cli/src/lib.rs:704-709), the
decode-latency line every 16 tokens (oxide-backend-cuda/src/lib.rs:4207-4213), OXIDE_DEBUG_LAYER
dumps of the first 4 values (llama3.rs:3478-3480) and the debug-layer / debug-prefill binaries.
"""
from __future__ import annotations

import contextlib
import json
import logging
import os
import sys
import time
from typing import Optional

_LEVELS = {"trace": 5, "debug": logging.DEBUG, "info": logging.INFO, "warn": logging.WARNING,
           "warning": logging.WARNING, "error": logging.ERROR}


def get_logger(name: str = "oxide") -> logging.Logger:
    log = logging.getLogger(name)
    if not log.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
        log.addHandler(h)
        lvl = os.environ.get("OXB_LOG", os.environ.get("RUST_LOG", "info")).lower()
        log.setLevel(_LEVELS.get(lvl, logging.INFO))
        log.propagate = False
    return log


class StepTrace:
    def __init__(self, path: Optional[str] = None):
        self.path = path or os.environ.get("OXB_TRACE_FILE")
        self.f = open(self.path, "a") if self.path else None
        self.t_last = time.perf_counter()
        self.tokens_since_log = 0

    def record(self, step: int, n_decode: int, n_prefill_tokens: int, wall_ms: float, **extra) -> None:
        if self.f:
            self.f.write(json.dumps({"step": step, "decode": n_decode, "prefill_tokens": n_prefill_tokens,
                                     "ms": round(wall_ms, 3), **extra}) + "\n")
            self.f.flush()
        self.tokens_since_log += n_decode
        if self.tokens_since_log >= 16 * max(n_decode, 1):
            now = time.perf_counter()
            get_logger().debug("decode %.1f tok/s over the last %d tokens", self.tokens_since_log / max(now - self.t_last, 1e-9),
                               self.tokens_since_log)
            self.t_last, self.tokens_since_log = now, 0

    def close(self) -> None:
        if self.f:
            self.f.close()
            self.f = None


@contextlib.contextmanager
def nvtx_range(name: str):
    try:
        import torch

        on = torch.cuda.is_available() and os.environ.get("OXB_NVTX", "0") == "1"
    except Exception:  # pragma: no cover
        on = False
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def debug_enabled() -> bool:
    return bool(os.environ.get("OXB_DEBUG_LAYER") or os.environ.get("OXIDE_DEBUG_LAYER"))


def debug_tensor(tag: str, t, n: int = 4) -> Optional[list]:
    """Prints and returns the first `n` values of a tensor when layer debugging is on."""
    if not debug_enabled():
        return None
    vals = [float(x) for x in t.reshape(-1)[:n].float().cpu().tolist()]
    get_logger("oxide.debug").info("%s: %s", tag, ["%.6f" % v for v in vals])
    return vals
