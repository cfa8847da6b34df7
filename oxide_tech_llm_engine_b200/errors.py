"""Typed error tree of the engine.

Mirrors the variants of the reference's `EngineError` enum (oxide-core/src/error.rs:5-101) as a
Python exception hierarchy; `CollectiveTimeout` is new (a bounded device-side wait on a peer
flag ran out; there is no multi-GPU path in the reference).
"""
from __future__ import annotations


class EngineError(Exception):
    """Base class of every error the engine raises on purpose."""


class ConfigError(EngineError):
    pass


class ModelLoadError(EngineError):
    pass


class UnsupportedFormat(ModelLoadError):
    pass


class TokenizerError(EngineError):
    pass


class OutOfMemory(EngineError):
    """KV pool or device memory exhausted."""


class SlotsExhausted(EngineError):
    """No free sequence slot (the server answers 503)."""


class BackendNotReady(EngineError):
    pass


class UninitializedStream(EngineError):
    pass


class HardwareFault(EngineError):
    def __init__(self, msg: str, recoverable: bool = False):
        super().__init__(msg)
        self.recoverable = recoverable


class CollectiveTimeout(HardwareFault):
    """A kernel's bounded wait on a peer flag expired; the context stays usable."""

    def __init__(self, msg: str):
        super().__init__(msg, recoverable=True)


class TransactionAborted(EngineError):
    pass


class NumericalDrift(EngineError):
    pass


class BenchmarkIntegrityViolation(EngineError):
    pass


class GoldenParityFailure(EngineError):
    pass


class RequestCancelled(EngineError):
    pass


class PrefillError(EngineError):
    pass


class GrammarError(EngineError):
    pass
