"""Multi-LoRA: adapter registry, SafeTensors ingest and per-layer A/B application.

y = W x + (alpha / r) * B (A x). Adapters are merged into a copy of the base weight source, so
the serving kernels run unchanged; several adapters can be registered and selected by name.
Reference parity: multi_lora.rs:11-105 (per-layer A/B apply, adapter registry) and
unsloth_lora.rs:13-308 (safetensors adapter ingest, `lora_A` / `lora_B` key naming, alpha / r).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from ..models.weights import WeightSource, hf_name_to_gguf


@dataclass
class LoraAdapter:
    name: str
    rank: int
    alpha: float
    a: dict = field(default_factory=dict)  # gguf tensor name -> A [r, in]
    b: dict = field(default_factory=dict)  # gguf tensor name -> B [out, r]

    @property
    def scale(self) -> float:
        return self.alpha / max(self.rank, 1)

    def delta(self, name: str) -> Optional[np.ndarray]:
        if name not in self.a or name not in self.b:
            return None
        return (self.b[name] @ self.a[name]) * self.scale

    def apply_activation(self, name: str, x: np.ndarray) -> np.ndarray:
        """LoRA contribution for activations x [T, in] without materialising the delta."""
        return (x @ self.a[name].T) @ self.b[name].T * self.scale


def load_adapter_safetensors(path: str, name: str, alpha: Optional[float] = None) -> LoraAdapter:
    from ..formats.safetensors import SafeTensorsFile

    f = SafeTensorsFile(path)
    a, b, rank = {}, {}, 0
    for key in f.names():
        base = key.replace("base_model.model.", "")
        for tag, store in ((".lora_A.weight", a), (".lora_B.weight", b), (".lora_A.default.weight", a),
                           (".lora_B.default.weight", b)):
            if base.endswith(tag):
                g = hf_name_to_gguf(base[: -len(tag)] + ".weight")
                if g is not None:
                    store[g] = f.f32(key)
                    if store is a:
                        rank = store[g].shape[0]
    al = float(f.metadata.get("lora_alpha", alpha if alpha is not None else rank)) if f.metadata else float(alpha or rank)
    return LoraAdapter(name, rank, al, a, b)


class LoraRegistry:
    def __init__(self):
        self.adapters: dict[str, LoraAdapter] = {}

    def register(self, ad: LoraAdapter) -> None:
        self.adapters[ad.name] = ad

    def get(self, name: str) -> LoraAdapter:
        return self.adapters[name]

    def names(self) -> list[str]:
        return list(self.adapters)


class MergedSource(WeightSource):
    """A weight source with one adapter merged in (W + scale * B A)."""

    def __init__(self, base: WeightSource, adapter: LoraAdapter):
        self.base, self.adapter, self.cfg = base, adapter, base.cfg

    def names(self):
        return self.base.names()

    def has(self, name):
        return self.base.has(name)

    def shape(self, name):
        return self.base.shape(name)

    def type_name(self, name):
        return "F32" if self.adapter.delta(name) is not None else self.base.type_name(name)

    def f32(self, name):
        w = self.base.f32(name)
        d = self.adapter.delta(name)
        return w if d is None else (w + d).astype(np.float32)

    def raw(self, name):
        if self.adapter.delta(name) is None:
            return self.base.raw(name)
        return super().raw(name)
