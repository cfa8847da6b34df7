"""Per-request sampling parameters (defaults of the reference's SamplerConfig,
oxide-core/src/sampler.rs:17-73: T=0.8, top_k=40, top_p=0.95, min_p=0.05, repeat 1.1 over 64)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.05
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    newline_penalty: float = 0.0
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    xtc_probability: float = 0.0
    xtc_threshold: float = 0.1
    tfs_z: float = 1.0
    typical_p: float = 1.0
    mirostat: int = 0          # 0 off, 1, 2
    mirostat_tau: float = 5.0
    mirostat_eta: float = 0.1
    seed: int = 42
    max_tokens: int = 64
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    logit_bias: dict[int, float] = field(default_factory=dict)
    banned_tokens: list[int] = field(default_factory=list)
    grammar: Optional[str] = None   # "json" | "json_prefix:<text>" | None
    greedy: bool = False

    def is_greedy(self) -> bool:
        return self.greedy or self.temperature <= 0.0 or self.top_k == 1

    def device_ok(self) -> bool:
        """True when the device sampler covers the request (temperature/top-k/top-p/min-p/mask);
        everything else runs through the host pipeline."""
        return (self.repeat_penalty == 1.0 and self.frequency_penalty == 0.0 and
                self.presence_penalty == 0.0 and self.newline_penalty == 0.0 and
                self.dry_multiplier == 0.0 and self.xtc_probability == 0.0 and self.tfs_z >= 1.0 and
                self.typical_p >= 1.0 and self.mirostat == 0 and not self.logit_bias)
