"""Beam search step and best-of-N ranking with length normalisation.

Reference parity: oxide-engine/src/decoding.rs:11-151 (length-normalised score
sum_logprob / ((5 + len) / 6) ** alpha with alpha = 0.6, beam expansion, candidate ranking).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


def length_penalty(length: int, alpha: float = 0.6) -> float:
    return ((5.0 + length) / 6.0) ** alpha


@dataclass
class Beam:
    tokens: list = field(default_factory=list)
    logprob: float = 0.0
    finished: bool = False

    def score(self, alpha: float = 0.6) -> float:
        return self.logprob / length_penalty(max(len(self.tokens), 1), alpha)


def beam_step(beams: list[Beam], logprobs: np.ndarray, beam_width: int, eos_id: int, alpha: float = 0.6) -> list[Beam]:
    """logprobs[i] = log-softmax over the vocabulary for live beam i (finished beams carry over)."""
    cands: list[Beam] = [b for b in beams if b.finished]
    live = [b for b in beams if not b.finished]
    for b, lp in zip(live, logprobs):
        top = np.argpartition(-lp, min(beam_width, lp.size - 1))[:beam_width]
        for t in top:
            cands.append(Beam(b.tokens + [int(t)], b.logprob + float(lp[t]), int(t) == eos_id))
    cands.sort(key=lambda c: -c.score(alpha))
    return cands[:beam_width]


def rank_candidates(cands: list[tuple[list, float]], alpha: float = 0.6) -> list[int]:
    """Best-of-N: indices of (tokens, sum_logprob) candidates, best first."""
    scores = [lp / length_penalty(max(len(t), 1), alpha) for t, lp in cands]
    return sorted(range(len(cands)), key=lambda i: -scores[i])
