"""Speculative decoding helpers: n-gram drafter, acceptance rule, adaptive draft length.

The engine attaches drafts to greedy requests; the scheduler turns `[last token] + drafts` into a
short verify chunk, the model scores all positions in one pass, and the longest draft prefix that
matches the model's own greedy choices is accepted (the block table is rolled back past it).

Reference parity: DrafterEnsemble 2..5-gram tables (oxide-engine/src/speculative.rs:514-801),
verify rule `p_t >= p_d or p_t / p_d >= threshold` (speculative.rs:72-113), AdaptiveSpeculator
K in [min, max] from rolling acceptance (speculative.rs:374-497), GPU verify = batched forward of
[cur] + <= 5 drafts then argmax compare (oxide-backend-cuda/src/lib.rs:1817-2541).
"""
from __future__ import annotations

from collections import deque
from typing import Sequence

import numpy as np


class NgramDrafter:
    """Proposes the continuation that followed the most recent earlier occurrence of the current
    suffix (longest n-gram first)."""

    def __init__(self, max_draft: int = 5, min_n: int = 2, max_n: int = 5):
        self.max_draft, self.min_n, self.max_n = max_draft, min_n, max_n

    def propose(self, history: Sequence[int]) -> list[int]:
        h = np.asarray(history)
        n_hist = h.size
        for n in range(min(self.max_n, n_hist - 1), self.min_n - 1, -1):
            suffix = h[n_hist - n:]
            # scan backwards for the latest earlier match
            for start in range(n_hist - n - 1, -1, -1):
                if np.array_equal(h[start:start + n], suffix):
                    cont = h[start + n:start + n + self.max_draft]
                    if cont.size:
                        return [int(t) for t in cont]
                    break
        return []


def accept_draft(p_target: float, p_draft: float, threshold: float = 0.8) -> bool:
    """Leviathan-style relaxed acceptance of one drafted token."""
    if p_draft <= 0.0:
        return p_target > 0.0
    return p_target >= p_draft or p_target / p_draft >= threshold


def longest_accepted_prefix(drafts: Sequence[int], verified: Sequence[int]) -> int:
    """Greedy verification: number of leading drafts equal to the model's own choices."""
    n = 0
    for d, v in zip(drafts, verified):
        if d != v:
            break
        n += 1
    return n


class AdaptiveSpeculator:
    """Keeps the draft length K in [k_min, k_max] following the rolling acceptance rate."""

    def __init__(self, k_min: int = 1, k_max: int = 5, window: int = 32, up: float = 0.7, down: float = 0.3):
        self.k_min, self.k_max, self.up, self.down = k_min, k_max, up, down
        self.k = max(k_min, min(k_max, (k_min + k_max) // 2))
        self.hist: deque = deque(maxlen=window)
        self.proposed = 0
        self.accepted = 0

    def record(self, n_proposed: int, n_accepted: int) -> None:
        if n_proposed <= 0:
            return
        self.proposed += n_proposed
        self.accepted += n_accepted
        self.hist.append(n_accepted / n_proposed)
        rate = sum(self.hist) / len(self.hist)
        if rate >= self.up and self.k < self.k_max:
            self.k += 1
        elif rate <= self.down and self.k > self.k_min:
            self.k -= 1

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0
