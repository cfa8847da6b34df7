"""Host sampler: the full pipeline, in the reference's order.

bans -> logit bias -> newline penalty -> DRY -> repeat / frequency / presence penalties over the
last `repeat_last_n` tokens -> temperature -> candidates = top max(k, 256) sorted -> softmax ->
Mirostat v1/v2 (early return) -> min-p -> XTC -> top-k -> tail-free -> locally typical -> top-p ->
renormalise -> greedy or inverse-CDF draw from a xorshift64 stream.

Reference parity: AcademicSamplerEngine::sample_token (oxide-core/src/sampler.rs:173-390), DRY
(:393-415), Mirostat (:418-456), TFS (:459-490), typical (:493-520), xorshift64 state (:139-146).
The device kernels (csrc/kernels/sampler.cu) cover temperature/top-k/min-p/top-p/masks; requests
that use any other stage come through here.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np

from .sampling_params import SamplingParams


class XorShift64:
    def __init__(self, seed: int):
        self.s = (seed & 0xFFFFFFFFFFFFFFFF) or 0x9E3779B97F4A7C15

    def next_u64(self) -> int:
        x = self.s
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        self.s = x
        return x

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


class HostSampler:
    def __init__(self, params: SamplingParams, newline_token_id: int = -1):
        self.p = params
        self.rng = XorShift64(params.seed)
        self.mu = 2.0 * params.mirostat_tau
        self.newline_token_id = newline_token_id
        self.dry_range = 1024

    # ------------------------------------------------------------------ stages
    def _dry(self, logits: np.ndarray, hist: np.ndarray) -> None:
        p = self.p
        h = hist[-self.dry_range:]
        n = len(h)
        for match_len in range(32, p.dry_allowed_length - 1, -1):
            if n < match_len or match_len <= 0:
                continue
            suffix = h[n - match_len:]
            for i in range(0, max(n - match_len, 0)):
                if np.array_equal(h[i:i + match_len], suffix) and i + match_len < n:
                    nxt = int(h[i + match_len])
                    pen = p.dry_multiplier * (p.dry_base ** (match_len - p.dry_allowed_length))
                    if 0 <= nxt < logits.size:
                        logits[nxt] -= pen

    @staticmethod
    def _tfs(ids, pr, z):
        if len(pr) < 3:
            return ids, pr
        d1 = pr[:-1] - pr[1:]
        d2 = np.abs(d1[:-1] - d1[1:])
        tot = d2.sum()
        if tot <= 0:
            return ids, pr
        cum = np.cumsum(d2 / tot)
        hit = np.nonzero(cum >= z)[0]
        cut = int(hit[0]) + 1 if hit.size else len(pr)
        cut = max(cut, 1)
        return ids[:cut], pr[:cut]

    @staticmethod
    def _typical(ids, pr, typical_p):
        with np.errstate(divide="ignore"):
            surprisal = np.where(pr > 0, -np.log(pr), 0.0)
        entropy = float((pr * surprisal).sum())
        order = np.argsort(np.abs(surprisal - entropy), kind="stable")
        cum = np.cumsum(pr[order])
        hit = np.nonzero(cum >= typical_p)[0]
        cut = int(hit[0]) + 1 if hit.size else len(pr)
        keep = order[:cut]
        return ids[keep], pr[keep]

    # ------------------------------------------------------------------ main
    def sample(self, logits_in: np.ndarray, history: Sequence[int], allow_mask: Optional[np.ndarray] = None) -> int:
        p = self.p
        logits = np.array(logits_in, dtype=np.float32, copy=True)
        hist = np.asarray(history, dtype=np.int64)
        if allow_mask is not None:
            bits = np.unpackbits(allow_mask.view(np.uint8), bitorder="little")[: logits.size].astype(bool)
            logits[~bits] = -np.inf
        for b in p.banned_tokens:
            if 0 <= b < logits.size:
                logits[b] = -np.inf
        for t, bias in p.logit_bias.items():
            if 0 <= int(t) < logits.size:
                logits[int(t)] += bias
        if p.newline_penalty and 0 <= self.newline_token_id < logits.size:
            logits[self.newline_token_id] -= p.newline_penalty
        if p.dry_multiplier > 0 and hist.size:
            self._dry(logits, hist)
        if hist.size:
            window = hist[-p.repeat_last_n:] if p.repeat_last_n > 0 else hist
            if abs(p.repeat_penalty - 1.0) > 1e-5 and p.repeat_penalty > 0:
                seen = np.unique(window)
                seen = seen[(seen >= 0) & (seen < logits.size)]
                v = logits[seen]
                logits[seen] = np.where(v > 0, v / p.repeat_penalty, v * p.repeat_penalty)
            if abs(p.frequency_penalty) > 1e-5 or abs(p.presence_penalty) > 1e-5:
                toks, counts = np.unique(window, return_counts=True)
                ok = (toks >= 0) & (toks < logits.size)
                logits[toks[ok]] -= counts[ok] * p.frequency_penalty + p.presence_penalty
        if p.temperature > 0 and p.mirostat == 0:
            logits *= 1.0 / p.temperature
        finite = np.nonzero(logits > -np.inf)[0]
        if finite.size == 0:
            return 0
        filter_k = min(max(p.top_k, 256), finite.size)
        vals = logits[finite]
        if filter_k < finite.size:
            part = np.argpartition(-vals, filter_k - 1)[:filter_k]
            finite, vals = finite[part], vals[part]
        order = np.lexsort((finite, -vals))  # descending logit, ascending id on ties
        ids, vals = finite[order], vals[order]
        pr = np.exp(vals - vals[0])
        pr = pr / pr.sum()
        if p.mirostat == 1:
            prob = max(float(pr[0]), 1e-6)
            self.mu -= p.mirostat_eta * (-math.log2(prob) - p.mirostat_tau)
            return int(ids[0])
        if p.mirostat == 2:
            cutoff, cum = 1, 0.0
            for i in range(len(pr)):
                if -math.log2(max(float(pr[i]), 1e-8)) > self.mu and i > 0:
                    break
                cum += float(pr[i])
                cutoff = i + 1
            prob = float(pr[0]) / max(cum, 1e-6)
            self.mu -= p.mirostat_eta * (-math.log2(max(prob, 1e-8)) - p.mirostat_tau)
            return int(ids[0])
        if p.min_p > 0:
            keep = pr >= pr[0] * p.min_p
            ids, pr = ids[keep], pr[keep]
        if p.xtc_probability > 0 and len(pr) > 1:
            if p.xtc_threshold <= pr[0] < 0.98:
                ids, pr = ids[1:], pr[1:]
        if p.top_k > 0 and len(pr) > p.top_k:
            ids, pr = ids[:p.top_k], pr[:p.top_k]
        if p.tfs_z < 1.0 and len(pr) > 2:
            ids, pr = self._tfs(ids, pr, p.tfs_z)
        if p.typical_p < 1.0 and len(pr) > 1:
            ids, pr = self._typical(ids, pr, p.typical_p)
        if p.top_p < 1.0:
            cum = np.cumsum(pr)
            hit = np.nonzero(cum >= p.top_p)[0]
            cut = int(hit[0]) + 1 if hit.size else len(pr)
            ids, pr = ids[:cut], pr[:cut]
        tot = pr.sum()
        pr = pr / tot if tot > 0 else pr
        if p.temperature <= 1e-6 or p.greedy:
            return int(ids[0])
        r = self.rng.next_f32()
        acc = np.cumsum(pr)
        hit = np.nonzero(r <= acc)[0]
        return int(ids[int(hit[0])] if hit.size else ids[0])


def first_char_mask(vocab_bytes: list[bytes], allowed_first_bytes: set[int]) -> np.ndarray:
    """GBNF-style first-byte mask: a token is allowed when its first byte is in the set
    (reference: sampler.rs:525-584, grammar_mask.rs:18-66). Returns packed int32 words."""
    n = len(vocab_bytes)
    bits = np.zeros((n + 31) // 32 * 32, dtype=np.uint8)
    for i, b in enumerate(vocab_bytes):
        if b and b[0] in allowed_first_bytes:
            bits[i] = 1
    return np.packbits(bits, bitorder="little").view(np.int32)
