"""Byte-level DFA grammars for structured output: token masks, transitions and jump-forward.

A grammar is a flat [states x 256] transition table (0xFFFFFFFF = reject) plus a set of
accepting states. A token is allowed in a state when walking its bytes never rejects. When a
state has exactly one outgoing byte the engine can skip sampling and emit the forced bytes
(jump-forward). Two stock grammars exist, as in the reference: a flat JSON object and a JSON
object with a fixed prefix.

Reference parity: DfaSchemaGrammar (oxide-core/src/dfa.rs:7-189: table, accepting set,
transition, apply_dfa_mask, deterministic_transition, find_jump_forward_bytes; JSON object
:16-64, fixed prefix :68-108), AsciiGrammarMask (grammar_mask.rs:18-66) and the server's
GrammarConstraintType, which compiles JsonSchema/Regex/Ebnf requests to the same JSON DFA
(oxide-server/src/grammar_engine.rs:11-76).
"""
from __future__ import annotations

from typing import Optional

import numpy as np

from .errors import GrammarError

REJECT = 0xFFFFFFFF


class Dfa:
    def __init__(self, n_states: int):
        self.table = np.full((n_states, 256), REJECT, dtype=np.uint32)
        self.accepting: set[int] = set()
        self.start = 0

    @property
    def n_states(self) -> int:
        return self.table.shape[0]

    def add(self, src: int, chars, dst: int) -> None:
        if isinstance(chars, (bytes, str)):
            chars = chars.encode() if isinstance(chars, str) else chars
            chars = list(chars)
        for c in chars:
            self.table[src, c] = dst

    def transition(self, state: int, byte: int) -> int:
        if state == REJECT:
            return REJECT
        return int(self.table[state, byte])

    def walk(self, state: int, data: bytes) -> int:
        for b in data:
            state = self.transition(state, b)
            if state == REJECT:
                return REJECT
        return state

    def is_accepting(self, state: int) -> bool:
        return state in self.accepting

    def deterministic_transition(self, state: int) -> Optional[tuple[int, int]]:
        """(byte, next_state) when exactly one byte is legal in `state`."""
        row = self.table[state]
        ok = np.nonzero(row != REJECT)[0]
        if ok.size == 1:
            return int(ok[0]), int(row[ok[0]])
        return None

    def find_jump_forward_bytes(self, state: int, limit: int = 64) -> tuple[bytes, int]:
        """Longest forced byte string from `state` and the state it leads to."""
        out = bytearray()
        while len(out) < limit and state not in self.accepting:
            det = self.deterministic_transition(state)
            if det is None:
                break
            out.append(det[0])
            state = det[1]
        return bytes(out), state

    def token_mask(self, state: int, vocab_bytes: list[bytes]) -> np.ndarray:
        """Packed allow-mask (int32 words, bit i = token i allowed) for one state."""
        n = len(vocab_bytes)
        bits = np.zeros((n + 31) // 32 * 32, dtype=np.uint8)
        for i, tb in enumerate(vocab_bytes):
            if tb and self.walk(state, tb) != REJECT:
                bits[i] = 1
        return np.packbits(bits, bitorder="little").view(np.int32)


_WS = b" \t\n\r"
_DIGITS = b"0123456789"


def ascii_first_byte_mask(allowed: bytes, vocab_bytes: list) -> np.ndarray:
    """Allow-mask over the vocabulary by the FIRST byte of each token (the reference's small
    `GrammarMask`, oxide-core/src/grammar_mask.rs:18-66): token i is allowed iff it is non-empty and its
    first byte is in `allowed`."""
    ok = np.zeros(256, dtype=bool)
    ok[np.frombuffer(bytes(allowed), dtype=np.uint8)] = True
    return np.fromiter((len(t) > 0 and ok[t[0]] for t in vocab_bytes), dtype=bool, count=len(vocab_bytes))


def json_object_dfa() -> Dfa:
    """Flat JSON object: { "key": value, ... } with string / number / true / false / null values."""
    d = Dfa(32)
    S_START, S_OPEN, S_KEY, S_KEY_ESC, S_AFTER_KEY, S_COLON, S_STR, S_STR_ESC, S_NUM, S_NUM_FRAC, \
        S_AFTER_VAL, S_COMMA, S_DONE = range(13)
    lit_base = 13  # literal states for true/false/null
    d.add(S_START, _WS, S_START)
    d.add(S_START, b"{", S_OPEN)
    d.add(S_OPEN, _WS, S_OPEN)
    d.add(S_OPEN, b'"', S_KEY)
    d.add(S_OPEN, b"}", S_DONE)
    printable = [c for c in range(0x20, 0x100) if c not in (0x22, 0x5C)]
    d.add(S_KEY, printable, S_KEY)
    d.add(S_KEY, b"\\", S_KEY_ESC)
    d.add(S_KEY_ESC, b'"\\/bfnrtu', S_KEY)
    d.add(S_KEY, b'"', S_AFTER_KEY)
    d.add(S_AFTER_KEY, _WS, S_AFTER_KEY)
    d.add(S_AFTER_KEY, b":", S_COLON)
    d.add(S_COLON, _WS, S_COLON)
    d.add(S_COLON, b'"', S_STR)
    d.add(S_STR, printable, S_STR)
    d.add(S_STR, b"\\", S_STR_ESC)
    d.add(S_STR_ESC, b'"\\/bfnrtu', S_STR)
    d.add(S_STR, b'"', S_AFTER_VAL)
    d.add(S_COLON, b"-" + _DIGITS, S_NUM)
    d.add(S_NUM, _DIGITS, S_NUM)
    d.add(S_NUM, b".", S_NUM_FRAC)
    d.add(S_NUM_FRAC, _DIGITS, S_NUM_FRAC)
    for s in (S_NUM, S_NUM_FRAC):
        d.add(s, _WS, S_AFTER_VAL)
        d.add(s, b",", S_COMMA)
        d.add(s, b"}", S_DONE)
    nxt = lit_base
    for word in (b"true", b"false", b"null"):
        cur = S_COLON
        for i, ch in enumerate(word):
            last = i == len(word) - 1
            if i == 0:
                d.add(S_COLON, bytes([ch]), nxt)
                cur = nxt
                nxt += 1
            else:
                dst = S_AFTER_VAL if last else nxt
                d.add(cur, bytes([ch]), dst)
                if not last:
                    cur = nxt
                    nxt += 1
    d.add(S_AFTER_VAL, _WS, S_AFTER_VAL)
    d.add(S_AFTER_VAL, b",", S_COMMA)
    d.add(S_AFTER_VAL, b"}", S_DONE)
    d.add(S_COMMA, _WS, S_COMMA)
    d.add(S_COMMA, b'"', S_KEY)
    d.add(S_DONE, _WS, S_DONE)
    d.accepting = {S_DONE}
    return d


def json_prefix_dfa(prefix: bytes) -> Dfa:
    """The fixed byte string `prefix` (e.g. b'{"answer": "'), then the rest of a flat JSON object."""
    body = json_object_dfa()
    n_pre = len(prefix)
    d = Dfa(n_pre + body.n_states)
    # where in the body automaton does the prefix leave us?
    land = body.walk(body.start, prefix)
    if land == REJECT:
        raise GrammarError("prefix is not a prefix of a JSON object")
    off = n_pre
    d.table[off:off + body.n_states] = np.where(body.table == REJECT, REJECT, body.table + off)
    for i, ch in enumerate(prefix):
        dst = i + 1 if i + 1 < n_pre else land + off
        d.table[i, ch] = dst
    d.accepting = {s + off for s in body.accepting}
    d.start = 0 if n_pre else land + off
    return d


class GrammarState:
    """Per-request grammar cursor used by the engine."""

    def __init__(self, dfa: Dfa, vocab_bytes: Optional[list[bytes]] = None):
        self.dfa = dfa
        self.state = dfa.start
        self.vocab_bytes = vocab_bytes
        self._mask_cache: dict[int, np.ndarray] = {}

    def set_vocab(self, vocab_bytes: list[bytes]) -> None:
        self.vocab_bytes = vocab_bytes
        self._mask_cache.clear()

    def allow_mask(self, vocab_size: int) -> np.ndarray:
        words = (vocab_size + 31) // 32
        if self.vocab_bytes is None or self.state == REJECT:
            return np.full(words, -1, dtype=np.int32)
        m = self._mask_cache.get(self.state)
        if m is None:
            m = self.dfa.token_mask(self.state, self.vocab_bytes)
            if not m.any():  # nothing fits: do not dead-lock generation
                m = np.full_like(m, -1)
            self._mask_cache[self.state] = m
        out = np.zeros(words, dtype=np.int32)
        out[: min(words, m.size)] = m[:words]
        return out

    def advance(self, token: int) -> None:
        if self.vocab_bytes is None or self.state == REJECT:
            return
        if 0 <= token < len(self.vocab_bytes):
            self.state = self.dfa.walk(self.state, self.vocab_bytes[token])

    def done(self) -> bool:
        return self.dfa.is_accepting(self.state)

    def jump_forward(self) -> bytes:
        data, nxt = self.dfa.find_jump_forward_bytes(self.state)
        return data


def grammar_from_spec(spec: str, vocab_bytes: Optional[list[bytes]] = None) -> GrammarState:
    """'json' | 'json_schema' | 'regex' | 'ebnf' -> flat JSON object; 'json_prefix:<text>'."""
    if spec.startswith("json_prefix:"):
        return GrammarState(json_prefix_dfa(spec[len("json_prefix:"):].encode()), vocab_bytes)
    if spec in ("json", "json_schema", "json_object", "regex", "ebnf"):
        return GrammarState(json_object_dfa(), vocab_bytes)
    raise GrammarError(f"unknown grammar spec {spec!r}")
