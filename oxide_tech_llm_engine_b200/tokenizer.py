"""Tokenizer: GGUF vocabulary with greedy longest-match encoding, plus an ASCII/byte fallback.

Behaviour follows the reference's GgufTokenizer (oxide-models/src/tokenizer.rs:38-378): vocab /
special ids from GGUF metadata; encode = split on special tokens, then greedy longest match
(<= 64 bytes) trying the SentencePiece `▁` and GPT-2 `Ġ` space conventions, `<0xHH>` byte
fallback; decode cleans those markers up; `is_stop_token` knows the EOS id, the usual end-of-turn
strings and the hard-coded ids 2/128001/128008/128009/151643/151645 (tokenizer.rs:162-184).
"""
from __future__ import annotations

from typing import Iterable, Optional

STOP_STRINGS = ("<|endoftext|>", "<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<eos>", "</s>")
HARD_STOP_IDS = (2, 128001, 128008, 128009, 151643, 151645)
_GPT2_SPACE = "Ġ"  # Ġ
_SP_SPACE = "▁"    # ▁


class Tokenizer:
    def __init__(self, vocab: list[str], *, bos_id: int = 1, eos_id: int = 2, model: str = "llama",
                 special: Optional[Iterable[str]] = None, add_bos: bool = True):
        self.vocab = list(vocab)
        self.bos_id, self.eos_id, self.model, self.add_bos = bos_id, eos_id, model, add_bos
        self.index: dict[str, int] = {}
        for i, t in enumerate(self.vocab):
            self.index.setdefault(t, i)
        self.max_len = min(64, max((len(t) for t in self.vocab), default=1))
        sp = set(special or [])
        for t in self.vocab:
            if len(t) > 2 and t.startswith("<") and t.endswith(">") and not t.startswith("<0x"):
                sp.add(t)
        self.special = sorted((s for s in sp if s in self.index), key=len, reverse=True)
        self.space = _SP_SPACE if any(_SP_SPACE in t for t in self.vocab[:4096]) else (
            _GPT2_SPACE if any(_GPT2_SPACE in t for t in self.vocab[:4096]) else " ")
        self.byte_tokens = {b: self.index[f"<0x{b:02X}>"] for b in range(256) if f"<0x{b:02X}>" in self.index}
        self._bytes_cache: Optional[list[bytes]] = None

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_gguf(cls, g) -> "Tokenizer":
        md = g.metadata
        toks = md.get("tokenizer.ggml.tokens")
        if toks is None:
            raise KeyError("GGUF file carries no tokenizer.ggml.tokens")
        return cls([str(t) for t in toks], bos_id=int(md.get("tokenizer.ggml.bos_token_id", 1)),
                   eos_id=int(md.get("tokenizer.ggml.eos_token_id", 2)),
                   model=str(md.get("tokenizer.ggml.model", "llama")),
                   add_bos=bool(md.get("tokenizer.ggml.add_bos_token", True)))

    @classmethod
    def ascii_fallback(cls, vocab_size: int = 1024) -> "Tokenizer":
        """Byte-level stand-in used when a checkpoint has no vocabulary: ids 0..2 are
        <unk>/<s>/</s>, then the 256 bytes, then unused filler ids."""
        vocab = ["<unk>", "<s>", "</s>"] + [chr(b) if 32 <= b < 127 else f"<0x{b:02X}>" for b in range(256)]
        vocab += [f"<unused{i}>" for i in range(max(0, vocab_size - len(vocab)))]
        t = cls(vocab[:max(vocab_size, 259)], bos_id=1, eos_id=2, model="ascii")
        for b in range(256):
            t.byte_tokens.setdefault(b, 3 + b)
        return t

    def gguf_metadata(self) -> dict:
        return {"tokenizer.ggml.model": self.model, "tokenizer.ggml.tokens": list(self.vocab),
                "tokenizer.ggml.bos_token_id": self.bos_id, "tokenizer.ggml.eos_token_id": self.eos_id}

    # ------------------------------------------------------------------ encode / decode
    def _encode_plain(self, text: str, out: list[int]) -> None:
        if self.space != " ":
            text = text.replace(" ", self.space)
            if self.space == _SP_SPACE and not text.startswith(self.space) and self.model != "ascii":
                text = self.space + text
        i, n = 0, len(text)
        while i < n:
            hit = -1
            for ln in range(min(self.max_len, n - i), 0, -1):
                tid = self.index.get(text[i:i + ln])
                if tid is not None:
                    hit, step = tid, ln
                    break
            if hit >= 0:
                out.append(hit)
                i += step
                continue
            ch = text[i].replace(self.space, " ") if self.space != " " else text[i]
            for b in ch.encode("utf-8"):
                out.append(self.byte_tokens.get(b, 0))
            i += 1

    def encode(self, text: str, add_bos: Optional[bool] = None) -> list[int]:
        out: list[int] = []
        if self.add_bos if add_bos is None else add_bos:
            out.append(self.bos_id)
        rest = text
        while rest:
            pos, tok = -1, None
            for s in self.special:
                p = rest.find(s)
                if p >= 0 and (pos < 0 or p < pos):
                    pos, tok = p, s
            if tok is None:
                self._encode_plain(rest, out)
                break
            if pos > 0:
                self._encode_plain(rest[:pos], out)
            out.append(self.index[tok])
            rest = rest[pos + len(tok):]
        return out

    def token_bytes(self, tid: int) -> bytes:
        if not 0 <= tid < len(self.vocab):
            return b""
        t = self.vocab[tid]
        if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
            try:
                return bytes([int(t[3:5], 16)])
            except ValueError:
                return t.encode()
        if t in self.special or t.startswith("<unused"):
            return b""
        return t.replace(_SP_SPACE, " ").replace(_GPT2_SPACE, " ").replace("Ċ", "\n").encode("utf-8")

    def vocab_bytes(self) -> list[bytes]:
        if self._bytes_cache is None:
            self._bytes_cache = [self.token_bytes(i) for i in range(len(self.vocab))]
        return self._bytes_cache

    def decode_token(self, tid: int) -> str:
        return self.token_bytes(tid).decode("utf-8", errors="replace")

    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        buf = bytearray()
        for t in ids:
            if not skip_special and 0 <= t < len(self.vocab) and self.vocab[t] in self.special:
                buf += self.vocab[t].encode()
            else:
                buf += self.token_bytes(int(t))
        s = buf.decode("utf-8", errors="replace")
        return s[1:] if s.startswith(" ") and self.space == _SP_SPACE else s

    def is_stop_token(self, tid: int) -> bool:
        if tid == self.eos_id or tid in HARD_STOP_IDS and self.model != "ascii" and len(self.vocab) > tid and \
                self.vocab[tid] in STOP_STRINGS:
            return True
        return 0 <= tid < len(self.vocab) and self.vocab[tid] in STOP_STRINGS

    def stop_ids(self) -> list[int]:
        ids = {self.eos_id}
        for s in STOP_STRINGS:
            if s in self.index:
                ids.add(self.index[s])
        return sorted(ids)

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)
