"""KV tiers and block hand-off: device (tier 1) -> pinned host (tier 2) -> file (tier 3), chained
prefix hashes, LRU demotion, promotion on hit, checksummed block payloads, quantised KV blocks,
context shifting, prompt-cache registry and JSON dumps.

Reference parity: HierarchicalKvCache (oxide-alloc/src/hierarchical_kv.rs:27-310: FNV-1a chained
prefix hash :124-131, tier maps, LRU demotion T1->T2->T3 :135-173, promote on hit :207-242,
DistributedKvBlockPayload with additive checksum :51-79,245-294), QuantizedKvBlock F32/F16/Q8/Q4
(kv_advanced.rs:39-175), ContextShiftManager (:299-339), PromptCacheRegistry (:343-390),
KvCacheDumpContainer (:394-414). In the reference all three tiers are host hash maps; here tier 1
is the device block pool of the engine, tier 2 pinned host memory and tier 3 files.
"""
from __future__ import annotations

import json
import os
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from ..errors import EngineError

FNV_OFFSET, FNV_PRIME, MASK64 = 0xCBF29CE484222325, 0x100000001B3, 0xFFFFFFFFFFFFFFFF


def fnv1a_chain(prev: int, tokens) -> int:
    """Hash of a block given the hash of everything before it (prefix identity)."""
    h = (FNV_OFFSET ^ prev) & MASK64
    for t in np.asarray(tokens, dtype=np.uint32).tolist():
        for b in range(4):
            h ^= (t >> (8 * b)) & 0xFF
            h = (h * FNV_PRIME) & MASK64
    return h


def prefix_hashes(tokens, block: int = 16) -> list[int]:
    """Chained hash of every whole block of `tokens` (native when the host runtime is built)."""
    try:
        from .._build import host_ext

        return [int(h) for h in host_ext().prefix_hashes(np.ascontiguousarray(tokens, dtype=np.int32), int(block))]
    except (ImportError, AttributeError):
        pass
    out, prev = [], 0
    for i in range(0, len(tokens) // block * block, block):
        prev = fnv1a_chain(prev, tokens[i:i + block])
        out.append(prev)
    return out


@dataclass
class KvBlockPayload:
    """One KV block in transit between tiers or ranks."""
    prefix_hash: int
    tokens: np.ndarray          # [16] int32
    k: np.ndarray               # [layers, hkv, 16, D]; float16, float32, bf16 bit patterns as int16, or int8 codes
    v: np.ndarray
    checksum: int = 0
    scales: Optional[np.ndarray] = None   # [2, layers] fp32 (K row, V row) when k / v hold int8 codes: value = code * scale

    def compute_checksum(self) -> int:
        s = int(self.tokens.astype(np.int64).sum())
        s += int(self.k.view(np.uint16).astype(np.uint64).sum()) + int(self.v.view(np.uint16).astype(np.uint64).sum())
        return s & MASK64

    def seal(self) -> "KvBlockPayload":
        self.checksum = self.compute_checksum()
        return self

    def verify(self) -> bool:
        return self.checksum == self.compute_checksum()

    def to_bytes(self) -> bytes:
        hdr = json.dumps({"hash": self.prefix_hash, "checksum": self.checksum, "kshape": list(self.k.shape),
                          "dtype": str(self.k.dtype),
                          "scales": None if self.scales is None else np.asarray(self.scales, np.float32).tolist()}).encode()
        return len(hdr).to_bytes(4, "little") + hdr + self.tokens.astype(np.int32).tobytes() + \
            np.ascontiguousarray(self.k).tobytes() + np.ascontiguousarray(self.v).tobytes()

    @classmethod
    def from_bytes(cls, b: bytes) -> "KvBlockPayload":
        n = int.from_bytes(b[:4], "little")
        hdr = json.loads(b[4:4 + n])
        off = 4 + n
        toks = np.frombuffer(b, dtype=np.int32, count=16, offset=off)
        off += 64
        shape = tuple(hdr["kshape"])
        cnt = int(np.prod(shape))
        dt = np.dtype(hdr.get("dtype", "float16"))
        k = np.frombuffer(b, dtype=dt, count=cnt, offset=off).reshape(shape)
        v = np.frombuffer(b, dtype=dt, count=cnt, offset=off + dt.itemsize * cnt).reshape(shape)
        sc = hdr.get("scales")
        p = cls(hdr["hash"], toks.copy(), k.copy(), v.copy(), hdr["checksum"],
                None if sc is None else np.asarray(sc, dtype=np.float32))
        if not p.verify():
            raise EngineError("KV block payload failed its checksum")
        return p


class HierarchicalKvCache:
    """Tier 2 (pinned host) and tier 3 (directory of files) behind the device pool.

    `demote(payload)` is called with blocks evicted from the device radix cache; `lookup(hash)`
    promotes a block back (the caller scatters it into a fresh device block)."""

    def __init__(self, host_blocks: int = 8192, storage_blocks: int = 32768, storage_dir: Optional[str] = None):
        self.host_cap, self.storage_cap, self.dir = host_blocks, storage_blocks, storage_dir
        self.host: "OrderedDict[int, KvBlockPayload]" = OrderedDict()
        self.storage: "OrderedDict[int, str]" = OrderedDict()
        self.stats = {"host_hits": 0, "storage_hits": 0, "misses": 0, "demoted_to_storage": 0, "dropped": 0}
        if storage_dir:
            os.makedirs(storage_dir, exist_ok=True)

    def demote(self, p: KvBlockPayload) -> None:
        self.host[p.prefix_hash] = p.seal()
        self.host.move_to_end(p.prefix_hash)
        while len(self.host) > self.host_cap:
            h, old = self.host.popitem(last=False)
            self._to_storage(h, old)

    def _to_storage(self, h: int, p: KvBlockPayload) -> None:
        if not self.dir or self.storage_cap <= 0:
            self.stats["dropped"] += 1
            return
        path = os.path.join(self.dir, f"{h:016x}.kvb")
        try:
            tmp = f"{path}.{os.getpid()}.tmp"
            with open(tmp, "wb") as f:
                f.write(p.to_bytes())
            os.replace(tmp, path)          # never a half-written file under the final name
        except OSError:
            self.stats["dropped"] += 1
            self.stats["storage_errors"] = self.stats.get("storage_errors", 0) + 1
            return
        self.storage[h] = path
        self.stats["demoted_to_storage"] += 1
        while len(self.storage) > self.storage_cap:
            _, old = self.storage.popitem(last=False)
            try:
                os.unlink(old)
            except OSError:
                pass
            self.stats["dropped"] += 1

    def lookup(self, h: int) -> Optional[KvBlockPayload]:
        if h in self.host:
            self.host.move_to_end(h)
            self.stats["host_hits"] += 1
            return self.host[h]
        path = self.storage.pop(h, None)
        if path is not None:
            try:
                with open(path, "rb") as f:
                    p = KvBlockPayload.from_bytes(f.read())
                os.unlink(path)
            except (OSError, EngineError, ValueError):
                # the file is gone or damaged (another process cleaned the directory, a torn write):
                # the block is simply not cached any more and the prompt is prefilled
                self.stats["misses"] += 1
                self.stats["storage_errors"] = self.stats.get("storage_errors", 0) + 1
                return None
            self.stats["storage_hits"] += 1
            self.demote(p)  # promoted one tier up
            return p
        self.stats["misses"] += 1
        return None

    def match_prefix(self, tokens) -> list[KvBlockPayload]:
        out = []
        for h in prefix_hashes(tokens):
            p = self.lookup(h)
            if p is None:
                break
            out.append(p)
        return out


# ------------------------------------------------------------------------------------------------
class QuantizedKvBlock:
    """Per-tensor quantised copy of a KV block: f32, f16, q8 (absmax / 127) or q4 (absmax / 7,
    two values per byte)."""

    def __init__(self, mode: str, data: np.ndarray, scale: float, shape: tuple):
        self.mode, self.data, self.scale, self.shape = mode, data, scale, shape

    @classmethod
    def quantize(cls, x: np.ndarray, mode: str) -> "QuantizedKvBlock":
        x = np.ascontiguousarray(x, dtype=np.float32)
        if mode == "f32":
            return cls(mode, x.copy(), 1.0, x.shape)
        if mode == "f16":
            return cls(mode, x.astype(np.float16), 1.0, x.shape)
        amax = float(np.abs(x).max())
        if mode == "q8":
            s = amax / 127.0 if amax > 0 else 1.0
            return cls(mode, np.clip(np.rint(x / s), -127, 127).astype(np.int8), s, x.shape)
        if mode == "q4":
            s = amax / 7.0 if amax > 0 else 1.0
            q = (np.clip(np.rint(x / s), -7, 7).astype(np.int8) + 8).astype(np.uint8).reshape(-1)
            if q.size % 2:
                q = np.append(q, np.uint8(8))
            return cls(mode, (q[0::2] | (q[1::2] << 4)).astype(np.uint8), s, x.shape)
        raise ValueError(mode)

    def dequantize(self) -> np.ndarray:
        if self.mode in ("f32", "f16"):
            return self.data.astype(np.float32)
        if self.mode == "q8":
            return self.data.astype(np.float32) * self.scale
        n = int(np.prod(self.shape))
        q = np.empty(self.data.size * 2, np.int16)
        q[0::2] = self.data & 0xF
        q[1::2] = self.data >> 4
        return ((q[:n] - 8).astype(np.float32) * self.scale).reshape(self.shape)

    def nbytes(self) -> int:
        return int(self.data.nbytes)


class ContextShiftManager:
    """When a sequence outgrows the window keep the first `keep_prefix` tokens and drop the
    oldest `max(shift_step, overflow)` tokens after them (positions are renumbered by the caller)."""

    def __init__(self, max_ctx: int, keep_prefix: int = 4, shift_step: int = 256):
        self.max_ctx, self.keep_prefix, self.shift_step = max_ctx, keep_prefix, shift_step

    def plan(self, n_tokens: int, incoming: int = 1) -> Optional[tuple[int, int]]:
        """None when everything fits, else (first_dropped, n_dropped)."""
        overflow = n_tokens + incoming - self.max_ctx
        if overflow <= 0:
            return None
        drop = max(self.shift_step, overflow)
        drop = min(drop, max(n_tokens - self.keep_prefix, 0))
        return self.keep_prefix, drop

    def apply(self, tokens: list) -> list:
        p = self.plan(len(tokens))
        if p is None:
            return tokens
        first, n = p
        return tokens[:first] + tokens[first + n:]


class PromptCacheRegistry:
    """Exact-match (FNV) registry of prompt -> saved state path, with a longest-prefix fallback."""

    def __init__(self):
        self.exact: dict[int, str] = {}
        self.entries: list[tuple[list, str]] = []

    @staticmethod
    def key(tokens) -> int:
        return fnv1a_chain(0, tokens)

    def register(self, tokens, path: str) -> None:
        self.exact[self.key(tokens)] = path
        self.entries.append((list(tokens), path))

    def lookup(self, tokens) -> tuple[Optional[str], int]:
        p = self.exact.get(self.key(tokens))
        if p is not None:
            return p, len(tokens)
        best, best_n = None, 0
        for t, path in self.entries:
            n = 0
            for a, b in zip(t, tokens):
                if a != b:
                    break
                n += 1
            if n == len(t) and n > best_n:
                best, best_n = path, n
        return best, best_n


class KvCacheDumpContainer:
    """JSON dump / reload of quantised KV blocks (debugging aid)."""

    def __init__(self):
        self.blocks: list[dict] = []

    def add(self, layer: int, kind: str, q: QuantizedKvBlock) -> None:
        self.blocks.append({"layer": layer, "kind": kind, "mode": q.mode, "scale": q.scale, "shape": list(q.shape),
                            "data": q.data.reshape(-1).tolist()})

    def dump(self, path: str) -> None:
        json.dump({"format": "oxide-kv-dump", "blocks": self.blocks}, open(path, "w"))

    @classmethod
    def load(cls, path: str) -> list[tuple[int, str, QuantizedKvBlock]]:
        out = []
        dt = {"f32": np.float32, "f16": np.float16, "q8": np.int8, "q4": np.uint8}
        for b in json.load(open(path))["blocks"]:
            data = np.asarray(b["data"], dtype=dt[b["mode"]])
            if b["mode"] in ("f32", "f16", "q8"):
                data = data.reshape(b["shape"])
            out.append((b["layer"], b["kind"], QuantizedKvBlock(b["mode"], data, b["scale"], tuple(b["shape"]))))
        return out
