"""CSKV: flat binary KV-state files (checkpoint / resume of a sequence's KV cache).

Layout (little endian): magic ``CSKV`` | u32 version | u32 num_layers | u32 seq_len | variant header |
per layer K then V, each ``seq_len * num_kv_heads * head_dim`` elements in token-major order
``[token][kv_head][head_dim]``. Versions: 1 dense f32, 4 dense f32 + ``space_prefix_next`` byte,
5 dense f16; 2/6 hybrid (attention + GatedDeltaNet) and 3/7 MLA headers are parsed and written so
that files of those kinds can be inspected, but only dense states map onto this engine's pools.

Reference parity: oxide-core/src/cskv.rs:11-20 (versions), :144-325 (header parse), :328-368
(serialise), :370+ (layout of byte ranges). Paged pools are gathered into the contiguous layout on
save and scattered back on load; with tensor parallelism each rank writes its KV-head shard and a
JSON manifest names the shards.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from ..errors import EngineError, UnsupportedFormat

MAGIC = b"CSKV"
V_DENSE_V1, V_HYBRID, V_MLA, V_DENSE_V4, V_DENSE_F16, V_HYBRID_F16, V_MLA_F16 = 1, 2, 3, 4, 5, 6, 7
MAX_LAYERS = 1 << 16
_F16 = {V_DENSE_F16, V_HYBRID_F16, V_MLA_F16}


@dataclass
class CskvHeader:
    version: int
    num_layers: int
    seq_len: int
    num_kv_heads: int = 0
    head_dim: int = 0
    space_prefix_next: bool = False
    gdn_conv_state_len: int = 0
    gdn_recurrent_len: int = 0
    layer_kinds: list = field(default_factory=list)
    qk_dim: int = 0

    @property
    def kind(self) -> str:
        return {1: "dense", 4: "dense", 5: "dense", 2: "hybrid", 6: "hybrid", 3: "mla", 7: "mla"}[self.version]

    @property
    def dtype(self):
        return np.float16 if self.version in _F16 else np.float32

    def to_bytes(self) -> bytes:
        out = MAGIC + struct.pack("<III", self.version, self.num_layers, self.seq_len)
        if self.kind == "dense":
            out += struct.pack("<II", self.num_kv_heads, self.head_dim)
            if self.version >= V_DENSE_V4:
                out += bytes([1 if self.space_prefix_next else 0])
        elif self.kind == "hybrid":
            out += struct.pack("<IIII", self.num_kv_heads, self.head_dim, self.gdn_conv_state_len, self.gdn_recurrent_len)
            out += bytes(int(k) for k in self.layer_kinds)
        else:
            out += struct.pack("<I", self.qk_dim)
        return out

    @classmethod
    def parse(cls, b: bytes) -> tuple["CskvHeader", int]:
        if len(b) < 16 or b[:4] != MAGIC:
            raise UnsupportedFormat("not a CSKV file")
        version, n_layers, seq_len = struct.unpack_from("<III", b, 4)
        if version not in (1, 2, 3, 4, 5, 6, 7):
            raise UnsupportedFormat(f"unsupported CSKV version: {version}")
        if n_layers == 0 or n_layers > MAX_LAYERS:
            raise UnsupportedFormat(f"invalid layer count: {n_layers}")
        h = cls(version, n_layers, seq_len)
        off = 16
        if h.kind == "dense":
            h.num_kv_heads, h.head_dim = struct.unpack_from("<II", b, off)
            off += 8
            if version >= V_DENSE_V4:
                h.space_prefix_next = b[off] != 0
                off += 1
        elif h.kind == "hybrid":
            h.num_kv_heads, h.head_dim, h.gdn_conv_state_len, h.gdn_recurrent_len = struct.unpack_from("<IIII", b, off)
            off += 16
            h.layer_kinds = list(b[off:off + n_layers])
            off += n_layers
        else:
            (h.qk_dim,) = struct.unpack_from("<I", b, off)
            off += 4
        return h, off

    def layout(self) -> list[dict]:
        """Byte ranges of every buffer: [{layer, kind, offset, num_elements}] (dense variant)."""
        if self.kind != "dense":
            raise EngineError("byte-range layout is provided for dense states")
        off = len(self.to_bytes())
        n = self.seq_len * self.num_kv_heads * self.head_dim
        nb = n * np.dtype(self.dtype).itemsize
        out = []
        for li in range(self.num_layers):
            for kind in ("key", "value"):
                out.append({"layer": li, "kind": kind, "offset": off, "num_elements": n})
                off += nb
        return out


def write_dense(path: str, k_layers: list[np.ndarray], v_layers: list[np.ndarray], *, f16: bool = True,
                space_prefix_next: bool = False) -> CskvHeader:
    """k_layers[i], v_layers[i]: [seq_len, num_kv_heads, head_dim]."""
    seq_len, hkv, d = k_layers[0].shape
    h = CskvHeader(V_DENSE_F16 if f16 else V_DENSE_V4, len(k_layers), seq_len, hkv, d, space_prefix_next)
    dt = np.float16 if f16 else np.float32
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(h.to_bytes())
        for k, v in zip(k_layers, v_layers):
            f.write(np.ascontiguousarray(k, dtype=dt).tobytes())
            f.write(np.ascontiguousarray(v, dtype=dt).tobytes())
    os.replace(tmp, path)
    return h


def read_dense(path: str) -> tuple[CskvHeader, list[np.ndarray], list[np.ndarray]]:
    raw = np.fromfile(path, dtype=np.uint8)
    h, off = CskvHeader.parse(raw[:4096].tobytes())
    if h.kind != "dense":
        raise EngineError(f"{path} holds a {h.kind} state; only dense states can be restored")
    shape = (h.seq_len, h.num_kv_heads, h.head_dim)
    n = int(np.prod(shape))
    dt = np.dtype(h.dtype)
    ks, vs = [], []
    for _ in range(h.num_layers):
        ks.append(raw[off:off + n * dt.itemsize].view(dt).reshape(shape).astype(np.float32))
        off += n * dt.itemsize
        vs.append(raw[off:off + n * dt.itemsize].view(dt).reshape(shape).astype(np.float32))
        off += n * dt.itemsize
    return h, ks, vs


def save_sequence(engine, req_id: int, path: str, f16: bool = True) -> CskvHeader:
    """Gathers the pages of a running or just-finished request into a CSKV file (per rank: this
    rank's KV-head shard; rank 0 also writes `<path>.manifest.json`)."""
    import torch

    info = engine.sched.request_info(req_id)
    if info is None:
        raise EngineError(f"request {req_id} is not resident")
    n_tok, blocks = int(info["computed"]), list(info["blocks"])
    nb = (n_tok + 15) // 16
    idx = torch.as_tensor(blocks[:nb], dtype=torch.long)
    model = engine.model
    caches = (model.pk, model.pv) if engine.cpu else (model.k_cache, model.v_cache)
    ks, vs = [], []
    for li in range(engine.model_cfg.n_layers):
        for dst, cache in ((ks, caches[0][li]), (vs, caches[1][li])):
            g = cache[idx.to(cache.device)]  # [nb, hkv, 16, D]
            dst.append(g.permute(0, 2, 1, 3).reshape(nb * 16, g.shape[1], g.shape[3])[:n_tok].float().cpu().numpy())
    rank, world = getattr(engine, "rank", 0), getattr(engine, "world", 1)
    shard = path if world == 1 else f"{path}.rank{rank}"
    h = write_dense(shard, ks, vs, f16=f16)
    if rank == 0:
        toks = engine.sched.request_tokens(req_id)
        json.dump({"format": "CSKV", "version": h.version, "world": world, "tokens": int(n_tok),
                   "token_ids": [int(t) for t in toks[:n_tok]] if toks is not None else [],
                   "shards": [path if world == 1 else f"{path}.rank{r}" for r in range(world)]},
                  open(path + ".manifest.json", "w"))
    return h


def load_prefix(engine, path: str) -> int:
    """Restores a saved state as a cached prefix: the KV is scattered into fresh blocks which are
    handed to the radix cache under the saved token ids, so the next request with that prefix
    resumes without recomputation. Returns the number of tokens restored (whole blocks)."""
    import torch

    man = json.load(open(path + ".manifest.json"))
    rank, world = getattr(engine, "rank", 0), getattr(engine, "world", 1)
    if man["world"] != world:
        raise EngineError(f"state was saved with world={man['world']}, engine runs world={world}")
    h, ks, vs = read_dense(man["shards"][rank])
    toks = np.asarray(man["token_ids"], dtype=np.int32)
    n_full = min(h.seq_len, toks.size) // 16
    if n_full == 0:
        return 0
    pool = engine.sched
    blocks = engine.sched.alloc_blocks(n_full)
    if blocks is None:
        raise EngineError("not enough free KV blocks to restore the state")
    model = engine.model
    caches = (model.pk, model.pv) if engine.cpu else (model.k_cache, model.v_cache)
    idx = torch.as_tensor(blocks, dtype=torch.long)
    for li in range(h.num_layers):
        for src, cache in ((ks[li], caches[0][li]), (vs[li], caches[1][li])):
            t = torch.from_numpy(src[:n_full * 16]).reshape(n_full, 16, h.num_kv_heads, h.head_dim).permute(0, 2, 1, 3)
            cache[idx.to(cache.device)] = t.to(device=cache.device, dtype=cache.dtype)
    engine.sched.radix_insert(toks[:n_full * 16], blocks)
    engine.sched.release_blocks(blocks)  # the cache keeps its own reference
    return n_full * 16
