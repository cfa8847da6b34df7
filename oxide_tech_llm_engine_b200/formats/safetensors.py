"""SafeTensors reader/writer (single file, sharded index, directory with config.json).

Header: u64 little-endian length + JSON {name: {dtype, shape, data_offsets}, "__metadata__": ...}.
Reference parity: SafeTensorsHeader (oxide-models/src/formats.rs:165-234). The reference's model
loader only copies `model.embed_tokens.weight` (llama3.rs:1936-1954); this one loads every tensor,
including bf16, fp16, fp8 (e4m3) and sharded checkpoints.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Any, Optional

import numpy as np

from ..errors import UnsupportedFormat
from . import quants

_DTYPES = {
    "F64": (np.float64, 8), "F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2),
    "I64": (np.int64, 8), "I32": (np.int32, 4), "I16": (np.int16, 2), "I8": (np.int8, 1),
    "U8": (np.uint8, 1), "BOOL": (np.bool_, 1), "F8_E4M3": (np.uint8, 1), "F8_E5M2": (np.uint8, 1),
}


class SafeTensorsFile:
    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            self._mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._mm) < 8:
            raise UnsupportedFormat("safetensors: file too small")
        (n,) = struct.unpack_from("<Q", self._mm, 0)
        if 8 + n > len(self._mm):
            raise UnsupportedFormat("safetensors: header length exceeds file size")
        self.header: dict[str, Any] = json.loads(bytes(self._mm[8:8 + n]).decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self.data_start = 8 + n

    def names(self):
        return self.header.keys()

    def info(self, name: str) -> dict:
        return self.header[name]

    def raw(self, name: str) -> np.ndarray:
        e = self.header[name]
        if e["dtype"] not in _DTYPES:
            raise UnsupportedFormat(f"safetensors dtype {e['dtype']}")
        dt, sz = _DTYPES[e["dtype"]]
        lo, hi = e["data_offsets"]
        count = (hi - lo) // sz
        return np.frombuffer(self._mm, dtype=dt, count=count, offset=self.data_start + lo).reshape(e["shape"])

    def f32(self, name: str) -> np.ndarray:
        e = self.header[name]
        a = self.raw(name)
        if e["dtype"] == "BF16":
            return (a.astype(np.uint32) << 16).view(np.float32)
        if e["dtype"] == "F8_E4M3":
            return quants.e4m3_to_f32(a.reshape(-1)).reshape(e["shape"])
        return a.astype(np.float32)


class SafeTensorsRepo:
    """A model directory, an index json or one .safetensors file."""

    def __init__(self, path: str):
        self.path = path
        self.files: dict[str, SafeTensorsFile] = {}
        self.where: dict[str, str] = {}
        self.dir = path if os.path.isdir(path) else os.path.dirname(os.path.abspath(path))
        shards: list[str] = []
        if os.path.isdir(path):
            idx = os.path.join(path, "model.safetensors.index.json")
            if os.path.exists(idx):
                shards = sorted(set(json.load(open(idx))["weight_map"].values()))
            else:
                shards = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
            shards = [os.path.join(path, s) for s in shards]
        elif path.endswith(".index.json"):
            shards = [os.path.join(self.dir, s) for s in sorted(set(json.load(open(path))["weight_map"].values()))]
        else:
            shards = [path]
        if not shards:
            raise UnsupportedFormat(f"no .safetensors files under {path}")
        for s in shards:
            f = SafeTensorsFile(s)
            self.files[s] = f
            for n in f.names():
                self.where[n] = s

    def names(self):
        return self.where.keys()

    def has(self, name):
        return name in self.where

    def shape(self, name):
        return tuple(self.files[self.where[name]].info(name)["shape"])

    def f32(self, name):
        return self.files[self.where[name]].f32(name)

    def model_config(self):
        from ..models.config import ModelConfig

        cfg_path = os.path.join(self.dir, "config.json")
        if not os.path.exists(cfg_path):
            raise UnsupportedFormat(f"{cfg_path} is needed to size a SafeTensors model")
        c = json.load(open(cfg_path))
        n_heads = c["num_attention_heads"]
        arch = "mixtral" if c.get("num_local_experts", 0) else "llama"
        rs = c.get("rope_scaling") or {}
        return ModelConfig(
            name=c.get("_name_or_path", arch) or arch, arch=arch, n_layers=c["num_hidden_layers"],
            d_model=c["hidden_size"], n_heads=n_heads, n_kv_heads=c.get("num_key_value_heads", n_heads),
            head_dim=c.get("head_dim") or c["hidden_size"] // n_heads, ffn_dim=c["intermediate_size"],
            vocab_size=c["vocab_size"], max_ctx=c.get("max_position_embeddings", 8192),
            rope_theta=float(c.get("rope_theta", 10000.0)), rms_eps=float(c.get("rms_norm_eps", 1e-5)),
            rope_scaling={"llama3": "llama3", "linear": "linear", "yarn": "yarn"}.get(
                rs.get("rope_type", rs.get("type", "none")), "none"),
            rope_factor=float(rs.get("factor", 1.0)),
            rope_orig_ctx=int(rs.get("original_max_position_embeddings", 8192)),
            rope_low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
            rope_high_freq_factor=float(rs.get("high_freq_factor", 4.0)),
            tie_embeddings=bool(c.get("tie_word_embeddings", False)),
            n_experts=int(c.get("num_local_experts", 0) or 0),
            n_experts_used=int(c.get("num_experts_per_tok", 0) or 0),
            sliding_window=int(c.get("sliding_window") or 0) if arch != "mixtral" else 0,
            attn_bias=bool(c.get("attention_bias", False)),
            bos_id=int(c.get("bos_token_id", 1) or 1),
            eos_id=int(c["eos_token_id"][0] if isinstance(c.get("eos_token_id"), list) else c.get("eos_token_id", 2) or 2),
        )


def write_safetensors(path: str, tensors: dict[str, np.ndarray], dtype: str = "F32",
                      metadata: Optional[dict[str, str]] = None) -> None:
    """Writes float arrays as F32, F16 or BF16."""
    header: dict[str, Any] = {}
    blobs = []
    off = 0
    for name, arr in tensors.items():
        a = np.ascontiguousarray(arr, dtype=np.float32)
        if dtype == "BF16":
            raw = quants.quantize("BF16", a)
        elif dtype == "F16":
            raw = a.astype(np.float16).view(np.uint8).reshape(-1)
        else:
            raw = a.view(np.uint8).reshape(-1)
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [off, off + raw.size]}
        blobs.append(raw)
        off += raw.size
    if metadata:
        header["__metadata__"] = metadata
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for b in blobs:
            f.write(b.tobytes())
