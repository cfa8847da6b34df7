"""GGUF v1-v3 reader (mmap, zero-copy tensor views) and v3 writer.

Layout handled: magic ``GGUF`` | version u32 | n_tensors u64 | n_kv u64 | metadata key/values of
the 13 GGUF value types | tensor directory (name, n_dims, dims u64[], type u32, offset u64) |
padding to ``general.alignment`` (default 32) | tensor data. Version 1 files use u32 counts and
string lengths.

Reference parity: GgufFile::parse (oxide-models/src/formats.rs:308-459), value types
(formats.rs:461-562), type codes (formats.rs:380-421); the reference has no writer besides its
`oxide-quantize` tool (oxide-cli/src/bin/oxide_quantize.rs).
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Any, BinaryIO

import numpy as np

from ..errors import UnsupportedFormat
from . import quants

GGUF_MAGIC = b"GGUF"

# metadata value types
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {
    T_U8: ("<B", 1), T_I8: ("<b", 1), T_U16: ("<H", 2), T_I16: ("<h", 2), T_U32: ("<I", 4),
    T_I32: ("<i", 4), T_F32: ("<f", 4), T_BOOL: ("<?", 1), T_U64: ("<Q", 8), T_I64: ("<q", 8),
    T_F64: ("<d", 8),
}
_NP_SCALAR = {
    T_U8: np.uint8, T_I8: np.int8, T_U16: np.uint16, T_I16: np.int16, T_U32: np.uint32,
    T_I32: np.int32, T_F32: np.float32, T_BOOL: np.bool_, T_U64: np.uint64, T_I64: np.int64,
    T_F64: np.float64,
}


@dataclass
class GgufTensorInfo:
    name: str
    shape: tuple[int, ...]  # GGUF order: innermost dimension first
    type_code: int
    offset: int  # relative to the start of the data section

    @property
    def type_name(self) -> str:
        return quants.CODE_TO_NAME[self.type_code]

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        q = quants.type_info(self.type_code)
        return self.n_elements // q.block * q.nbytes

    @property
    def torch_shape(self) -> tuple[int, ...]:
        """Row-major shape as used by the models ([out_features, in_features] for weights)."""
        return tuple(reversed(self.shape))


@dataclass
class GgufFile:
    version: int
    metadata: dict[str, Any]
    tensors: dict[str, GgufTensorInfo]
    data_offset: int
    path: str | None = None
    _mm: Any = field(default=None, repr=False)
    _buf: Any = field(default=None, repr=False)

    # ------------------------------------------------------------------ parsing
    @classmethod
    def open(cls, path: str) -> "GgufFile":
        f = open(path, "rb")
        try:
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        finally:
            f.close()
        g = cls.parse(memoryview(mm))
        g.path = path
        g._mm = mm
        return g

    @classmethod
    def parse(cls, buf: bytes | memoryview) -> "GgufFile":
        buf = memoryview(buf)
        if len(buf) < 16 or bytes(buf[0:4]) != GGUF_MAGIC:
            raise UnsupportedFormat("not a GGUF file (bad magic)")
        version = struct.unpack_from("<I", buf, 4)[0]
        if version not in (1, 2, 3):
            raise UnsupportedFormat(f"unsupported GGUF version {version}")
        wide = version >= 2
        off = 8

        def rd_count():
            nonlocal off
            if wide:
                v = struct.unpack_from("<Q", buf, off)[0]
                off += 8
            else:
                v = struct.unpack_from("<I", buf, off)[0]
                off += 4
            return v

        def rd_str():
            nonlocal off
            n = rd_count()
            if off + n > len(buf):
                raise UnsupportedFormat("truncated GGUF string")
            s = bytes(buf[off:off + n]).decode("utf-8", errors="replace")
            off += n
            return s

        def rd_value(t):
            nonlocal off
            if t in _SCALAR:
                fmt, n = _SCALAR[t]
                v = struct.unpack_from(fmt, buf, off)[0]
                off += n
                return v
            if t == T_STR:
                return rd_str()
            if t == T_ARR:
                et = struct.unpack_from("<I", buf, off)[0]
                off += 4
                cnt = rd_count()
                if et in _NP_SCALAR:
                    dt = np.dtype(_NP_SCALAR[et])
                    arr = np.frombuffer(buf, dtype=dt, count=cnt, offset=off)
                    off += cnt * dt.itemsize
                    return arr
                return [rd_value(et) for _ in range(cnt)]
            raise UnsupportedFormat(f"unknown GGUF metadata type {t}")

        n_tensors = rd_count()
        n_kv = rd_count()
        metadata: dict[str, Any] = {}
        for _ in range(n_kv):
            key = rd_str()
            t = struct.unpack_from("<I", buf, off)[0]
            off += 4
            metadata[key] = rd_value(t)
        tensors: dict[str, GgufTensorInfo] = {}
        for _ in range(n_tensors):
            name = rd_str()
            nd = struct.unpack_from("<I", buf, off)[0]
            off += 4
            if wide:
                dims = struct.unpack_from(f"<{nd}Q", buf, off)
                off += 8 * nd
            else:
                dims = struct.unpack_from(f"<{nd}I", buf, off)
                off += 4 * nd
            code = struct.unpack_from("<I", buf, off)[0]
            off += 4
            if code not in quants.CODE_TO_NAME:
                raise UnsupportedFormat(f"Unsupported GGUF quant type code: {code}")
            toff = struct.unpack_from("<Q", buf, off)[0]
            off += 8
            tensors[name] = GgufTensorInfo(name, tuple(int(d) for d in dims), code, toff)
        align = int(metadata.get("general.alignment", 32))
        data_offset = (off + align - 1) // align * align
        g = cls(version, metadata, tensors, data_offset)
        g._buf = buf
        return g

    # ------------------------------------------------------------------ access
    def raw(self, name: str) -> np.ndarray:
        """uint8 view (zero copy) of the packed bytes of a tensor."""
        t = self.tensors[name]
        start = self.data_offset + t.offset
        return np.frombuffer(self._buf, dtype=np.uint8, count=t.nbytes, offset=start)

    def dequantize(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return quants.dequantize(t.type_code, self.raw(name), t.n_elements).reshape(t.torch_shape)

    def architecture(self) -> str:
        return str(self.metadata.get("general.architecture", "llama"))

    def close(self) -> None:
        self._buf = None
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass
            self._mm = None


# ---------------------------------------------------------------------------------------- writer
def _wr_str(f: BinaryIO, s: str) -> None:
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)))
    f.write(b)


def _wr_value(f: BinaryIO, v: Any) -> None:
    if isinstance(v, bool):
        f.write(struct.pack("<I?", T_BOOL, v))
    elif isinstance(v, (int, np.integer)):
        v = int(v)
        if 0 <= v < 2 ** 32:
            f.write(struct.pack("<II", T_U32, v))
        elif v < 0 and v >= -2 ** 31:
            f.write(struct.pack("<Ii", T_I32, v))
        elif v < 0:
            f.write(struct.pack("<Iq", T_I64, v))
        else:
            f.write(struct.pack("<IQ", T_U64, v))
    elif isinstance(v, (float, np.floating)):
        f.write(struct.pack("<If", T_F32, float(v)))
    elif isinstance(v, str):
        f.write(struct.pack("<I", T_STR))
        _wr_str(f, v)
    elif isinstance(v, np.ndarray):
        et = {np.dtype(np.int32): T_I32, np.dtype(np.uint32): T_U32, np.dtype(np.float32): T_F32,
              np.dtype(np.uint8): T_U8, np.dtype(np.int64): T_I64}.get(v.dtype)
        if et is None:
            raise TypeError(f"unsupported array dtype {v.dtype}")
        f.write(struct.pack("<IIQ", T_ARR, et, v.size))
        f.write(np.ascontiguousarray(v).tobytes())
    elif isinstance(v, (list, tuple)):
        if all(isinstance(x, str) for x in v):
            f.write(struct.pack("<IIQ", T_ARR, T_STR, len(v)))
            for x in v:
                _wr_str(f, x)
        elif all(isinstance(x, (int, np.integer)) and not isinstance(x, bool) for x in v):
            f.write(struct.pack("<IIQ", T_ARR, T_I32, len(v)))
            f.write(np.asarray(v, dtype=np.int32).tobytes())
        elif all(isinstance(x, (float, int)) for x in v):
            f.write(struct.pack("<IIQ", T_ARR, T_F32, len(v)))
            f.write(np.asarray(v, dtype=np.float32).tobytes())
        else:
            raise TypeError("unsupported metadata list")
    else:
        raise TypeError(f"unsupported metadata value {type(v)}")


class GgufWriter:
    """Streams a GGUF v3 file: metadata first, then tensors (already packed bytes or float arrays)."""

    def __init__(self, path: str, metadata: dict[str, Any], alignment: int = 32):
        self.path = path
        self.metadata = dict(metadata)
        self.alignment = alignment
        self.metadata.setdefault("general.alignment", alignment)
        self._tensors: list[tuple[str, tuple[int, ...], int, np.ndarray]] = []

    def add_tensor(self, name: str, array: np.ndarray, type_name: str = "F32") -> None:
        """`array` is row-major float data ([out, in] for weights); it is encoded to `type_name`."""
        arr = np.ascontiguousarray(array, dtype=np.float32)
        code = quants.TYPES[type_name].code
        if arr.ndim >= 1 and arr.shape[-1] % quants.TYPES[type_name].block:
            raise ValueError(f"{name}: inner dimension {arr.shape[-1]} does not fit {type_name} blocks")
        packed = quants.quantize(type_name, arr)
        self._tensors.append((name, tuple(reversed(arr.shape)), code, packed))

    def add_raw(self, name: str, torch_shape: tuple[int, ...], type_name: str, packed: np.ndarray) -> None:
        code = quants.TYPES[type_name].code
        self._tensors.append((name, tuple(reversed(torch_shape)), code,
                              np.ascontiguousarray(packed).view(np.uint8).reshape(-1)))

    def write(self) -> None:
        tmp = self.path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(GGUF_MAGIC)
            f.write(struct.pack("<IQQ", 3, len(self._tensors), len(self.metadata)))
            for k, v in self.metadata.items():
                _wr_str(f, k)
                _wr_value(f, v)
            off = 0
            offsets = []
            for _, _, _, packed in self._tensors:
                offsets.append(off)
                off += (packed.size + self.alignment - 1) // self.alignment * self.alignment
            for (name, dims, code, _), o in zip(self._tensors, offsets):
                _wr_str(f, name)
                f.write(struct.pack("<I", len(dims)))
                f.write(struct.pack(f"<{len(dims)}Q", *dims))
                f.write(struct.pack("<IQ", code, o))
            pos = f.tell()
            pad = (pos + self.alignment - 1) // self.alignment * self.alignment - pos
            f.write(b"\x00" * pad)
            for (_, _, _, packed) in self._tensors:
                f.write(packed.tobytes())
                pad = (packed.size + self.alignment - 1) // self.alignment * self.alignment - packed.size
                f.write(b"\x00" * pad)
        os.replace(tmp, self.path)
