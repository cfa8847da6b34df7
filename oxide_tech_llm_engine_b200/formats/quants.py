"""GGML-exact block codecs (numpy) for every GGUF tensor type the engine serves.

``dequantize(type, raw_bytes, n_elements)`` is bit-compatible with GGUF files written by
llama.cpp-compatible tools and is the CPU oracle for the device decoders in
``csrc/kernels/quant_blocks.cuh``. ``quantize(type, x)`` produces valid encodings for synthetic
checkpoints (it uses straightforward scale searches, not llama.cpp's iterative refinements; any
valid encoding is decodable by every reader).

Reference parity: block structs of oxide-quant/src/int_quant.rs:10-811 and gguf_quants.rs:16-444,
NVFP4 of nvfp4.rs:27-129, FP8 E4M3 of fp8.rs:13-112; type codes of oxide-models/src/formats.rs:380-421.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class QuantInfo:
    name: str
    code: int
    block: int  # elements per block
    nbytes: int  # bytes per block


TYPES: dict[str, QuantInfo] = {
    q.name: q
    for q in [
        QuantInfo("F32", 0, 1, 4),
        QuantInfo("F16", 1, 1, 2),
        QuantInfo("Q4_0", 2, 32, 18),
        QuantInfo("Q4_1", 3, 32, 20),
        QuantInfo("Q5_0", 6, 32, 22),
        QuantInfo("Q5_1", 7, 32, 24),
        QuantInfo("Q8_0", 8, 32, 34),
        QuantInfo("Q8_1", 9, 32, 36),
        QuantInfo("Q2_K", 10, 256, 84),
        QuantInfo("Q3_K", 11, 256, 110),
        QuantInfo("Q4_K", 12, 256, 144),
        QuantInfo("Q5_K", 13, 256, 176),
        QuantInfo("Q6_K", 14, 256, 210),
        QuantInfo("Q8_K", 15, 256, 292),
        QuantInfo("IQ2_XXS", 16, 256, 66),
        QuantInfo("IQ2_XS", 17, 256, 74),
        QuantInfo("IQ3_XXS", 18, 256, 98),
        QuantInfo("IQ1_S", 19, 256, 50),
        QuantInfo("IQ4_NL", 20, 32, 18),
        QuantInfo("IQ3_S", 21, 256, 110),
        QuantInfo("IQ2_S", 22, 256, 82),
        QuantInfo("IQ4_XS", 23, 256, 136),
        QuantInfo("I8", 24, 1, 1),
        QuantInfo("I16", 25, 1, 2),
        QuantInfo("I32", 26, 1, 4),
        QuantInfo("I64", 27, 1, 8),
        QuantInfo("F64", 28, 1, 8),
        QuantInfo("IQ1_M", 29, 256, 56),
        QuantInfo("BF16", 30, 1, 2),
        QuantInfo("TQ1_0", 34, 256, 54),
        QuantInfo("TQ2_0", 35, 256, 66),
        QuantInfo("MXFP4", 39, 32, 17),
        QuantInfo("PQ2_0", 142, 128, 36),
        QuantInfo("PTQ1_0", 143, 128, 28),
        QuantInfo("NVFP4", 144, 16, 16),
    ]
}
CODE_TO_NAME = {q.code: q.name for q in TYPES.values()}
# alternate codes used by the reference for its custom types
CODE_TO_NAME.update({200: "PQ2_0", 201: "PTQ1_0", 202: "NVFP4"})

# types with a device decoder (mmvq / dequant kernels)
DEVICE_TYPES = ("Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K",
                "IQ4_NL", "TQ2_0", "NVFP4")

IQ4NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113],
                        dtype=np.float32)
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def type_info(t: str | int) -> QuantInfo:
    if isinstance(t, (int, np.integer)):
        return TYPES[CODE_TO_NAME[int(t)]]
    return TYPES[t]


def row_bytes(t: str | int, k: int) -> int:
    q = type_info(t)
    if k % q.block:
        raise ValueError(f"{q.name}: row length {k} is not a multiple of the block size {q.block}")
    return k // q.block * q.nbytes


# ----------------------------------------------------------------------------------------------
# FP8 E4M3 (finite-only variant: max 448, 0x7F/0xFF are NaN)
# ----------------------------------------------------------------------------------------------
def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    b = b.astype(np.uint8)
    s = (b >> 7).astype(np.int32)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 7).astype(np.float32)
    sub = np.ldexp(m, -9)
    nor = np.ldexp(1.0 + m / 8.0, e - 7)
    v = np.where(e == 0, sub, nor).astype(np.float32)
    v = np.where((e == 15) & ((b & 7) == 7), 0.0, v)
    return np.where(s == 1, -v, v).astype(np.float32)


_E4M3_TABLE = None


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest encode, saturating at +-448."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        codes = np.arange(0, 0x7F, dtype=np.uint8)  # positive finite codes
        _E4M3_TABLE = (codes, e4m3_to_f32(codes))
    codes, vals = _E4M3_TABLE
    a = np.clip(np.abs(x.astype(np.float32)), 0, 448.0)
    idx = np.searchsorted(vals, a)
    idx = np.clip(idx, 1, len(vals) - 1)
    lo, hi = vals[idx - 1], vals[idx]
    pick = np.where((a - lo) <= (hi - a), idx - 1, idx)
    out = codes[pick].astype(np.uint8)
    return np.where(np.signbit(x), out | 0x80, out).astype(np.uint8)


# ----------------------------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------------------------
def _f16_bytes(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).view(np.uint8).reshape(*x.shape, 2)


def _rd_f16(raw: np.ndarray, off: int) -> np.ndarray:
    return raw[:, off:off + 2].copy().view(np.float16).astype(np.float32).reshape(-1)


def _scale_min_k4_unpack(sc12: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """sc12: [nb, 12] uint8 -> (scales [nb, 8], mins [nb, 8]) 6-bit each."""
    q = sc12.astype(np.int32)
    sc = np.empty((q.shape[0], 8), np.int32)
    mn = np.empty((q.shape[0], 8), np.int32)
    for j in range(4):
        sc[:, j] = q[:, j] & 63
        mn[:, j] = q[:, j + 4] & 63
    for j in range(4, 8):
        sc[:, j] = (q[:, j + 4] & 0xF) | ((q[:, j - 4] >> 6) << 4)
        mn[:, j] = (q[:, j + 4] >> 4) | ((q[:, j] >> 6) << 4)
    return sc, mn


def _scale_min_k4_pack(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    out = np.zeros((sc.shape[0], 12), np.uint8)
    sc = sc.astype(np.int32)
    mn = mn.astype(np.int32)
    for j in range(4):
        out[:, j] = (sc[:, j] & 63) | ((sc[:, j + 4] >> 4) << 6)
        out[:, j + 4] = (mn[:, j] & 63) | ((mn[:, j + 4] >> 4) << 6)
        out[:, j + 8] = (sc[:, j + 4] & 0xF) | ((mn[:, j + 4] & 0xF) << 4)
    return out


# ----------------------------------------------------------------------------------------------
# dequantize
# ----------------------------------------------------------------------------------------------
def dequantize(t: str | int, raw: np.ndarray | bytes | memoryview, n: int) -> np.ndarray:
    """Decode `n` elements from packed bytes; returns float32 [n]."""
    q = type_info(t)
    name = q.name
    buf = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw.view(np.uint8).reshape(-1)
    if name == "F32":
        return buf[: n * 4].view(np.float32).copy()
    if name == "F16":
        return buf[: n * 2].view(np.float16).astype(np.float32)
    if name == "BF16":
        u = buf[: n * 2].view(np.uint16).astype(np.uint32) << 16
        return u.view(np.float32)
    if n % q.block:
        raise ValueError(f"{name}: {n} elements is not a multiple of {q.block}")
    nb = n // q.block
    b = buf[: nb * q.nbytes].reshape(nb, q.nbytes)
    if name == "Q4_0":
        d = _rd_f16(b, 0)[:, None]
        qs = b[:, 2:18].astype(np.int32)
        lo, hi = (qs & 0xF) - 8, (qs >> 4) - 8
        return (np.concatenate([lo, hi], 1) * d).astype(np.float32).reshape(-1)
    if name == "Q4_1":
        d, m = _rd_f16(b, 0)[:, None], _rd_f16(b, 2)[:, None]
        qs = b[:, 4:20].astype(np.int32)
        return (np.concatenate([qs & 0xF, qs >> 4], 1) * d + m).astype(np.float32).reshape(-1)
    if name in ("Q5_0", "Q5_1"):
        off = 2 if name == "Q5_0" else 4
        d = _rd_f16(b, 0)[:, None]
        qh = b[:, off:off + 4].copy().view(np.uint32).astype(np.int64)  # [nb, 1]
        qs = b[:, off + 4:off + 20].astype(np.int64)
        j = np.arange(16)[None, :]
        h0 = ((qh >> j) << 4) & 0x10
        h1 = (qh >> (j + 12)) & 0x10
        lo, hi = (qs & 0xF) | h0, (qs >> 4) | h1
        v = np.concatenate([lo, hi], 1).astype(np.float32)
        if name == "Q5_0":
            return ((v - 16) * d).astype(np.float32).reshape(-1)
        m = _rd_f16(b, 2)[:, None]
        return (v * d + m).astype(np.float32).reshape(-1)
    if name == "Q8_0":
        d = _rd_f16(b, 0)[:, None]
        return (b[:, 2:34].view(np.int8).astype(np.float32) * d).reshape(-1)
    if name == "IQ4_NL":
        d = _rd_f16(b, 0)[:, None]
        qs = b[:, 2:18].astype(np.int32)
        v = np.concatenate([IQ4NL_VALUES[qs & 0xF], IQ4NL_VALUES[qs >> 4]], 1)
        return (v * d).astype(np.float32).reshape(-1)
    if name == "Q2_K":
        scales = b[:, 0:16].astype(np.int32)
        qs = b[:, 16:80].astype(np.int32).reshape(nb, 2, 32)
        d, dmin = _rd_f16(b, 80)[:, None], _rd_f16(b, 82)[:, None]
        out = np.empty((nb, 256), np.float32)
        for n_ in range(2):
            for j in range(4):
                for half in range(2):
                    sc = scales[:, n_ * 8 + j * 2 + half][:, None]
                    dl, ml = d * (sc & 0xF), dmin * (sc >> 4)
                    qv = (qs[:, n_, half * 16:half * 16 + 16] >> (2 * j)) & 3
                    o = n_ * 128 + j * 32 + half * 16
                    out[:, o:o + 16] = dl * qv - ml
        return out.reshape(-1)
    if name == "Q3_K":
        hm = b[:, 0:32].astype(np.int32)
        qs = b[:, 32:96].astype(np.int32).reshape(nb, 2, 32)
        sc12 = b[:, 96:108].copy()
        d_all = _rd_f16(b, 108)[:, None]
        aux = sc12.view(np.uint32).astype(np.uint64)  # [nb, 3]
        a0, a1, tmp = aux[:, 0], aux[:, 1], aux[:, 2]
        km1, km2 = np.uint64(0x03030303), np.uint64(0x0F0F0F0F)
        w = np.stack([
            (a0 & km2) | (((tmp >> np.uint64(0)) & km1) << np.uint64(4)),
            (a1 & km2) | (((tmp >> np.uint64(2)) & km1) << np.uint64(4)),
            ((a0 >> np.uint64(4)) & km2) | (((tmp >> np.uint64(4)) & km1) << np.uint64(4)),
            ((a1 >> np.uint64(4)) & km2) | (((tmp >> np.uint64(6)) & km1) << np.uint64(4)),
        ], 1).astype(np.uint32)
        scales = w.view(np.uint8).reshape(nb, 16).astype(np.int32) - 32
        out = np.empty((nb, 256), np.float32)
        for n_ in range(2):
            for j in range(4):
                bit = 1 << (n_ * 4 + j)
                for half in range(2):
                    dl = d_all * scales[:, n_ * 8 + j * 2 + half][:, None]
                    sl = slice(half * 16, half * 16 + 16)
                    qv = ((qs[:, n_, sl] >> (2 * j)) & 3) - np.where(hm[:, sl] & bit, 0, 4)
                    o = n_ * 128 + j * 32 + half * 16
                    out[:, o:o + 16] = dl * qv
        return out.reshape(-1)
    if name in ("Q4_K", "Q5_K"):
        d, dmin = _rd_f16(b, 0)[:, None], _rd_f16(b, 2)[:, None]
        sc, mn = _scale_min_k4_unpack(b[:, 4:16])
        out = np.empty((nb, 256), np.float32)
        if name == "Q4_K":
            qs = b[:, 16:144].astype(np.int32).reshape(nb, 4, 32)
            qh = None
        else:
            qh = b[:, 16:48].astype(np.int32)
            qs = b[:, 48:176].astype(np.int32).reshape(nb, 4, 32)
        for sub in range(8):
            qv = (qs[:, sub // 2, :] >> (4 * (sub & 1))) & 0xF
            if qh is not None:
                qv = qv + (((qh >> sub) & 1) << 4)
            out[:, sub * 32:(sub + 1) * 32] = d * sc[:, sub:sub + 1] * qv - dmin * mn[:, sub:sub + 1]
        return out.reshape(-1)
    if name == "Q6_K":
        ql = b[:, 0:128].astype(np.int32).reshape(nb, 2, 64)
        qh = b[:, 128:192].astype(np.int32).reshape(nb, 2, 32)
        sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(nb, 2, 8)
        d = _rd_f16(b, 208)[:, None]
        out = np.empty((nb, 256), np.float32)
        for half in range(2):
            for quarter in range(4):
                l_ = ql[:, half, (quarter & 1) * 32:(quarter & 1) * 32 + 32]
                nib = (l_ >> (4 * (quarter >> 1))) & 0xF
                hv = (qh[:, half, :] >> (2 * quarter)) & 3
                qv = (nib | (hv << 4)) - 32
                s = np.repeat(sc[:, half, quarter * 2:quarter * 2 + 2], 16, axis=1)
                o = half * 128 + quarter * 32
                out[:, o:o + 32] = d * s * qv
        return out.reshape(-1)
    if name == "TQ2_0":
        qs = b[:, 0:64].astype(np.int32).reshape(nb, 2, 32)
        d = _rd_f16(b, 64)[:, None]
        out = np.empty((nb, 256), np.float32)
        for j in range(2):
            for l_ in range(4):
                o = j * 128 + l_ * 32
                out[:, o:o + 32] = (((qs[:, j, :] >> (2 * l_)) & 3) - 1) * d
        return out.reshape(-1)
    if name == "NVFP4":
        s = e4m3_to_f32(b[:, 0])[:, None]
        qs = b[:, 1:9].astype(np.int32)
        lo, hi = qs & 0xF, qs >> 4
        def dec(nib):
            mag = E2M1_VALUES[nib & 7]
            return np.where(nib & 8, -mag, mag)
        return (np.concatenate([dec(lo), dec(hi)], 1) * s).astype(np.float32).reshape(-1)
    if name == "Q8_1":
        d = _rd_f16(b, 0)[:, None]
        return (b[:, 4:36].view(np.int8).astype(np.float32) * d).reshape(-1)
    raise NotImplementedError(f"no decoder for GGUF type {name} (parse-only)")


# ----------------------------------------------------------------------------------------------
# quantize
# ----------------------------------------------------------------------------------------------
def _nearest_int(x):
    return np.rint(x).astype(np.int32)


def quantize(t: str | int, x: np.ndarray) -> np.ndarray:
    """Encode float32 values (flattened; length must be a block multiple) -> uint8 bytes."""
    q = type_info(t)
    name = q.name
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if name == "F32":
        return x.view(np.uint8).copy()
    if name == "F16":
        return x.astype(np.float16).view(np.uint8).copy()
    if name == "BF16":
        u = x.view(np.uint32)
        r = ((u >> 16) & 1) + 0x7FFF  # round to nearest even
        return ((u + r) >> 16).astype(np.uint16).view(np.uint8).copy()
    if x.size % q.block:
        raise ValueError(f"{name}: {x.size} elements is not a multiple of {q.block}")
    nb = x.size // q.block
    xb = x.reshape(nb, q.block)
    out = np.zeros((nb, q.nbytes), np.uint8)

    def safe_inv(d):
        return np.where(d != 0, 1.0 / np.where(d != 0, d, 1.0), 0.0).astype(np.float32)

    if name in ("Q4_0", "Q5_0"):
        bits = 4 if name == "Q4_0" else 5
        half = 1 << (bits - 1)
        idx = np.abs(xb).argmax(1)
        mx = xb[np.arange(nb), idx]
        d = (mx / -half).astype(np.float16).astype(np.float32)
        qv = np.minimum((1 << bits) - 1, (xb * safe_inv(mx / -half)[:, None] + half + 0.5).astype(np.int32))
        qv = np.maximum(qv, 0)
        out[:, 0:2] = _f16_bytes(d)
        lo, hi = qv[:, :16], qv[:, 16:]
        if name == "Q4_0":
            out[:, 2:18] = (lo | (hi << 4)).astype(np.uint8)
        else:
            j = np.arange(16, dtype=np.int64)[None, :]
            qh = (((lo >> 4) & 1).astype(np.int64) << j).sum(1) | (((hi >> 4) & 1).astype(np.int64) << (j + 16)).sum(1)
            out[:, 2:6] = qh.astype(np.uint32).view(np.uint8).reshape(nb, 4)
            out[:, 6:22] = ((lo & 0xF) | ((hi & 0xF) << 4)).astype(np.uint8)
        return out.reshape(-1)
    if name in ("Q4_1", "Q5_1"):
        bits = 4 if name == "Q4_1" else 5
        levels = (1 << bits) - 1
        mn, mx = xb.min(1), xb.max(1)
        d = ((mx - mn) / levels).astype(np.float16).astype(np.float32)
        m16 = mn.astype(np.float16).astype(np.float32)
        qv = np.clip(_nearest_int((xb - m16[:, None]) * safe_inv(d)[:, None]), 0, levels)
        out[:, 0:2] = _f16_bytes(d)
        out[:, 2:4] = _f16_bytes(m16)
        lo, hi = qv[:, :16], qv[:, 16:]
        if name == "Q4_1":
            out[:, 4:20] = (lo | (hi << 4)).astype(np.uint8)
        else:
            j = np.arange(16, dtype=np.int64)[None, :]
            qh = (((lo >> 4) & 1).astype(np.int64) << j).sum(1) | (((hi >> 4) & 1).astype(np.int64) << (j + 16)).sum(1)
            out[:, 4:8] = qh.astype(np.uint32).view(np.uint8).reshape(nb, 4)
            out[:, 8:24] = ((lo & 0xF) | ((hi & 0xF) << 4)).astype(np.uint8)
        return out.reshape(-1)
    if name == "Q8_0":
        d = (np.abs(xb).max(1) / 127.0).astype(np.float16).astype(np.float32)
        qv = np.clip(_nearest_int(xb * safe_inv(d)[:, None]), -127, 127).astype(np.int8)
        out[:, 0:2] = _f16_bytes(d)
        out[:, 2:34] = qv.view(np.uint8)
        return out.reshape(-1)
    if name == "IQ4_NL":
        d = (np.abs(xb).max(1) / 127.0).astype(np.float16).astype(np.float32)
        y = xb * safe_inv(d)[:, None]
        qv = np.abs(y[:, :, None] - IQ4NL_VALUES[None, None, :]).argmin(2)
        out[:, 0:2] = _f16_bytes(d)
        out[:, 2:18] = (qv[:, :16] | (qv[:, 16:] << 4)).astype(np.uint8)
        return out.reshape(-1)
    if name in ("Q4_K", "Q5_K"):
        levels = 15 if name == "Q4_K" else 31
        sub = xb.reshape(nb, 8, 32)
        mn = np.minimum(sub.min(2), 0.0)
        mx = sub.max(2)
        scale = (mx - mn) / levels
        d = (scale.max(1) / 63.0).astype(np.float16).astype(np.float32)
        dmin = ((-mn).max(1) / 63.0).astype(np.float16).astype(np.float32)
        sc = np.clip(_nearest_int(scale * safe_inv(d)[:, None]), 0, 63)
        mq = np.clip(_nearest_int(-mn * safe_inv(dmin)[:, None]), 0, 63)
        eff_d = d[:, None] * sc
        eff_m = dmin[:, None] * mq
        qv = np.clip(_nearest_int((sub + eff_m[:, :, None]) * safe_inv(eff_d)[:, :, None]), 0, levels)
        out[:, 0:2] = _f16_bytes(d)
        out[:, 2:4] = _f16_bytes(dmin)
        out[:, 4:16] = _scale_min_k4_pack(sc, mq)
        lo4 = qv & 0xF
        packed = (lo4[:, 0::2, :] | (lo4[:, 1::2, :] << 4)).astype(np.uint8).reshape(nb, 128)
        if name == "Q4_K":
            out[:, 16:144] = packed
        else:
            hb = (qv >> 4) & 1  # [nb, 8, 32]
            qh = np.zeros((nb, 32), np.int32)
            for s_ in range(8):
                qh |= hb[:, s_, :] << s_
            out[:, 16:48] = qh.astype(np.uint8)
            out[:, 48:176] = packed
        return out.reshape(-1)
    if name == "Q6_K":
        sub = xb.reshape(nb, 16, 16)
        amax = np.abs(sub).max(2)
        scale = amax / 31.0
        d = (scale.max(1) / 127.0).astype(np.float16).astype(np.float32)
        sc = np.clip(_nearest_int(scale * safe_inv(d)[:, None]), -128, 127)
        eff = d[:, None] * sc
        qv = np.clip(_nearest_int(sub * safe_inv(eff)[:, :, None]), -32, 31) + 32
        qv = qv.reshape(nb, 2, 4, 32)  # [half][quarter][l]
        ql = np.zeros((nb, 2, 64), np.int32)
        qh = np.zeros((nb, 2, 32), np.int32)
        for quarter in range(4):
            v = qv[:, :, quarter, :]
            sl = slice((quarter & 1) * 32, (quarter & 1) * 32 + 32)
            ql[:, :, sl] |= (v & 0xF) << (4 * (quarter >> 1))
            qh |= ((v >> 4) & 3) << (2 * quarter)
        out[:, 0:128] = ql.reshape(nb, 128).astype(np.uint8)
        out[:, 128:192] = qh.reshape(nb, 64).astype(np.uint8)
        out[:, 192:208] = sc.astype(np.int8).view(np.uint8)
        out[:, 208:210] = _f16_bytes(d)
        return out.reshape(-1)
    if name == "Q2_K":
        sub = xb.reshape(nb, 16, 16)
        mn = np.minimum(sub.min(2), 0.0)
        mx = sub.max(2)
        scale = (mx - mn) / 3.0
        d = (scale.max(1) / 15.0).astype(np.float16).astype(np.float32)
        dmin = ((-mn).max(1) / 15.0).astype(np.float16).astype(np.float32)
        sc = np.clip(_nearest_int(scale * safe_inv(d)[:, None]), 0, 15)
        mq = np.clip(_nearest_int(-mn * safe_inv(dmin)[:, None]), 0, 15)
        eff_d, eff_m = d[:, None] * sc, dmin[:, None] * mq
        qv = np.clip(_nearest_int((sub + eff_m[:, :, None]) * safe_inv(eff_d)[:, :, None]), 0, 3)
        # sub-block index = n*8 + j*2 + half ; element l in 0..15
        qv = qv.reshape(nb, 2, 4, 2, 16)
        qs = np.zeros((nb, 2, 32), np.int32)
        for j in range(4):
            for half in range(2):
                qs[:, :, half * 16:half * 16 + 16] |= qv[:, :, j, half, :] << (2 * j)
        out[:, 0:16] = (sc | (mq << 4)).astype(np.uint8)
        out[:, 16:80] = qs.reshape(nb, 64).astype(np.uint8)
        out[:, 80:82] = _f16_bytes(d)
        out[:, 82:84] = _f16_bytes(dmin)
        return out.reshape(-1)
    if name == "Q3_K":
        sub = xb.reshape(nb, 16, 16)
        amax_i = np.abs(sub).argmax(2)
        mxv = np.take_along_axis(sub, amax_i[:, :, None], 2)[:, :, 0]
        scale = mxv / -4.0
        d = (np.abs(scale).max(1) / 31.0).astype(np.float16).astype(np.float32)
        sc = np.clip(_nearest_int(scale * safe_inv(d)[:, None]), -32, 31)
        eff = d[:, None] * sc
        qv = np.clip(_nearest_int(sub * safe_inv(eff)[:, :, None]), -4, 3) + 4  # 0..7
        qv = qv.reshape(nb, 2, 4, 2, 16)
        qs = np.zeros((nb, 2, 32), np.int32)
        hm = np.zeros((nb, 32), np.int32)
        for n_ in range(2):
            for j in range(4):
                for half in range(2):
                    v = qv[:, n_, j, half, :]
                    sl = slice(half * 16, half * 16 + 16)
                    qs[:, n_, sl] |= (v & 3) << (2 * j)
                    hm[:, sl] |= ((v >> 2) & 1) << (n_ * 4 + j)
        # pack 16 6-bit (value+32) scales into 12 bytes (inverse of the kmask unpack)
        s6 = (sc + 32).astype(np.uint32)  # 0..63
        lo4, hi2 = s6 & 0xF, s6 >> 4
        sc12 = np.zeros((nb, 12), np.uint32)
        for i in range(4):
            sc12[:, i] = lo4[:, i] | (lo4[:, 8 + i] << 4)
            sc12[:, 4 + i] = lo4[:, 4 + i] | (lo4[:, 12 + i] << 4)
            sc12[:, 8 + i] = hi2[:, i] | (hi2[:, 4 + i] << 2) | (hi2[:, 8 + i] << 4) | (hi2[:, 12 + i] << 6)
        out[:, 0:32] = hm.astype(np.uint8)
        out[:, 32:96] = qs.reshape(nb, 64).astype(np.uint8)
        out[:, 96:108] = sc12.astype(np.uint8)
        out[:, 108:110] = _f16_bytes(d)
        return out.reshape(-1)
    if name == "TQ2_0":
        d = np.abs(xb).max(1).astype(np.float16).astype(np.float32)
        qv = np.clip(_nearest_int(xb * safe_inv(d)[:, None]), -1, 1) + 1
        qv = qv.reshape(nb, 2, 4, 32)
        qs = np.zeros((nb, 2, 32), np.int32)
        for l_ in range(4):
            qs |= qv[:, :, l_, :] << (2 * l_)
        out[:, 0:64] = qs.reshape(nb, 64).astype(np.uint8)
        out[:, 64:66] = _f16_bytes(d)
        return out.reshape(-1)
    if name == "NVFP4":
        amax = np.abs(xb).max(1)
        raw_scale = np.where(amax > 0, amax / 6.0, 1.0)
        sb = f32_to_e4m3(raw_scale)
        s = e4m3_to_f32(sb)
        y = xb * safe_inv(s)[:, None]
        mag = np.abs(np.abs(y)[:, :, None] - E2M1_VALUES[None, None, :]).argmin(2)
        nib = (mag | np.where(y < 0, 8, 0)).astype(np.int32)
        out[:, 0] = sb
        out[:, 1:9] = (nib[:, :8] | (nib[:, 8:] << 4)).astype(np.uint8)
        return out.reshape(-1)
    raise NotImplementedError(f"no encoder for GGUF type {name}")


def quantize_2d(t: str | int, w: np.ndarray) -> np.ndarray:
    """Quantize a [rows, K] matrix row by row -> uint8 [rows, row_bytes]."""
    rows, k = w.shape
    rb = row_bytes(t, k)
    return quantize(t, w).reshape(rows, rb)


def dequantize_2d(t: str | int, raw: np.ndarray, rows: int, k: int) -> np.ndarray:
    return dequantize(t, raw, rows * k).reshape(rows, k)
