"""RoPE frequency tables: default, linear, Llama-3 and YaRN scaling of `inv_freq`.

One definition shared by the CPU oracle and the device kernel (the kernel receives the table;
rotation is half-split: pairs (x[i], x[i + d/2])). Reference parity: RopeScalingEngine
(oxide-models/src/rope.rs:11-143, rotation rope.rs:162-179). The reference's CUDA path uses a
different YaRN ramp than its CPU path (vec_ops_activations.cu:140-154); here both sides use this
module.
"""
from __future__ import annotations

import math

import numpy as np

from .config import ModelConfig


def inv_freq_table(cfg: ModelConfig) -> tuple[np.ndarray, float]:
    """Returns (inv_freq [head_dim/2] float32, attention magnitude scale)."""
    d = cfg.head_dim
    i = np.arange(0, d, 2, dtype=np.float64)
    inv = 1.0 / (cfg.rope_theta ** (i / d))
    mscale = 1.0
    kind = cfg.rope_scaling
    if kind == "linear" and cfg.rope_factor > 0:
        inv = inv / cfg.rope_factor
    elif kind == "llama3":
        factor = cfg.rope_factor
        lo, hi = cfg.rope_low_freq_factor, cfg.rope_high_freq_factor
        orig = float(cfg.rope_orig_ctx)
        wavelen = 2.0 * math.pi / inv
        low_wl, high_wl = orig / lo, orig / hi
        smooth = (orig / wavelen - lo) / (hi - lo)
        scaled = np.where(wavelen > low_wl, inv / factor, inv)
        mid = (wavelen <= low_wl) & (wavelen >= high_wl)
        scaled = np.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
        inv = scaled
    elif kind == "yarn":
        factor = cfg.rope_factor
        orig = float(cfg.rope_orig_ctx)
        beta_fast, beta_slow = 32.0, 1.0

        def corr_dim(n_rot):
            return d * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(cfg.rope_theta))

        low = max(math.floor(corr_dim(beta_fast)), 0)
        high = min(math.ceil(corr_dim(beta_slow)), d // 2 - 1)
        ramp = np.clip((np.arange(d // 2, dtype=np.float64) - low) / max(high - low, 1e-3), 0, 1)
        extrap_mask = 1.0 - ramp
        inv = inv / factor * (1 - extrap_mask) + inv * extrap_mask
        mscale = 0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0
    return inv.astype(np.float32), float(mscale)


def apply_rope_np(x: np.ndarray, pos: np.ndarray, inv_freq: np.ndarray, mscale: float = 1.0) -> np.ndarray:
    """x: [T, H, D]; pos: [T]. Half-split rotation."""
    half = x.shape[-1] // 2
    ang = pos.astype(np.float32)[:, None] * inv_freq[None, :]
    cs, sn = np.cos(ang)[:, None, :] * mscale, np.sin(ang)[:, None, :] * mscale
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cs - b * sn, b * cs + a * sn], -1)
