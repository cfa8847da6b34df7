"""Ulysses-style context parallelism for prefill: swap the sharded axis from sequence to heads with an
all-to-all, run ordinary causal attention over the FULL sequence on `heads / cp` heads, swap back.

Compared with the ring (parallel/ring_attention.py) this moves Q, K, V and O once each (4 all-to-alls of
`T_local x H x D`) instead of circulating K/V `cp - 1` times, and needs `heads % cp == 0` and
`kv_heads % cp == 0`. The transport is `torch.distributed.all_to_all_single` (NCCL); process groups
without it (gloo) fall back to an all-gather and a local slice, which moves more bytes but keeps the
semantics testable on CPU ranks. The reference names neither variant (its context parallelism is the
three integers of `RingAttentionStep`, oxide-engine/src/distributed.rs:109-142).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from .ring_attention import partial_attention


def _seq_to_heads(x: torch.Tensor, cp: int, rank: int, group) -> torch.Tensor:
    """[T_local, H, D] on every rank -> [cp * T_local, H / cp, D] (all tokens, this rank's heads)."""
    t, h, d = x.shape
    hl = h // cp
    send = x.reshape(t, cp, hl, d).permute(1, 0, 2, 3).contiguous()      # [cp, T_local, hl, D]
    recv = torch.empty_like(send)
    try:
        dist.all_to_all_single(recv.view(cp * t, hl * d), send.view(cp * t, hl * d), group=group)
    except (RuntimeError, NotImplementedError):
        full = [torch.empty_like(send) for _ in range(cp)]
        dist.all_gather(full, send, group=group)
        recv = torch.stack([full[src][rank] for src in range(cp)])
    return recv.reshape(cp * t, hl, d)


def _heads_to_seq(x: torch.Tensor, cp: int, rank: int, group) -> torch.Tensor:
    """Inverse of `_seq_to_heads`: [cp * T_local, H / cp, D] -> [T_local, H, D]."""
    tt, hl, d = x.shape
    t = tt // cp
    send = x.reshape(cp, t, hl, d).contiguous()                          # chunk j goes to rank j
    recv = torch.empty_like(send)
    try:
        dist.all_to_all_single(recv.view(cp * t, hl * d), send.view(cp * t, hl * d), group=group)
    except (RuntimeError, NotImplementedError):
        full = [torch.empty_like(send) for _ in range(cp)]
        dist.all_gather(full, send, group=group)
        recv = torch.stack([full[src][rank] for src in range(cp)])
    return recv.permute(1, 0, 2, 3).reshape(t, cp * hl, d)               # heads of source j at [j*hl, (j+1)*hl)


def ulysses_attention(q, k, v, *, rank: int, cp: int, group=None, scale: Optional[float] = None):
    """q [T_local, H, D], k/v [T_local, Hkv, D]: the rank holds the contiguous token chunk
    [rank * T_local, (rank + 1) * T_local). Returns the causal attention output for those tokens."""
    if q.shape[1] % cp or k.shape[1] % cp:
        raise ValueError("Ulysses needs heads and kv heads divisible by the context-parallel size")
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    qh = _seq_to_heads(q, cp, rank, group)
    kh = _seq_to_heads(k, cp, rank, group)
    vh = _seq_to_heads(v, cp, rank, group)
    pos = torch.arange(qh.shape[0], device=q.device)
    o, _ = partial_attention(qh, kh, vh, pos, pos, scale)
    return _heads_to_seq(o.to(q.dtype), cp, rank, group)
