"""Context-parallel causal attention: a ring over KV chunks with log-sum-exp merging.

Every rank keeps the queries of its own sequence chunk; KV chunks travel around the ring
(rank r sends to r-1 and receives from r+1, the peers of the reference's RingAttentionStep,
oxide-engine/src/distributed.rs:109-142), and partial results are merged with the same
(max, sum) rule the split-KV decode kernel uses. Zig-zag chunk placement balances the causal
triangle: with 2*cp chunks, rank r owns chunks r and 2*cp-1-r. The transport is
`torch.distributed` send/recv (NCCL on GPUs, gloo on CPU ranks); on a GPU the per-chunk partial
attention runs on the device. The reference has only the peer arithmetic, no attention maths.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist


def zigzag_chunks(cp: int, rank: int) -> tuple[int, int]:
    return rank, 2 * cp - 1 - rank


def partial_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor,
                      k_pos: torch.Tensor, scale: float):
    """Causal attention of q against one KV chunk. q [Tq,H,D], k/v [Tk,Hkv,D].
    Returns (o [Tq,H,D] normalised within the chunk, lse [Tq,H])."""
    g = q.shape[1] // k.shape[1]
    kk, vv = k.float().repeat_interleave(g, 1), v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    mask = k_pos[None, :] <= q_pos[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, -1)                       # [H, Tq]
    p = torch.exp(s - lse.clamp_min(-1e30)[..., None])
    p = torch.where(torch.isfinite(lse)[..., None], p, torch.zeros_like(p))
    o = torch.einsum("hqk,khd->qhd", p, vv)
    return o, lse.transpose(0, 1)


def merge(o1, lse1, o2, lse2):
    """Combine two partial results that attended to disjoint key sets."""
    m = torch.maximum(lse1, lse2)
    m_safe = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    w1, w2 = torch.exp(lse1 - m_safe), torch.exp(lse2 - m_safe)
    w1 = torch.where(torch.isfinite(lse1), w1, torch.zeros_like(w1))
    w2 = torch.where(torch.isfinite(lse2), w2, torch.zeros_like(w2))
    tot = (w1 + w2).clamp_min(1e-38)
    o = (o1 * w1[..., None] + o2 * w2[..., None]) / tot[..., None]
    return o, m_safe + torch.log(tot)


def ring_attention(q, k, v, q_pos, k_pos, *, rank: int, cp: int, group=None, scale: Optional[float] = None):
    """q/k/v and their absolute positions are this rank's local chunks; returns the attention
    output of the local queries over the keys of ALL ranks (causal by position)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    o, lse = partial_attention(q, k, v, q_pos, k_pos, scale)
    send_to, recv_from = (rank - 1) % cp, (rank + 1) % cp
    cur = [k.contiguous(), v.contiguous(), k_pos.contiguous()]
    for _ in range(cp - 1):
        nxt = [torch.empty_like(t) for t in cur]
        ops = []
        for t_send, t_recv in zip(cur, nxt):
            ops.append(dist.P2POp(dist.isend, t_send, send_to, group))
            ops.append(dist.P2POp(dist.irecv, t_recv, recv_from, group))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        cur = nxt
        o2, lse2 = partial_attention(q, cur[0], cur[1], q_pos, cur[2], scale)
        o, lse = merge(o, lse, o2, lse2)
    return o
