"""CPU backend: the fp32 oracle's math over the same paged KV layout and step plans as the GPU
model, so the scheduler, block manager, radix cache, server and CLI run end to end without a GPU.

Reference parity: Llama3Model::forward_step_paged / forward_layer_paged over PagedKvArena
(oxide-models/src/llama3.rs:3739-3944) -- the path the reference's HTTP server actually runs
(oxide-cli/src/lib.rs:1864-1884).
"""
from __future__ import annotations

import numpy as np
import torch

from .config import ModelConfig
from .reference import ReferenceModel
from .weights import WeightSource


class CpuPagedModel(ReferenceModel):
    def __init__(self, cfg: ModelConfig, src: WeightSource, num_blocks: int):
        super().__init__(cfg, src)
        self.num_blocks = num_blocks
        shape = (num_blocks, cfg.n_kv_heads, 16, cfg.head_dim)
        self.pk = [torch.zeros(shape) for _ in range(cfg.n_layers)]
        self.pv = [torch.zeros(shape) for _ in range(cfg.n_layers)]
        self.logits = None

    def copy_blocks(self, src: np.ndarray, dst: np.ndarray) -> None:
        for s, d in zip(src.tolist(), dst.tolist()):
            for li in range(self.cfg.n_layers):
                self.pk[li][d] = self.pk[li][s]
                self.pv[li][d] = self.pv[li][s]

    def _gather(self, cache: torch.Tensor, table: np.ndarray, n_tok: int) -> torch.Tensor:
        nb = (n_tok + 15) // 16
        blk = cache[torch.as_tensor(table[:nb].astype(np.int64))]  # [nb, hkv, 16, D]
        return blk.permute(0, 2, 1, 3).reshape(nb * 16, cache.shape[1], cache.shape[3])[:n_tok]

    def _attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        g = cfg.n_heads // cfg.n_kv_heads
        kk, vv = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, kk) / (cfg.head_dim ** 0.5)
        kpos = torch.arange(kk.shape[0])
        mask = kpos[None, :] <= q_pos[:, None]
        if cfg.sliding_window > 0:
            mask &= kpos[None, :] > (q_pos[:, None] - cfg.sliding_window)
        s = s.masked_fill(~mask[None], float("-inf"))
        return torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv)

    @torch.no_grad()
    def forward_plan(self, plan, layer_range=None, x_in=None, return_hidden: bool = False) -> torch.Tensor:
        """Runs the step; with `layer_range` only those layers (pipeline stage): `x_in` is the hidden
        state received from the previous stage, `return_hidden` skips the head."""
        cfg = self.cfg
        tok = torch.as_tensor(plan.token_ids.astype(np.int64))
        pos = torch.as_tensor(plan.positions.astype(np.int64))
        slots = plan.slot_mapping
        T = tok.numel()
        nd, npf, W = plan.n_decode, plan.n_prefill, plan.max_blocks
        dbt = plan.decode_block_tables.reshape(nd, W) if nd else None
        pbt = plan.prefill_block_tables.reshape(npf, W) if npf else None
        blk = torch.as_tensor(slots // 16)
        off = torch.as_tensor(slots % 16)
        x = self.embed[tok] * cfg.emb_scale if x_in is None else x_in
        lo, hi = layer_range if layer_range is not None else (0, cfg.n_layers)
        for li in range(lo, hi):
            L = self.layers[li]
            h = self._norm(x, L["attn_norm"])
            q, k, v = h @ L["attn_q"].T, h @ L["attn_k"].T, h @ L["attn_v"].T
            if L["attn_q.bias"] is not None:
                q, k, v = q + L["attn_q.bias"], k + L["attn_k.bias"], v + L["attn_v.bias"]
            q = q.view(T, cfg.n_heads, cfg.head_dim)
            k = k.view(T, cfg.n_kv_heads, cfg.head_dim)
            v = v.view(T, cfg.n_kv_heads, cfg.head_dim)
            if L["attn_q_norm"] is not None:
                q, k = self._norm(q, L["attn_q_norm"], 1e-6), self._norm(k, L["attn_k_norm"], 1e-6)
            q, k = self._rope(q, pos), self._rope(k, pos)
            self.pk[li][blk, :, off] = k
            self.pv[li][blk, :, off] = v
            a = torch.zeros(T, cfg.n_heads, cfg.head_dim)
            for i in range(nd):
                n_ctx = int(plan.decode_seq_lens[i])
                kk = self._gather(self.pk[li], dbt[i], n_ctx)
                vv = self._gather(self.pv[li], dbt[i], n_ctx)
                a[i:i + 1] = self._attend(q[i:i + 1], kk, vv, pos[i:i + 1])
            for s_ in range(npf):
                r0, ql, cl = int(plan.q_start[s_]), int(plan.q_lens[s_]), int(plan.ctx_lens[s_])
                kk = self._gather(self.pk[li], pbt[s_], cl)
                vv = self._gather(self.pv[li], pbt[s_], cl)
                a[r0:r0 + ql] = self._attend(q[r0:r0 + ql], kk, vv, pos[r0:r0 + ql])
            x = x + a.reshape(T, cfg.q_dim) @ L["attn_output"].T
            x = x + self._ffn(L, self._norm(x, L["ffn_norm"]))
        if return_hidden:
            return x
        rows = torch.as_tensor(plan.logit_rows.astype(np.int64))
        logits = self._norm(x[rows], self.out_norm) @ self.lm_head.T
        if cfg.logit_softcap > 0:
            logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
        self.logits = logits
        return logits
