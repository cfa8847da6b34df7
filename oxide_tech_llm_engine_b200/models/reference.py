"""PyTorch fp32 CPU oracle of the decoder (dense Llama family and Mixtral-style MoE).

Restates the reference's CPU forward (oxide-models/src/llama3.rs:3295-3733): embed -> per layer
[RMSNorm -> QKV -> bias -> QK-norm -> RoPE -> KV append -> causal GQA attention -> O-proj ->
residual -> RMSNorm -> gate/up -> SwiGLU/GeGLU -> down -> residual] -> final norm -> LM head ->
softcap. MoE routing = top-k over router logits with a softmax over the selected logits
(oxide-engine/src/moe_gemm.rs:104-129). Every device kernel and the whole engine are tested
against this module.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .config import ModelConfig
from .rope import inv_freq_table
from .weights import WeightSource


class ReferenceModel:
    def __init__(self, cfg: ModelConfig, src: WeightSource, dtype=torch.float32):
        self.cfg = cfg
        self.dtype = dtype
        t = lambda n: torch.from_numpy(np.ascontiguousarray(src.f32(n))).to(dtype)
        self.embed = t("token_embd.weight")
        self.out_norm = t("output_norm.weight")
        self.lm_head = t("output.weight") if src.has("output.weight") else self.embed
        self.layers = []
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            L = {k: t(p + k + ".weight") for k in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_output",
                                                    "ffn_norm")}
            for b in ("attn_q", "attn_k", "attn_v"):
                L[b + ".bias"] = t(p + b + ".bias") if src.has(p + b + ".bias") else None
            for nrm in ("attn_q_norm", "attn_k_norm"):
                L[nrm] = t(p + nrm + ".weight") if src.has(p + nrm + ".weight") else None
            if cfg.is_moe:
                for k in ("ffn_gate_inp", "ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
                    L[k] = t(p + k + ".weight")
            else:
                for k in ("ffn_gate", "ffn_up", "ffn_down"):
                    L[k] = t(p + k + ".weight")
            self.layers.append(L)
        inv, self.mscale = inv_freq_table(cfg)
        self.inv_freq = torch.from_numpy(inv)
        self.reset()

    def reset(self):
        self.k_cache = [None] * self.cfg.n_layers
        self.v_cache = [None] * self.cfg.n_layers
        self.pos = 0

    # ------------------------------------------------------------------ pieces
    def _norm(self, x, w, eps=None):
        eps = self.cfg.rms_eps if eps is None else eps
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w + self.cfg.norm_weight_offset)

    def _rope(self, x, pos):
        half = x.shape[-1] // 2
        ang = pos.to(torch.float32)[:, None] * self.inv_freq[None, :]
        cs, sn = (ang.cos() * self.mscale)[:, None, :].to(x.dtype), (ang.sin() * self.mscale)[:, None, :].to(x.dtype)
        a, b = x[..., :half], x[..., half:]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1)

    def _act(self, g):
        if self.cfg.act == "gelu_tanh":
            return torch.nn.functional.gelu(g, approximate="tanh")
        return torch.nn.functional.silu(g)

    def _ffn(self, L, x):
        cfg = self.cfg
        if not cfg.is_moe:
            return (self._act(x @ L["ffn_gate"].T) * (x @ L["ffn_up"].T)) @ L["ffn_down"].T
        logits = x @ L["ffn_gate_inp"].T
        tv, ti = logits.topk(cfg.n_experts_used, dim=-1)
        w = torch.softmax(tv, -1) * cfg.routed_scale
        y = torch.zeros_like(x)
        for e in range(cfg.n_experts):
            sel = (ti == e)
            rows = sel.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            xe = x[rows]
            h = (self._act(xe @ L["ffn_gate_exps"][e].T) * (xe @ L["ffn_up_exps"][e].T)) @ L["ffn_down_exps"][e].T
            y[rows] += h * (w[rows] * sel[rows]).sum(-1, keepdim=True)
        return y

    # ------------------------------------------------------------------ forward
    @torch.no_grad()
    def forward(self, tokens, *, all_logits: bool = False) -> torch.Tensor:
        """Appends `tokens` to the sequence and returns logits of the last (or of every) position."""
        cfg = self.cfg
        tok = torch.as_tensor(np.asarray(tokens), dtype=torch.long)
        T = tok.numel()
        pos = torch.arange(self.pos, self.pos + T)
        x = self.embed[tok] * cfg.emb_scale
        for li, L in enumerate(self.layers):
            h = self._norm(x, L["attn_norm"])
            q = h @ L["attn_q"].T
            k = h @ L["attn_k"].T
            v = h @ L["attn_v"].T
            if L["attn_q.bias"] is not None:
                q, k, v = q + L["attn_q.bias"], k + L["attn_k.bias"], v + L["attn_v.bias"]
            q = q.view(T, cfg.n_heads, cfg.head_dim)
            k = k.view(T, cfg.n_kv_heads, cfg.head_dim)
            v = v.view(T, cfg.n_kv_heads, cfg.head_dim)
            if L["attn_q_norm"] is not None:
                q = self._norm(q, L["attn_q_norm"], 1e-6)
                k = self._norm(k, L["attn_k_norm"], 1e-6)
            q, k = self._rope(q, pos), self._rope(k, pos)
            self.k_cache[li] = k if self.k_cache[li] is None else torch.cat([self.k_cache[li], k], 0)
            self.v_cache[li] = v if self.v_cache[li] is None else torch.cat([self.v_cache[li], v], 0)
            kk = self.k_cache[li].repeat_interleave(cfg.n_heads // cfg.n_kv_heads, dim=1)
            vv = self.v_cache[li].repeat_interleave(cfg.n_heads // cfg.n_kv_heads, dim=1)
            s = torch.einsum("qhd,khd->hqk", q, kk) / (cfg.head_dim ** 0.5)
            kpos = torch.arange(kk.shape[0])
            mask = kpos[None, :] <= pos[:, None]
            if cfg.sliding_window > 0:
                mask &= kpos[None, :] > (pos[:, None] - cfg.sliding_window)
            s = s.masked_fill(~mask[None], float("-inf"))
            a = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), vv).reshape(T, cfg.q_dim)
            x = x + a @ L["attn_output"].T
            x = x + self._ffn(L, self._norm(x, L["ffn_norm"]))
        self.pos += T
        xo = x if all_logits else x[-1:]
        logits = self._norm(xo, self.out_norm) @ self.lm_head.T
        if cfg.logit_softcap > 0:
            logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
        return logits

    @torch.no_grad()
    def generate_greedy(self, prompt, n_new: int, stop_ids: Optional[set] = None) -> list[int]:
        self.reset()
        logits = self.forward(prompt)
        out = []
        for _ in range(n_new):
            t = int(logits[-1].argmax())
            out.append(t)
            if stop_ids and t in stop_ids:
                break
            logits = self.forward([t])
        return out
