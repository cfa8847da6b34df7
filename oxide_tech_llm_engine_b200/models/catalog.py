"""Model catalog: name -> shape specification with fuzzy lookup.

A compact table of the decoder families the engine serves (the reference ships 142 entries across
modalities, oxide-models/src/registry.rs:478-514; this table keeps the text decoders that map onto
`ModelConfig`). `lookup("Meta-Llama-3-8B-Instruct-Q4_K_M.gguf")` finds `llama3-8b`; SafeTensors
checkpoints without config.json and `/v1/models` use it.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Optional

from .config import ModelConfig, PRESETS


@dataclass(frozen=True)
class ModelSpecification:
    key: str
    family: str
    modality: str
    arch_type: str
    default_quant: str
    config: ModelConfig


def _c(name, **kw) -> ModelConfig:
    return ModelConfig(name=name, **kw)


_EXTRA = {
    "llama2-7b": _c("llama2-7b", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=32, head_dim=128, ffn_dim=11008,
                    vocab_size=32000, max_ctx=4096),
    "llama3.1-8b": _c("llama3.1-8b", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                      ffn_dim=14336, vocab_size=128256, rope_theta=500000.0, rope_scaling="llama3", rope_factor=8.0,
                      max_ctx=131072, bos_id=128000, eos_id=128001),
    "qwen3-8b": _c("qwen3-8b", arch="qwen3", n_layers=36, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                   ffn_dim=12288, vocab_size=151936, rope_theta=1000000.0, rms_eps=1e-6, qk_norm=True,
                   max_ctx=40960, bos_id=151643, eos_id=151645),
    "qwen2.5-7b": _c("qwen2.5-7b", arch="qwen2", n_layers=28, d_model=3584, n_heads=28, n_kv_heads=4, head_dim=128,
                     ffn_dim=18944, vocab_size=152064, rope_theta=1000000.0, rms_eps=1e-6, attn_bias=True,
                     max_ctx=32768, bos_id=151643, eos_id=151645),
    "mistral-7b": _c("mistral-7b", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=14336,
                     vocab_size=32000, sliding_window=4096, max_ctx=32768),
    "gemma2-9b": _c("gemma2-9b", arch="gemma2", n_layers=42, d_model=3584, n_heads=16, n_kv_heads=8, head_dim=256,
                    ffn_dim=14336, vocab_size=256000, norm_weight_offset=1.0, emb_scale=3584 ** 0.5, act="gelu_tanh",
                    logit_softcap=30.0, tie_embeddings=True, max_ctx=8192),
    "mixtral-8x22b": _c("mixtral-8x22b", arch="mixtral", n_layers=56, d_model=6144, n_heads=48, n_kv_heads=8,
                        head_dim=128, ffn_dim=16384, vocab_size=32768, rope_theta=1000000.0, n_experts=8,
                        n_experts_used=2, max_ctx=65536),
    "deepseek-r1-qwen3-8b": _c("deepseek-r1-qwen3-8b", arch="qwen3", n_layers=36, d_model=4096, n_heads=32,
                               n_kv_heads=8, head_dim=128, ffn_dim=12288, vocab_size=151936, rope_theta=1000000.0,
                               rms_eps=1e-6, qk_norm=True, max_ctx=131072, bos_id=151643, eos_id=151645),
}


def catalog() -> dict[str, ModelSpecification]:
    out = {}
    for key, cfg in {**PRESETS, **_EXTRA}.items():
        fam = re.split(r"[-0-9.]", key)[0] or key
        out[key] = ModelSpecification(key, fam, "text", "moe-decoder" if cfg.is_moe else "dense-decoder",
                                      "Q4_K" if cfg.n_params() > 2e9 else "Q8_0", cfg)
    return out


def _norm(s: str) -> str:
    return re.sub(r"[^a-z0-9]", "", s.lower())


def lookup(name: str) -> Optional[ModelSpecification]:
    """Exact key, else the most specific catalog key whose parts all occur, in order, in the name
    (`Meta-Llama-3-8B-Instruct-Q4_K_M.gguf` -> `llama3-8b`)."""
    cat = catalog()
    if name in cat:
        return cat[name]
    n = _norm(name.rsplit("/", 1)[-1])
    best, best_len = None, 0
    for key, spec in cat.items():
        parts = [p for p in re.split(r"[^a-z0-9.]+", key.lower()) if p]
        pos, ok = 0, True
        for part in parts:
            i = n.find(_norm(part), pos)
            if i < 0:
                ok = False
                break
            pos = i + len(_norm(part))
        size = sum(len(_norm(p)) for p in parts)
        if ok and size > best_len:
            best, best_len = spec, size
    return best
