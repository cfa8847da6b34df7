"""Model hyper-parameters, named presets and GGUF-metadata -> config mapping.

Reference parity: Llama3Config::from_gguf (oxide-models/src/llama3.rs:165-312) reads
`{arch}.embedding_length/block_count/attention.head_count(_kv)/context_length/rope.freq_base/
attention.layer_norm_rms_epsilon/rope.scaling.*/attention.sliding_window/final_logit_softcapping`,
derives head_dim from `blk.0.attn_q.weight`, the FFN width from `blk.0.ffn_gate.weight` and the
vocabulary from `token_embd.weight`; tiny_test_config (llama3.rs:66-91). MoE keys
(`{arch}.expert_count`, `{arch}.expert_used_count`) are an addition: the reference loads no experts.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Any


@dataclass
class ModelConfig:
    name: str = "llama"
    arch: str = "llama"
    n_layers: int = 2
    d_model: int = 128
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 32
    ffn_dim: int = 256
    vocab_size: int = 1024
    max_ctx: int = 8192
    rope_theta: float = 10000.0
    rope_scaling: str = "none"  # none | linear | llama3 | yarn
    rope_factor: float = 1.0
    rope_orig_ctx: int = 8192
    rope_low_freq_factor: float = 1.0
    rope_high_freq_factor: float = 4.0
    rms_eps: float = 1e-5
    norm_weight_offset: float = 0.0  # Gemma stores (w - 1)
    emb_scale: float = 1.0  # Gemma multiplies embeddings by sqrt(d_model)
    act: str = "silu"  # silu | gelu_tanh
    qk_norm: bool = False
    attn_bias: bool = False
    sliding_window: int = 0
    logit_softcap: float = 0.0
    tie_embeddings: bool = False
    # mixture of experts (0 experts = dense FFN)
    n_experts: int = 0
    n_experts_used: int = 0
    routed_scale: float = 1.0
    bos_id: int = 1
    eos_id: int = 2

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    def n_params(self) -> int:
        per_layer = self.d_model * (self.q_dim + 2 * self.kv_dim) + self.q_dim * self.d_model
        ffn = 3 * self.d_model * self.ffn_dim
        per_layer += ffn * max(1, self.n_experts) + (self.n_experts * self.d_model if self.is_moe else 0)
        per_layer += 2 * self.d_model
        emb = self.vocab_size * self.d_model * (1 if self.tie_embeddings else 2)
        return self.n_layers * per_layer + emb + self.d_model

    def active_params(self) -> int:
        if not self.is_moe:
            return self.n_params()
        per_layer = self.d_model * (self.q_dim + 2 * self.kv_dim) + self.q_dim * self.d_model
        per_layer += 3 * self.d_model * self.ffn_dim * self.n_experts_used
        return self.n_layers * per_layer + 2 * self.vocab_size * self.d_model

    def kv_bytes_per_token(self, dtype_bytes: int = 2) -> int:
        return 2 * self.n_layers * self.kv_dim * dtype_bytes

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


PRESETS: dict[str, ModelConfig] = {
    # the reference's tiny test model (llama3.rs:66-91): h=128, L=2, 4/2 heads, vocab 1024
    "tiny": ModelConfig(name="tiny", n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=64,
                        ffn_dim=256, vocab_size=1024, max_ctx=2048),
    "tiny-moe": ModelConfig(name="tiny-moe", arch="mixtral", n_layers=2, d_model=128, n_heads=4,
                            n_kv_heads=2, head_dim=64, ffn_dim=256, vocab_size=1024, max_ctx=2048,
                            n_experts=8, n_experts_used=2),
    # CPU plumbing config: 22 layers, 2048-d, 32q/4kv heads of 64, FFN 5632, vocab 32000
    "tinyllama-1.1b": ModelConfig(name="tinyllama-1.1b", n_layers=22, d_model=2048, n_heads=32,
                                  n_kv_heads=4, head_dim=64, ffn_dim=5632, vocab_size=32000,
                                  rope_theta=10000.0, rms_eps=1e-5, max_ctx=2048),
    "llama3-8b": ModelConfig(name="llama3-8b", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8,
                             head_dim=128, ffn_dim=14336, vocab_size=128256, rope_theta=500000.0,
                             rms_eps=1e-5, max_ctx=131072, bos_id=128000, eos_id=128001),
    "llama3-70b": ModelConfig(name="llama3-70b", n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8,
                              head_dim=128, ffn_dim=28672, vocab_size=128256, rope_theta=500000.0,
                              rms_eps=1e-5, max_ctx=131072, bos_id=128000, eos_id=128001),
    "mixtral-8x7b": ModelConfig(name="mixtral-8x7b", arch="mixtral", n_layers=32, d_model=4096,
                                n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=14336, vocab_size=32000,
                                rope_theta=1000000.0, rms_eps=1e-5, max_ctx=32768, n_experts=8,
                                n_experts_used=2),
}


def preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return replace(PRESETS[name], **overrides)


def config_from_gguf(g) -> ModelConfig:
    """Build a ModelConfig from GGUF metadata and tensor shapes."""
    md = g.metadata
    arch = str(md.get("general.architecture", "llama"))

    def get(key, default=None):
        return md.get(f"{arch}.{key}", default)

    d_model = int(get("embedding_length"))
    n_layers = int(get("block_count"))
    n_heads = int(get("attention.head_count"))
    n_kv = int(get("attention.head_count_kv", n_heads))
    if "blk.0.attn_q.weight" in g.tensors:
        q_out = g.tensors["blk.0.attn_q.weight"].torch_shape[0]
        head_dim = q_out // n_heads
    elif "blk.0.attn_qkv.weight" in g.tensors:
        qkv_out = g.tensors["blk.0.attn_qkv.weight"].torch_shape[0]
        head_dim = qkv_out // (n_heads + 2 * n_kv)
    else:
        head_dim = int(get("attention.key_length", d_model // n_heads))
    n_experts = int(get("expert_count", 0) or 0)
    if n_experts > 0 and "blk.0.ffn_gate_exps.weight" in g.tensors:
        ffn = g.tensors["blk.0.ffn_gate_exps.weight"].torch_shape[-2]
    elif "blk.0.ffn_gate.weight" in g.tensors:
        ffn = g.tensors["blk.0.ffn_gate.weight"].torch_shape[0]
    else:
        ffn = int(get("feed_forward_length", 4 * d_model))
    vocab = g.tensors["token_embd.weight"].torch_shape[0] if "token_embd.weight" in g.tensors else int(
        get("vocab_size", 32000))
    scaling = str(get("rope.scaling.type", "none") or "none")
    factor = float(get("rope.scaling.factor", 1.0) or 1.0)
    if scaling == "none" and factor > 1.0:
        scaling = "llama3" if arch == "llama" else "linear"
    is_gemma = arch.startswith("gemma")
    cfg = ModelConfig(
        name=str(md.get("general.name", arch)), arch=arch, n_layers=n_layers, d_model=d_model,
        n_heads=n_heads, n_kv_heads=n_kv, head_dim=head_dim, ffn_dim=int(ffn), vocab_size=int(vocab),
        max_ctx=int(get("context_length", 8192)), rope_theta=float(get("rope.freq_base", 10000.0)),
        rope_scaling=scaling, rope_factor=factor,
        rope_orig_ctx=int(get("rope.scaling.original_context_length", 8192) or 8192),
        rms_eps=float(get("attention.layer_norm_rms_epsilon", 1e-5)),
        norm_weight_offset=1.0 if is_gemma else 0.0,
        emb_scale=float(d_model) ** 0.5 if is_gemma else 1.0,
        act="gelu_tanh" if is_gemma else "silu",
        qk_norm="blk.0.attn_q_norm.weight" in g.tensors,
        attn_bias="blk.0.attn_q.bias" in g.tensors,
        sliding_window=int(get("attention.sliding_window", 0) or 0),
        logit_softcap=float(get("final_logit_softcapping", 0.0) or 0.0),
        tie_embeddings="output.weight" not in g.tensors,
        n_experts=n_experts, n_experts_used=int(get("expert_used_count", 0) or 0),
        bos_id=int(md.get("tokenizer.ggml.bos_token_id", 1)),
        eos_id=int(md.get("tokenizer.ggml.eos_token_id", 2)),
    )
    return cfg


def gguf_metadata(cfg: ModelConfig) -> dict[str, Any]:
    """Metadata block of a GGUF checkpoint for this config (inverse of config_from_gguf)."""
    a = cfg.arch
    md: dict[str, Any] = {
        "general.architecture": a,
        "general.name": cfg.name,
        f"{a}.embedding_length": cfg.d_model,
        f"{a}.block_count": cfg.n_layers,
        f"{a}.attention.head_count": cfg.n_heads,
        f"{a}.attention.head_count_kv": cfg.n_kv_heads,
        f"{a}.context_length": cfg.max_ctx,
        f"{a}.feed_forward_length": cfg.ffn_dim,
        f"{a}.rope.freq_base": float(cfg.rope_theta),
        f"{a}.attention.layer_norm_rms_epsilon": float(cfg.rms_eps),
        f"{a}.attention.key_length": cfg.head_dim,
        "tokenizer.ggml.bos_token_id": cfg.bos_id,
        "tokenizer.ggml.eos_token_id": cfg.eos_id,
    }
    if cfg.rope_scaling != "none":
        md[f"{a}.rope.scaling.type"] = cfg.rope_scaling
        md[f"{a}.rope.scaling.factor"] = float(cfg.rope_factor)
        md[f"{a}.rope.scaling.original_context_length"] = cfg.rope_orig_ctx
    if cfg.sliding_window:
        md[f"{a}.attention.sliding_window"] = cfg.sliding_window
    if cfg.logit_softcap:
        md[f"{a}.final_logit_softcapping"] = float(cfg.logit_softcap)
    if cfg.is_moe:
        md[f"{a}.expert_count"] = cfg.n_experts
        md[f"{a}.expert_used_count"] = cfg.n_experts_used
    return md
