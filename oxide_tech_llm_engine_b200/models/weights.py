"""Weight sources: GGUF files, SafeTensors files and seeded synthetic checkpoints.

Tensor names are the GGUF ones the reference loads (oxide-models/src/llama3.rs:2871-3166):
`token_embd.weight`, `output.weight` (tied fallback), `output_norm.weight`,
`blk.{i}.{attn_norm,attn_q,attn_k,attn_v,attn_output,ffn_norm,ffn_gate,ffn_up,ffn_down}.weight`,
optional `attn_qkv`, `attn_{q,k}_norm`, `attn_{q,k,v}.bias`; plus the MoE tensors the reference
never reads: `ffn_gate_inp.weight` [E, d], `ffn_{gate,up,down}_exps.weight` [E, out, in].
"""
from __future__ import annotations

from typing import Iterable, Optional

import numpy as np

from ..errors import ModelLoadError
from ..formats import quants
from ..formats.gguf import GgufFile, GgufWriter
from .config import ModelConfig, config_from_gguf, gguf_metadata

HF_TO_GGUF = {
    "model.embed_tokens.weight": "token_embd.weight",
    "lm_head.weight": "output.weight",
    "model.norm.weight": "output_norm.weight",
}
_HF_LAYER = {
    "input_layernorm.weight": "attn_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
    "self_attn.q_proj.weight": "attn_q.weight",
    "self_attn.k_proj.weight": "attn_k.weight",
    "self_attn.v_proj.weight": "attn_v.weight",
    "self_attn.o_proj.weight": "attn_output.weight",
    "self_attn.q_proj.bias": "attn_q.bias",
    "self_attn.k_proj.bias": "attn_k.bias",
    "self_attn.v_proj.bias": "attn_v.bias",
    "self_attn.q_norm.weight": "attn_q_norm.weight",
    "self_attn.k_norm.weight": "attn_k_norm.weight",
    "mlp.gate_proj.weight": "ffn_gate.weight",
    "mlp.up_proj.weight": "ffn_up.weight",
    "mlp.down_proj.weight": "ffn_down.weight",
    "block_sparse_moe.gate.weight": "ffn_gate_inp.weight",
}


def hf_name_to_gguf(name: str) -> Optional[str]:
    if name in HF_TO_GGUF:
        return HF_TO_GGUF[name]
    if name.startswith("model.layers."):
        rest = name[len("model.layers."):]
        idx, _, tail = rest.partition(".")
        if tail in _HF_LAYER:
            return f"blk.{idx}.{_HF_LAYER[tail]}"
    return None


def tensor_names(cfg: ModelConfig) -> list[tuple[str, tuple[int, ...]]]:
    """(name, row-major shape) of every tensor of the architecture."""
    out = [("token_embd.weight", (cfg.vocab_size, cfg.d_model))]
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        out += [
            (p + "attn_norm.weight", (cfg.d_model,)),
            (p + "attn_q.weight", (cfg.q_dim, cfg.d_model)),
            (p + "attn_k.weight", (cfg.kv_dim, cfg.d_model)),
            (p + "attn_v.weight", (cfg.kv_dim, cfg.d_model)),
            (p + "attn_output.weight", (cfg.d_model, cfg.q_dim)),
            (p + "ffn_norm.weight", (cfg.d_model,)),
        ]
        if cfg.attn_bias:
            out += [(p + "attn_q.bias", (cfg.q_dim,)), (p + "attn_k.bias", (cfg.kv_dim,)),
                    (p + "attn_v.bias", (cfg.kv_dim,))]
        if cfg.qk_norm:
            out += [(p + "attn_q_norm.weight", (cfg.head_dim,)), (p + "attn_k_norm.weight", (cfg.head_dim,))]
        if cfg.is_moe:
            out += [
                (p + "ffn_gate_inp.weight", (cfg.n_experts, cfg.d_model)),
                (p + "ffn_gate_exps.weight", (cfg.n_experts, cfg.ffn_dim, cfg.d_model)),
                (p + "ffn_up_exps.weight", (cfg.n_experts, cfg.ffn_dim, cfg.d_model)),
                (p + "ffn_down_exps.weight", (cfg.n_experts, cfg.d_model, cfg.ffn_dim)),
            ]
        else:
            out += [
                (p + "ffn_gate.weight", (cfg.ffn_dim, cfg.d_model)),
                (p + "ffn_up.weight", (cfg.ffn_dim, cfg.d_model)),
                (p + "ffn_down.weight", (cfg.d_model, cfg.ffn_dim)),
            ]
    out.append(("output_norm.weight", (cfg.d_model,)))
    if not cfg.tie_embeddings:
        out.append(("output.weight", (cfg.vocab_size, cfg.d_model)))
    return out


class WeightSource:
    """Access to named tensors as float32 arrays or as packed GGUF bytes."""

    cfg: ModelConfig

    def names(self) -> Iterable[str]:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        return name in set(self.names())

    def type_name(self, name: str) -> str:
        return "F32"

    def shape(self, name: str) -> tuple[int, ...]:
        raise NotImplementedError

    def f32(self, name: str) -> np.ndarray:
        raise NotImplementedError

    def raw(self, name: str) -> np.ndarray:
        """Packed bytes in the tensor's stored type."""
        return quants.quantize(self.type_name(name), self.f32(name))


class SyntheticSource(WeightSource):
    """Random-init N(0, std) weights from a seed; norm weights are 1.0; router logits N(0, 1)-ish.

    Each tensor has its own stream derived from (seed, name), so tensors can be produced in any
    order and shard by shard with identical values.
    """

    def __init__(self, cfg: ModelConfig, seed: int = 0, std: float = 0.02):
        self.cfg = cfg
        self.seed = seed
        self.std = std
        self._shapes = dict(tensor_names(cfg))

    def names(self):
        return self._shapes.keys()

    def has(self, name):
        return name in self._shapes

    def shape(self, name):
        return self._shapes[name]

    def f32(self, name: str) -> np.ndarray:
        shape = self._shapes[name]
        if name.endswith("norm.weight"):
            return np.full(shape, 1.0 - self.cfg.norm_weight_offset, dtype=np.float32)
        h = np.frombuffer(name.encode(), dtype=np.uint8).astype(np.uint64)
        key = int((h * np.arange(1, h.size + 1, dtype=np.uint64)).sum() % (2 ** 31))
        rng = np.random.default_rng([self.seed, key])
        std = self.std
        if name.endswith("ffn_gate_inp.weight"):
            # router logits of O(1): hidden states after RMSNorm have unit RMS
            std = 1.0 / np.sqrt(self.cfg.d_model)
        if name.endswith(".bias"):
            std = 0.01
        return (rng.standard_normal(shape, dtype=np.float32) * std).astype(np.float32)


class GgufSource(WeightSource):
    def __init__(self, path: str):
        self.file = GgufFile.open(path)
        self.cfg = config_from_gguf(self.file)
        self.path = path

    def names(self):
        return self.file.tensors.keys()

    def has(self, name):
        return name in self.file.tensors

    def type_name(self, name):
        return self.file.tensors[name].type_name

    def shape(self, name):
        return self.file.tensors[name].torch_shape

    def f32(self, name):
        return self.file.dequantize(name)

    def raw(self, name):
        return self.file.raw(name)


class SafeTensorsSource(WeightSource):
    """Hugging Face layout (sharded or single file) mapped onto the GGUF tensor names."""

    def __init__(self, path: str, cfg: Optional[ModelConfig] = None):
        from ..formats.safetensors import SafeTensorsRepo

        self.repo = SafeTensorsRepo(path)
        self._map: dict[str, str] = {}
        for hf in self.repo.names():
            g = hf_name_to_gguf(hf)
            if g is not None:
                self._map[g] = hf
        self.cfg = cfg or self.repo.model_config()
        self._experts: dict[str, list[str]] = {}
        if self.cfg.is_moe:
            for i in range(self.cfg.n_layers):
                for gname, hname in (("ffn_gate_exps", "w1"), ("ffn_down_exps", "w2"), ("ffn_up_exps", "w3")):
                    keys = [f"model.layers.{i}.block_sparse_moe.experts.{e}.{hname}.weight"
                            for e in range(self.cfg.n_experts)]
                    if all(self.repo.has(k) for k in keys):
                        self._experts[f"blk.{i}.{gname}.weight"] = keys

    def names(self):
        return list(self._map.keys()) + list(self._experts.keys())

    def has(self, name):
        return name in self._map or name in self._experts

    def shape(self, name):
        if name in self._experts:
            s = self.repo.shape(self._experts[name][0])
            return (len(self._experts[name]),) + tuple(s)
        return tuple(self.repo.shape(self._map[name]))

    def type_name(self, name):
        return "F32"

    def f32(self, name):
        if name in self._experts:
            return np.stack([self.repo.f32(k) for k in self._experts[name]], 0)
        if name not in self._map:
            raise ModelLoadError(f"tensor {name} not found in {self.repo.path}")
        return self.repo.f32(self._map[name])


def open_weights(path: str) -> WeightSource:
    import os

    if os.path.isdir(path) or path.endswith(".safetensors") or path.endswith(".safetensors.index.json"):
        return SafeTensorsSource(path)
    if path.endswith(".gguf"):
        return GgufSource(path)
    with open(path, "rb") as f:
        magic = f.read(4)
    if magic == b"GGUF":
        return GgufSource(path)
    return SafeTensorsSource(path)


def write_synthetic_gguf(path: str, cfg: ModelConfig, *, seed: int = 0, weight_type: str = "Q4_0",
                         embed_type: Optional[str] = "Q8_0", std: float = 0.02,
                         tokenizer_md: Optional[dict] = None) -> None:
    """Random-init checkpoint of `cfg` as a GGUF file (norms F32, matrices `weight_type`,
    embeddings/output `embed_type`)."""
    src = SyntheticSource(cfg, seed=seed, std=std)
    md = gguf_metadata(cfg)
    if tokenizer_md:
        md.update(tokenizer_md)
    w = GgufWriter(path, md)
    for name, shape in tensor_names(cfg):
        arr = src.f32(name)
        if len(shape) == 1 or name.endswith("ffn_gate_inp.weight"):
            t = "F32"
        elif name in ("token_embd.weight", "output.weight"):
            t = embed_type or weight_type
        else:
            t = weight_type
        if shape[-1] % quants.TYPES[t].block:
            t = "F16"
        w.add_tensor(name, arr, t)
    w.write()
