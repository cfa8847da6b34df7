"""Device model: Llama-family dense decoder and Mixtral-style MoE, tensor/expert parallel.

One process per GPU. Every rank holds its shard of the weights (column-parallel QKV / gate-up /
LM head, row-parallel O / down, KV heads sharded, experts sharded) and a symmetric workspace that
peers write into directly. Between the RS and the next AG the residual stream is sequence
parallel: rank r owns rows [r*M/tp, (r+1)*M/tp). Per layer the launch sequence is

    gemm(QKV, A = all-gather buffer, waits on per-source flags)      -> fp32 / bf16
    qkv_rope_append (bias, QK-norm, RoPE, paged K/V write)           -> q
    paged_decode / paged_prefill                                     -> attn
    gemm(O, routed fp32 red into the row owner's accumulator)        == GEMM -> reduce-scatter
    finalize_norm (wait, + residual, RMSNorm, push to every rank)    == ... + all-gather
    gemm(gate|up, SwiGLU epilogue)   or   MoE: routed dispatch + grouped GEMMs
    gemm(down, routed red)  ->  finalize_norm

so no NCCL call sits on the forward path; the same code runs with tp == 1 (all pointers local).
The reference's equivalent is the single-GPU launch chain of
oxide-backend-cuda/src/lib.rs:3584-3992 (about 11 kernels per layer, fp32 activations).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..errors import ConfigError
from ..formats import quants
from ..parallel.comm import SymmetricWorkspace
from .config import ModelConfig
from .rope import inv_freq_table
from .weights import WeightSource

F_ARRIVE0, F_ARRIVE1, F_AG0, F_AG1, F_LMG, F_MOE = 0, 1, 8, 16, 24, 32
T_FIN0, T_FIN1, T_AG0, T_AG1, T_LMG, T_MOE, T_DONE_O, T_DONE_D = range(8)


def interleave32(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up rows -> [2I, K] in units of 32 rows: g0..31 | u0..31 | g32..63 | ..."""
    i, k = g.shape[-2], g.shape[-1]
    lead = g.shape[:-2]
    gg = g.reshape(*lead, i // 32, 1, 32, k)
    uu = u.reshape(*lead, i // 32, 1, 32, k)
    return torch.cat([gg, uu], dim=-3).reshape(*lead, 2 * i, k).contiguous()


@dataclass
class StepInputs:
    """Device-side description of one engine step (static buffers, sliced by the counts)."""
    m: int                 # tokens in the step, padded to a multiple of tp
    n_decode: int
    n_prefill: int
    n_tiles: int
    n_logits: int
    token_ids: torch.Tensor      # [M] int32
    positions: torch.Tensor      # [M] int32
    slot_mapping: torch.Tensor   # [M] int64 (-1 = padding row)
    seq_lens: torch.Tensor       # [n_decode] int32
    block_tables: torch.Tensor   # [n_decode, max_blocks] int32
    pages_per_split: torch.Tensor  # [1] int32
    tile_seq: Optional[torch.Tensor] = None
    tile_q0: Optional[torch.Tensor] = None
    q_start: Optional[torch.Tensor] = None
    q_lens: Optional[torch.Tensor] = None
    ctx_lens: Optional[torch.Tensor] = None
    prefill_block_tables: Optional[torch.Tensor] = None
    logit_map: Optional[torch.Tensor] = None  # [M] int32: logits row of each token row or -1


class QuantLinear:
    """A GGUF-quantized weight kept packed in HBM (tp == 1 path)."""

    def __init__(self, type_name: str, raw: np.ndarray, n: int, k: int, device):
        self.code = quants.TYPES[type_name].code
        self.type_name = type_name
        self.n, self.k = n, k
        self.packed = type_name not in ("F32", "F16", "BF16")
        if self.packed:
            self.w = torch.from_numpy(np.ascontiguousarray(raw).reshape(-1).copy()).to(device)
        else:
            f = quants.dequantize(type_name, raw, n * k).reshape(n, k)
            self.w = torch.from_numpy(f).to(device=device, dtype=torch.bfloat16)


_RANDOM_BLOCK_HEADERS = {
    # type -> (byte offset in the block, fp16 values written there) that make uniformly random payload
    # bytes decode to roughly N(0, 0.02). Q6_K keeps its super-block scale at the end of the block and
    # multiplies it by a random int8 sub-block scale and a 6-bit code.
    "Q8_0": (0, (2.7e-4,)), "Q4_0": (0, (4.3e-3,)), "Q4_K": (0, (1.4e-4, 1.05e-3)), "Q6_K": (208, (1.46e-5,)),
}


def random_quant_linear(type_name: str, n: int, k: int, device, gen: torch.Generator) -> QuantLinear:
    """A packed weight with random payload bytes generated on the device (benchmarks: no host copy,
    no quantiser pass). Supported block types: Q8_0, Q4_0, Q4_K, Q6_K."""
    info = quants.TYPES[type_name]
    if type_name not in _RANDOM_BLOCK_HEADERS or k % info.block:
        raise ConfigError(f"random packed weights: unsupported type {type_name} or K % {info.block} != 0")
    n_blocks = n * k // info.block
    raw = torch.randint(0, 256, (n_blocks, info.nbytes), dtype=torch.uint8, device=device, generator=gen)
    off, vals = _RANDOM_BLOCK_HEADERS[type_name]
    hdr = torch.tensor(vals, dtype=torch.float16).view(torch.uint8).to(device)
    raw[:, off:off + hdr.numel()] = hdr
    lin = QuantLinear.__new__(QuantLinear)
    lin.code, lin.type_name, lin.n, lin.k, lin.packed = info.code, type_name, n, k, True
    lin.w = raw.view(-1)
    return lin


def random_nvfp4(groups: int, n: int, k: int, device, gen: torch.Generator, std: float = 0.02):
    """Packed NVFP4 expert matrices with random nibbles generated on the device (benchmarks: no float
    copy, no quantiser pass). Uniform e2m1 codes have a root mean square of 2.93, so one e4m3 scale of
    0.4375 for every block and a second-level scale of std / (2.93 * 0.4375) give values of about N(0, std)."""
    q = torch.randint(0, 256, (groups, n, k // 2), dtype=torch.uint8, device=device, generator=gen)
    tiles = (n + 127) // 128
    sf = torch.full((groups * tiles * (k // 64) * 512,), 0x2E, dtype=torch.uint8, device=device)   # e4m3 0.4375
    gs = torch.full((groups,), std / (2.93 * 0.4375), dtype=torch.float32, device=device)
    return ops.Nvfp4Weight(q, sf, gs, n, k)


def fuse_quant_rows(parts: list) -> Optional[QuantLinear]:
    """Stacks packed weights that share the block type and K into one matrix (rows are independent
    byte ranges, so this is a concatenation): Q|K|V and gate|up then take one GEMV launch instead of
    three / two. Returns None when the parts cannot be stacked."""
    if any((not q.packed) or q.type_name != parts[0].type_name or q.k != parts[0].k for q in parts):
        return None
    lin = QuantLinear.__new__(QuantLinear)
    lin.code, lin.type_name, lin.k, lin.packed = parts[0].code, parts[0].type_name, parts[0].k, True
    lin.n = sum(q.n for q in parts)
    lin.w = torch.cat([q.w.view(-1) for q in parts])
    return lin


class DeviceModel:
    def __init__(self, cfg: ModelConfig, *, rank: int = 0, world: int = 1, group=None,
                 device: Optional[torch.device] = None, max_tokens: int = 2048, max_seqs: int = 256,
                 num_blocks: int = 1024, max_blocks_per_seq: int = 512, max_logits: Optional[int] = None,
                 max_splits: int = 16, weight_mode: str = "bf16", tile_weights: Optional[bool] = None,
                 layer_range: Optional[tuple] = None):
        self.cfg = cfg
        self.rank, self.tp, self.group = rank, world, group
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        tp = world
        if cfg.n_heads % tp or cfg.n_kv_heads % tp or cfg.vocab_size % tp:
            raise ConfigError(f"heads/kv heads/vocab of {cfg.name} do not divide tp={tp}")
        if cfg.is_moe and cfg.n_experts % tp:
            raise ConfigError("n_experts must be a multiple of the expert-parallel size")
        if not cfg.is_moe and (cfg.ffn_dim % (32 * tp)):
            raise ConfigError("ffn_dim / tp must be a multiple of 32")
        if weight_mode == "quant" and tp != 1:
            raise ConfigError("packed GGUF weights are served at tp=1; use weight_mode='bf16' for tp>1")
        if weight_mode == "fp8" and cfg.is_moe:
            raise ConfigError("block-scaled fp8 weights are served on dense models")
        if weight_mode == "nvfp4" and (not cfg.is_moe or cfg.d_model % 256 or cfg.ffn_dim % 256):
            raise ConfigError("NVFP4 serving covers the expert matrices of MoE models with d_model and "
                              "ffn_dim multiples of 256 (attention projections stay bf16)")
        # pipeline stage: this model owns layers [lo, hi); the first stage embeds, the last one
        # runs the final norm and the LM head, the others hand the residual stream on
        self.layer_lo, self.layer_hi = layer_range if layer_range is not None else (0, cfg.n_layers)
        self.pp_first, self.pp_last = self.layer_lo == 0, self.layer_hi == cfg.n_layers
        if layer_range is not None and weight_mode not in ("bf16",):
            raise ConfigError("pipeline stages are served with bf16 weights")
        self.weight_mode = weight_mode
        # dense bf16 projections are kept tile-major in HBM (see ops.tile_weight) unless a library
        # GEMM has to read them
        # kernels of a step overlap their start-up with the tail of the kernel before them (OXB_PDL=0: off)
        ops.set_pdl(os.environ.get("OXB_PDL", "1") != "0")
        self.fold_q8 = os.environ.get("OXB_FOLD_Q8", "1") != "0"
        self.packed_gemm = os.environ.get("OXB_PACKED_GEMM", "1") != "0"   # GGUF blocks unpacked inside the GEMM
        self.gemv_small = os.environ.get("OXB_GEMV", "1") != "0"
        self.gemv_max_rows = int(os.environ.get("OXB_GEMV_MAX", "2"))
        self._sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 148
        self._gemm_cfg: dict = {}
        self.tile_weights = (os.environ.get("OXB_TILE_WEIGHTS", "1") != "0") if tile_weights is None else tile_weights
        self.D = cfg.head_dim
        self.hq = cfg.n_heads // tp
        self.hkv = cfg.n_kv_heads // tp
        self.wqkv = (self.hq + 2 * self.hkv) * self.D
        self.i_l = cfg.ffn_dim if cfg.is_moe else cfg.ffn_dim // tp
        self.e_l = cfg.n_experts // tp if cfg.is_moe else 0
        self.v_l = cfg.vocab_size // tp
        self.max_tokens = (max_tokens + tp - 1) // tp * tp
        self.max_seqs = max_seqs
        self.max_logits = max_logits or max(max_seqs, 64)
        self.max_splits = max_splits
        self.num_blocks = num_blocks
        self.max_blocks_per_seq = max_blocks_per_seq
        self.scale = 1.0 / math.sqrt(self.D)
        inv, self.rope_mscale = inv_freq_table(cfg)
        dev = self.device
        self.inv_freq = torch.from_numpy(inv).to(dev)
        d = cfg.d_model
        M = self.max_tokens
        rpr = M // tp
        specs = {
            "acc0": ((rpr, d), "f32"), "acc1": ((rpr, d), "f32"),
            "gather0": ((M, d), "bf16"), "gather1": ((M, d), "bf16"),
            "lmg": ((self.max_logits, d), "bf16"),
            "flags": ((128,), "i32"),
        }
        if tp > 1:
            # vocab-parallel argmax: [slot, source rank, row] 64-bit words (value | index), see ops.argmax_exchange
            specs["amax"] = ((2, tp, self.max_logits, 2), "i32")
            # receive slabs of the bf16 reduce-scatter: [source rank, rows of this rank, d]
            specs["slab0"] = ((tp, rpr, d), "bf16")
            specs["slab1"] = ((tp, rpr, d), "bf16")
        self._rs_slab = [False, False]
        self.amax_slot = 1   # slot of the last argmax exchange (alternates; re-armed with the other counters)
        if cfg.is_moe:
            # rows per expert slab; the fp4 scale atoms cover 128 rows, so that path rounds up
            self.cap = (M + 127) // 128 * 128 if weight_mode == "nvfp4" else M
            specs["slab"] = ((self.e_l, self.cap, d), "bf16")
            specs["meta"] = ((self.e_l, self.cap, 4), "i32")
            specs["cnt"] = ((16,), "i32")
        self.ws = SymmetricWorkspace(specs, rank=rank, world=world, group=group, device=dev)
        self.tickets = torch.zeros(16, dtype=torch.int32, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.residual = torch.zeros(rpr, d, **bf)
        self.q_buf = torch.zeros(M, self.hq * self.D, **bf)
        self.attn_out = torch.zeros(M, self.hq * self.D, **bf)
        self.qkv_acc = torch.zeros(M, self.wqkv, dtype=torch.float32, device=dev)
        self.qkv_bf16 = torch.zeros(M, self.wqkv, **bf)
        if cfg.is_moe:
            self.act_slab = torch.zeros(self.e_l, self.cap, self.i_l, **bf)
            if weight_mode == "nvfp4":
                # quantised copies of the two expert GEMM inputs: packed e2m1, scale atoms, row scales
                rows = self.e_l * self.cap
                u8 = dict(dtype=torch.uint8, device=dev)
                mk = lambda k: (torch.zeros(rows * k // 2, **u8), torch.zeros(rows // 128 * (k // 64) * 512, **u8),
                                torch.ones(rows, dtype=torch.float32, device=dev))
                self._fp4_slab, self._fp4_act = mk(d), mk(self.i_l)
        else:
            self.act = torch.zeros(M, self.i_l, **bf)
        self.logits = torch.zeros(self.max_logits, self.v_l, dtype=torch.float32, device=dev)
        self.part_o = torch.zeros(max_seqs * self.hq * max_splits * self.D, dtype=torch.float32, device=dev)
        self.part_ml = torch.zeros(max_seqs * self.hq * max_splits * 2, dtype=torch.float32, device=dev)
        self.page_ml = self.block_mass = None   # heavy-hitter statistics, see enable_block_mass()
        self._max_seqs, self._max_blocks_per_seq = max_seqs, max_blocks_per_seq
        n_local = self.layer_hi - self.layer_lo
        self.k_cache = [torch.zeros(num_blocks, self.hkv, 16, self.D, **bf) for _ in range(n_local)]
        self.v_cache = [torch.zeros(num_blocks, self.hkv, 16, self.D, **bf) for _ in range(n_local)]
        self.pp_out = torch.zeros(rpr, d, **bf) if not self.pp_last else None
        if weight_mode == "quant":
            self.gu_acc = torch.zeros(M, 2 * self.i_l, dtype=torch.float32, device=dev)
            self._scratch: Optional[torch.Tensor] = None
            self._has_dense = False
            k_max = max(d, cfg.q_dim, cfg.ffn_dim)
            self._q8_bufs = (torch.zeros(8 * k_max, dtype=torch.int8, device=dev),
                             torch.zeros(8 * k_max // 32, dtype=torch.float32, device=dev),
                             torch.zeros(8 * k_max // 32, dtype=torch.float32, device=dev))
        if weight_mode == "fp8":
            k_max = max(d, self.hq * self.D, self.i_l)
            self.a8_flat = torch.zeros(M * k_max, dtype=torch.float8_e4m3fn, device=dev)
            self.sa_flat = torch.zeros((k_max + 127) // 128 * M, dtype=torch.float32, device=dev)
            self.gu_bf16 = torch.zeros(M, 2 * self.i_l, **bf)
            self.proj_bf16 = torch.zeros(M, d, **bf)
        self.layers: list[dict] = []
        self.embed = None
        self.lm_head = None
        self.out_norm = None
        self._act_code = 1 if cfg.act == "gelu_tanh" else 0

    # ------------------------------------------------------------------ weights
    def kv_bytes(self) -> int:
        return 2 * (self.layer_hi - self.layer_lo) * self.num_blocks * self.hkv * 16 * self.D * 2

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random-init shards generated on the device (benchmarks; no host copy of the model)."""
        cfg, dev = self.cfg, self.device
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1000 + self.rank)
        gr = torch.Generator(device=dev)
        gr.manual_seed(seed * 1000 + 999)  # replicated tensors: same stream on every rank

        def rnd(*shape, gen=g, s=std):
            t = torch.empty(*shape, dtype=torch.bfloat16, device=dev)
            t.normal_(0.0, s, generator=gen)
            return t

        d = cfg.d_model
        ones = lambda n: torch.full((n,), 1.0 - cfg.norm_weight_offset, dtype=torch.bfloat16, device=dev)
        self.embed = rnd(cfg.vocab_size, d, gen=gr)
        self.lm_head = rnd(self.v_l, d)
        self.out_norm = ones(d)
        self.layers = []
        for _ in range(self.layer_lo, self.layer_hi):
            L = {"attn_norm": ones(d), "ffn_norm": ones(d), "w_qkv": rnd(self.wqkv, d),
                 "w_o": rnd(d, self.hq * self.D), "b_qkv": None, "q_norm": None, "k_norm": None}
            if cfg.is_moe and self.weight_mode == "nvfp4":
                L["router"] = rnd(cfg.n_experts, d, gen=gr, s=1.0 / math.sqrt(d))
                L["w_gu"] = random_nvfp4(self.e_l, 2 * self.i_l, d, dev, g, std)
                L["w_down"] = random_nvfp4(self.e_l, d, self.i_l, dev, g, std)
            elif cfg.is_moe:
                L["router"] = rnd(cfg.n_experts, d, gen=gr, s=1.0 / math.sqrt(d))
                L["w_gu"] = rnd(self.e_l, 2 * self.i_l, d)
                L["w_down"] = rnd(self.e_l, d, self.i_l)
            else:
                L["w_gu"] = rnd(2 * self.i_l, d)
                L["w_down"] = rnd(d, self.i_l)
            if self.weight_mode == "fp8":
                self._to_fp8(L)
            self._tile_layer(L)
            self.layers.append(L)
        self._tile_head()

    @staticmethod
    def _fuse_quant_layer(L: dict) -> None:
        """Q|K|V and gate|up as one launch each: one stacked matrix when the block types match, else a
        mixed-type stack for the integer GEMV (a Q4_K_M file keeps attn_v in Q6_K)."""
        def mixed(parts):
            ok = all(q.packed and q.code in ops.INT8_MMVQ_CODES and q.k == parts[0].k for q in parts)
            return [(q.code, q.w, q.n) for q in parts] if ok else None

        qkv = fuse_quant_rows([L["attn_q"], L["attn_k"], L["attn_v"]])
        if qkv is not None:
            L["attn_qkv"] = qkv
            del L["attn_q"], L["attn_k"], L["attn_v"]
        else:
            L["qkv_mix"] = mixed([L["attn_q"], L["attn_k"], L["attn_v"]])
        gu = fuse_quant_rows([L["ffn_gate"], L["ffn_up"]])
        if gu is not None:
            L["ffn_gate_up"] = gu
            del L["ffn_gate"], L["ffn_up"]
        else:
            L["gu_mix"] = mixed([L["ffn_gate"], L["ffn_up"]])

    def _tile_layer(self, L: dict) -> None:
        if self.weight_mode != "bf16" or not self.tile_weights:
            return
        for key in ("w_qkv", "w_o") + (() if self.cfg.is_moe else ("w_gu", "w_down")):
            L[key] = ops.tile_weight(L[key])

    def _tile_head(self) -> None:
        if self.weight_mode == "bf16" and self.tile_weights and self.lm_head is not None:
            self.lm_head = ops.tile_weight(self.lm_head)
        if self.device.type == "cuda":
            torch.cuda.empty_cache()  # the row-major originals of the re-laid-out weights

    def init_random_quant(self, type_name: str = "Q4_K", seed: int = 0, embed_type: str = "Q8_0") -> None:
        """Random packed GGUF-format weights generated on the device (weight_mode == 'quant').
        `type_name` "Q4_K_M" lays the types out like a stock file of that name: Q4_K everywhere except
        attn_v, half of the ffn_down matrices and the output matrix, which are Q6_K."""
        cfg, dev = self.cfg, self.device
        q4km = type_name == "Q4_K_M"
        if q4km:
            type_name = "Q4_K"
        g = torch.Generator(device=dev)
        g.manual_seed(seed * 1000 + 17)
        d = cfg.d_model
        ones = lambda n: torch.full((n,), 1.0 - cfg.norm_weight_offset, dtype=torch.bfloat16, device=dev)
        self.out_norm = ones(d)
        self.embed_q = random_quant_linear(embed_type, cfg.vocab_size, d, dev, g)
        self.embed = None
        self.lm_head_q = random_quant_linear("Q6_K" if q4km else embed_type, cfg.vocab_size, d, dev, g)
        self.layers = []
        for li in range(cfg.n_layers):
            L = {"attn_norm": ones(d), "ffn_norm": ones(d), "b_qkv": None, "q_norm": None, "k_norm": None}
            for key, n, k in (("attn_q", cfg.q_dim, d), ("attn_k", cfg.kv_dim, d), ("attn_v", cfg.kv_dim, d),
                              ("attn_output", d, cfg.q_dim), ("ffn_gate", cfg.ffn_dim, d), ("ffn_up", cfg.ffn_dim, d),
                              ("ffn_down", d, cfg.ffn_dim)):
                t = "Q6_K" if q4km and (key == "attn_v" or (key == "ffn_down" and li % 2 == 0)) else type_name
                L[key] = random_quant_linear(t, n, k, dev, g)
            self._fuse_quant_layer(L)
            self.layers.append(L)

    def load(self, src: WeightSource) -> None:
        """Shards and uploads a checkpoint (GGUF / SafeTensors / synthetic source)."""
        cfg, dev, r, tp, D = self.cfg, self.device, self.rank, self.tp, self.D
        bf = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=dev, dtype=torch.bfloat16)
        hq_lo, hq_hi = r * self.hq * D, (r + 1) * self.hq * D
        kv_lo, kv_hi = r * self.hkv * D, (r + 1) * self.hkv * D
        self.out_norm = bf(src.f32("output_norm.weight"))
        head_name = "output.weight" if src.has("output.weight") else "token_embd.weight"
        quant = self.weight_mode == "quant"
        if quant:
            self.embed_q = QuantLinear(src.type_name("token_embd.weight"), src.raw("token_embd.weight"),
                                       cfg.vocab_size, cfg.d_model, dev)
            self.embed = self.embed_q.w if not self.embed_q.packed else None
            self.lm_head_q = QuantLinear(src.type_name(head_name), src.raw(head_name), cfg.vocab_size,
                                         cfg.d_model, dev) if head_name != "token_embd.weight" else self.embed_q
        else:
            self.embed = bf(src.f32("token_embd.weight"))
            self.lm_head = bf(src.f32(head_name)[r * self.v_l:(r + 1) * self.v_l])
        self.layers = []
        for i in range(self.layer_lo, self.layer_hi):
            p = f"blk.{i}."
            L: dict = {"attn_norm": bf(src.f32(p + "attn_norm.weight")), "ffn_norm": bf(src.f32(p + "ffn_norm.weight"))}
            L["q_norm"] = bf(src.f32(p + "attn_q_norm.weight")) if src.has(p + "attn_q_norm.weight") else None
            L["k_norm"] = bf(src.f32(p + "attn_k_norm.weight")) if src.has(p + "attn_k_norm.weight") else None
            if src.has(p + "attn_q.bias"):
                L["b_qkv"] = bf(np.concatenate([src.f32(p + "attn_q.bias")[hq_lo:hq_hi],
                                                src.f32(p + "attn_k.bias")[kv_lo:kv_hi],
                                                src.f32(p + "attn_v.bias")[kv_lo:kv_hi]]))
            else:
                L["b_qkv"] = None
            if quant:
                for key, n, k in (("attn_q", cfg.q_dim, cfg.d_model), ("attn_k", cfg.kv_dim, cfg.d_model),
                                  ("attn_v", cfg.kv_dim, cfg.d_model), ("attn_output", cfg.d_model, cfg.q_dim),
                                  ("ffn_gate", cfg.ffn_dim, cfg.d_model), ("ffn_up", cfg.ffn_dim, cfg.d_model),
                                  ("ffn_down", cfg.d_model, cfg.ffn_dim)):
                    nm = p + key + ".weight"
                    L[key] = QuantLinear(src.type_name(nm), src.raw(nm), n, k, dev)
                self._fuse_quant_layer(L)
            else:
                wq, wk, wv = src.f32(p + "attn_q.weight"), src.f32(p + "attn_k.weight"), src.f32(p + "attn_v.weight")
                L["w_qkv"] = bf(np.concatenate([wq[hq_lo:hq_hi], wk[kv_lo:kv_hi], wv[kv_lo:kv_hi]], 0))
                L["w_o"] = bf(src.f32(p + "attn_output.weight")[:, hq_lo:hq_hi])
                if cfg.is_moe and self.weight_mode == "nvfp4":
                    e_lo, e_hi = r * self.e_l, (r + 1) * self.e_l
                    L["router"] = bf(src.f32(p + "ffn_gate_inp.weight"))
                    L["w_gu"], L["w_down"] = self._load_nvfp4_experts(src, p, e_lo, e_hi)
                elif cfg.is_moe:
                    e_lo, e_hi = r * self.e_l, (r + 1) * self.e_l
                    L["router"] = bf(src.f32(p + "ffn_gate_inp.weight"))
                    g = bf(src.f32(p + "ffn_gate_exps.weight")[e_lo:e_hi])
                    u = bf(src.f32(p + "ffn_up_exps.weight")[e_lo:e_hi])
                    L["w_gu"] = interleave32(g, u)
                    L["w_down"] = bf(src.f32(p + "ffn_down_exps.weight")[e_lo:e_hi])
                else:
                    i_lo, i_hi = r * self.i_l, (r + 1) * self.i_l
                    g = bf(src.f32(p + "ffn_gate.weight")[i_lo:i_hi])
                    u = bf(src.f32(p + "ffn_up.weight")[i_lo:i_hi])
                    L["w_gu"] = torch.cat([g, u], 0) if self.weight_mode == "fp8" else interleave32(g, u)
                    L["w_down"] = bf(src.f32(p + "ffn_down.weight")[:, i_lo:i_hi])
                if self.weight_mode == "fp8":
                    self._to_fp8(L)
                self._tile_layer(L)
            self.layers.append(L)
        self._tile_head()

    def _load_nvfp4_experts(self, src: WeightSource, p: str, e_lo: int, e_hi: int):
        """Expert matrices of one layer for the block-scaled fp4 GEMM. Tensors stored as NVFP4 blocks
        keep their e4m3 micro-scales and nibbles bit for bit (re-ordered for the tensor cores, never
        expanded to bf16); other storage types are quantised once at load."""
        cfg, dev = self.cfg, self.device
        d, i_l, e_l = cfg.d_model, self.i_l, self.e_l
        names = [p + f"ffn_{k}_exps.weight" for k in ("gate", "up", "down")]
        if all(src.type_name(n) == "NVFP4" for n in names):
            def blocks(name, n, k):   # [experts of this rank, n, k / 16, 16] uint8
                raw = np.ascontiguousarray(src.raw(name)).reshape(cfg.n_experts, n, k // 16, 16)[e_lo:e_hi]
                return torch.from_numpy(raw.copy()).to(dev)
            g, u = blocks(names[0], i_l, d), blocks(names[1], i_l, d)
            gu = torch.cat([g.view(e_l, i_l // 32, 1, 32, d // 16, 16), u.view(e_l, i_l // 32, 1, 32, d // 16, 16)], 2)
            w_gu = ops.Nvfp4Weight.from_gguf_blocks(gu.reshape(-1, 16), 2 * i_l, d, groups=e_l)
            w_dn = ops.Nvfp4Weight.from_gguf_blocks(blocks(names[2], d, i_l).reshape(-1, 16), d, i_l, groups=e_l)
        else:
            f = lambda n: torch.from_numpy(np.ascontiguousarray(src.f32(n)[e_lo:e_hi], dtype=np.float32)).to(dev)
            w_gu = ops.Nvfp4Weight.from_float(interleave32(f(names[0]), f(names[1])))
            w_dn = ops.Nvfp4Weight.from_float(f(names[2]))
        for w in (w_gu, w_dn):   # the grouped GEMM takes [experts, N, K / 2] even for one expert
            if w.q.dim() == 2:
                w.q = w.q[None]
        return w_gu, w_dn

    def _to_fp8(self, L: dict) -> None:
        """Replaces the bf16 projections of a layer by (e4m3 values, 128 x 128 block scales)."""
        for key in ("w_qkv", "w_o", "w_gu", "w_down"):
            L[key] = ops.quant_weight_fp8_block(L[key])

    # ------------------------------------------------------------------ helpers
    def _flag_ptrs(self, index: int) -> list[int]:
        return self.ws.ptrs("flags", 4 * index)

    def _finalize(self, rows: int, norm_w, *, acc: Optional[int], gather: str, flag_base: int,
                  r0: int, first: bool = False, row_map=None, layer: Optional[dict] = None,
                  moe: bool = False, moe_acc: bool = False, out_local: Optional[torch.Tensor] = None,
                  q8=None) -> None:
        tp, d = self.tp, self.cfg.d_model
        multi = tp > 1
        kw = {}
        if acc is not None:
            if self._rs_slab[acc] and not moe_acc:
                kw["rs_slab"] = self.ws.local(f"slab{acc}")
                kw["n_slabs"] = tp
                kw["slab_stride"] = rows * d
            else:
                kw["acc"] = self.ws.local(f"acc{acc}")
            if multi:
                kw["arrive"] = self.ws.local("flags")[F_ARRIVE0 + acc:F_ARRIVE0 + acc + 1]
                kw["expected"] = tp
                kw["ticket"] = self.tickets[T_FIN0 + acc:T_FIN0 + acc + 1]
        flag_ptrs = self._flag_ptrs(flag_base + self.rank) if multi else []
        if out_local is not None:
            # stage boundary: fold the pending accumulator into the residual stream, no norm, rows
            # stay on this rank (they travel to the next stage by NCCL send)
            ops.finalize_norm(rows=rows, n=d, residual_in=self.residual, residual_out=self.residual, norm_w=None,
                              eps=self.cfg.rms_eps, out_ptrs=[out_local.data_ptr()], out_flag_ptrs=[],
                              out_row_off=0, device=self.device, **kw)
            return
        if moe:
            ops.finalize_norm(rows=rows, n=d, residual_in=self.residual, residual_out=self.residual,
                              norm_w=norm_w, eps=self.cfg.rms_eps, w_offset=self.cfg.norm_weight_offset,
                              out_flag_ptrs=flag_ptrs, router_w=layer["router"], top_k=self.cfg.n_experts_used,
                              experts_per_rank=self.e_l, routed_scale=self.cfg.routed_scale,
                              slab_ptrs=self.ws.ptrs("slab"), meta_ptrs=self.ws.ptrs("meta"),
                              cnt_ptrs=self.ws.ptrs("cnt"), cap=self.cap, my_rank=self.rank,
                              device=self.device, **kw)
            return
        ops.finalize_norm(rows=rows, n=d, residual_in=self.residual,
                          residual_out=None if first else self.residual, norm_w=norm_w,
                          eps=self.cfg.rms_eps, w_offset=self.cfg.norm_weight_offset,
                          out_ptrs=self.ws.ptrs(gather), out_flag_ptrs=flag_ptrs, out_row_off=r0,
                          out_row_map=row_map, device=self.device, q8=q8, **kw)

    def _ag_kwargs(self, flag_base: int, ticket: int, rows_per_src: int, expected: int) -> dict:
        if self.tp == 1:
            return {}
        return dict(ag_flags=self.ws.local("flags")[flag_base:flag_base + self.tp], ag_expected=expected,
                    ag_rows_per_src=rows_per_src, ag_ticket=self.tickets[ticket:ticket + 1])

    def _gemm_shape(self, m: int, n: int, k: int, *, swiglu: bool = False, routed: bool = False,
                    store: bool = False) -> dict:
        """Tile width, rows per tile, split-K factor and split-K mode of one projection. Steps of
        129 to 256 rows (large decode batches) keep every row with the CTA that streams a weight
        tile and split K to fill the SMs, combined inside the kernel; a routed projection on one GPU
        adds its splits straight into the fp32 accumulator instead. Other steps use 128-row tiles."""
        key = (m, n, k, swiglu, routed, store)
        c = self._gemm_cfg.get(key)
        if c is not None:
            return c
        # the in-kernel split-K costs about 10 us of partial-tile traffic and barrier: it pays for the
        # large weight streams (gate/up, down), not for the small ones (QKV, O), measured in situ
        big = n * k * 2 >= (48 << 20)
        if 128 < m <= 256 and big and os.environ.get("OXB_DECODE_GEMM", "1") != "0":
            bn, mt, sp = ops.pick_decode_cfg(m, n, k, swiglu=swiglu, sms=self._sms)
            fixup = sp > 1 and not (routed and self.tp == 1)
        else:
            m_tiles = (m + 127) // 128
            bn = ops.pick_bn(n, m_tiles, can_split=not swiglu)
            mt = 1
            sp = 1 if swiglu else ops.pick_splits(m, n, k, bn, self._sms)
            fixup = False
            if sp > 1 and (store or (routed and self.tp > 1)):
                # these epilogues cannot add into an fp32 accumulator: combine the splits in the kernel
                # when the launch is one wave, else do not split
                fits = (((n + bn - 1) // bn) * m_tiles * sp <= self._sms
                        and sp <= ops.max_fixup_splits(bn, 1, False))
                fixup = fits
                if not fits:
                    sp = 1
        c = dict(bn=bn, mt=mt, splits=sp, fixup=fixup)
        self._gemm_cfg[key] = c
        return c

    def _ag_kwargs_quant(self, flag_base: int, ticket: int, expected: int) -> dict:
        if self.tp == 1:
            return {}
        return dict(ag_flags=self.ws.local("flags")[flag_base:flag_base + self.tp], ag_expected=expected,
                    ag_ticket=self.tickets[ticket:ticket + 1])

    def _red_kwargs(self, acc: int, ticket: int, rpr: int, gc: Optional[dict] = None) -> dict:
        """Epilogue routing of a row-parallel GEMM. Across GPUs the partial tiles travel as bf16
        row-contiguous stores into the owner's receive slab (half the NVLink bytes of fp32 and
        full-line packets; split-K is combined locally first, so every row crosses NVLink once);
        on one GPU they are added into the fp32 accumulator."""
        splits = gc["splits"] if gc is not None else 1
        self._rs_slab[acc] = self.tp > 1 and (splits == 1 or bool(gc and gc["fixup"]))
        if self._rs_slab[acc]:
            kw = dict(epi=ops.EPI_SLAB_BF16, dst_ptrs=self.ws.ptrs(f"slab{acc}"), rows_per_owner=rpr,
                      my_rank=self.rank, dst_ld=self.cfg.d_model)
        else:
            kw = dict(epi=ops.EPI_RED_F32, dst_ptrs=self.ws.ptrs(f"acc{acc}"), rows_per_owner=rpr)
        if self.tp > 1:
            kw["arrive_ptrs"] = self._flag_ptrs(F_ARRIVE0 + acc)
            kw["done_ticket"] = self.tickets[ticket:ticket + 1]
        return kw

    def make_dense_copies(self) -> int:
        """Keeps a bf16 (tile-major) copy of every packed projection next to its GGUF blocks: steps
        with more than 8 rows (prefill, batched decode) then run the tcgen05 GEMM on it directly instead
        of expanding the blocks on every call, while small batches keep streaming the packed weights.
        Returns the bytes added."""
        added = 0
        lins = [self.lm_head_q] + [v for L in self.layers for v in L.values() if isinstance(v, QuantLinear)]
        for lin in lins:
            if not lin.packed or getattr(lin, "dense", None) is not None:
                continue
            w = torch.empty(lin.n, lin.k, dtype=torch.bfloat16, device=self.device)
            ops.dequant_rows(lin.code, lin.w, w, n_src_rows=lin.n, k=lin.k)
            lin.dense = ops.tile_weight(w) if self.tile_weights else w
            added += lin.n * lin.k * 2
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        self._has_dense = added > 0 or self._has_dense
        return added

    def _scratch_for(self, n: int, k: int) -> torch.Tensor:
        need = n * k
        if self._scratch is None or self._scratch.numel() < need:
            self._scratch = torch.empty(need, dtype=torch.bfloat16, device=self.device)
        return self._scratch[:need].view(n, k)

    def _q8_views(self, m: int, k: int, producer: bool = True):
        """Views of the int8 activation buffers for `m` rows of `k` values, or None when the integer GEMV
        does not apply (more rows than it takes, K not a multiple of 256). `producer`: asked on behalf of
        a kernel that would write the int8 view next to its own output (OXB_FOLD_Q8=0 turns that off,
        the stand-alone quantiser then runs instead)."""
        if m > (4 if self._has_dense else 8) or k % 256 or (producer and not self.fold_q8):
            return None
        b = self._q8_bufs
        return b[0][:m * k].view(m, k), b[1][:m * (k // 32)].view(m, k // 32), b[2][:m * (k // 32)].view(m, k // 32)

    def _q8(self, x: torch.Tensor):
        """int8 view of the activation rows for the integer dot-product GEMV (small batches only)."""
        if self._q8_views(x.shape[0], x.shape[1], producer=False) is None:
            return None
        return ops.quant_q8_1(x, self._q8_bufs)

    @staticmethod
    def _mmvq_rows(lin: QuantLinear) -> int:
        """Most rows that still take the packed GEMV: with a bf16 copy at hand the MMA path wins from 5
        rows on (8B Q4_K, 8 rows: 5.4 vs 9.4 ms/step)."""
        return 4 if getattr(lin, "dense", None) is not None else 8

    def _qlinear(self, lin: QuantLinear, x: torch.Tensor, out_f32: torch.Tensor, ld_out: Optional[int] = None,
                 xq=None):
        """out_f32[:, :n] = x @ W^T for a packed weight: MMVQ for small batches, else dequant + tcgen05."""
        m = x.shape[0]
        if lin.packed and m <= self._mmvq_rows(lin):
            ops.mmvq(lin.code, lin.w, x, out_f32, n=lin.n, k=lin.k,
                     xq=xq if lin.code in ops.INT8_MMVQ_CODES else None)
            return
        w = lin.w
        if lin.packed and getattr(lin, "dense", None) is not None:
            w = lin.dense
        elif lin.packed and lin.code in ops.INT8_MMVQ_CODES and lin.k % 256 == 0 and self.packed_gemm and m <= 256:
            # one row tile: the GEMM unpacks every block exactly once itself (no bf16 copy, no scratch
            # pass). Above 256 rows each row tile would unpack the weights again, and expanding them
            # once into the scratch buffer is cheaper.
            mt = 2 if m > 128 else 1
            # the unpacking is the bound: spread it over as many SMs as the tiles and K allow
            tiles = (lin.n + 127) // 128
            sp = max(1, min(self._sms // tiles, lin.k // 256, 16))
            out_f32[:m].zero_() if out_f32.is_contiguous() else out_f32[:m].fill_(0)
            ops.gemm_packed(x, lin.code, lin.w, lin.n, out_f32[:m], epi=ops.EPI_RED_F32, mt=mt, splits=sp)
            return
        elif lin.packed:
            w = self._scratch_for(lin.n, lin.k)
            ops.dequant_rows(lin.code, lin.w, w, n_src_rows=lin.n, k=lin.k)
        bn = ops.pick_bn(lin.n, (m + 127) // 128, can_split=True)
        out_f32[:m].zero_() if out_f32.is_contiguous() else out_f32[:m].fill_(0)
        ops.gemm(x, w, epi=ops.EPI_RED_F32, dst_ptrs=[out_f32.data_ptr()], bn=bn,
                 splits=ops.pick_splits(m, lin.n, lin.k, bn), dst_ld=out_f32.stride(0))

    # ------------------------------------------------------------------ forward
    def forward(self, s: StepInputs, hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Runs one step; returns fp32 logits [n_logits, vocab/tp] (a view of a static buffer). A
        pipeline stage that is not the first takes the residual rows of this rank from the previous
        stage in `hidden_in`; one that is not the last returns its residual rows [M/tp, d] instead."""
        if self.weight_mode == "quant":
            return self._forward_quant(s)
        if self.weight_mode == "fp8":
            return self._forward_fp8(s)
        cfg, tp, rank = self.cfg, self.tp, self.rank
        M = s.m
        rpr = M // tp
        r0 = rank * rpr
        d = cfg.d_model
        if self.pp_first:
            ops.embed_gather(s.token_ids[r0:r0 + rpr], self.embed, self.residual[:rpr], cfg.emb_scale)
        else:
            self.residual[:rpr].copy_(hidden_in[:rpr])
        self._finalize(rpr, self.layers[0]["attn_norm"], acc=None, gather="gather0", flag_base=F_AG0, r0=r0,
                       first=True)
        g0 = self.ws.local("gather0")[:M]
        g1 = self.ws.local("gather1")[:M]
        # single GPU, a handful of rows (latency-mode decoding): weight-streaming GEMVs instead of
        # 128-row MMA tiles
        gemv = (tp == 1 and M <= self.gemv_max_rows and not cfg.is_moe and self.gemv_small and d % 64 == 0
                and (self.hq * self.D) % 64 == 0 and self.i_l % 64 == 0 and self.wqkv % 2 == 0)
        for li, L in enumerate(self.layers):
            if gemv:
                acc0, acc1 = self.ws.local("acc0"), self.ws.local("acc1")
                ops.gemv(g0, L["w_qkv"], self.qkv_bf16[:M])
                ops.qkv_rope_append(bias=L["b_qkv"], q_norm_w=L["q_norm"], k_norm_w=L["k_norm"], norm_eps=1e-6,
                                    norm_w_offset=cfg.norm_weight_offset, positions=s.positions,
                                    slot_mapping=s.slot_mapping, inv_freq=self.inv_freq,
                                    rope_mscale=self.rope_mscale, q_out=self.q_buf, k_cache=self.k_cache[li],
                                    v_cache=self.v_cache[li], m=M, hq=self.hq, hkv=self.hkv, d=self.D,
                                    qkv_bf16=self.qkv_bf16)
                self._attention(s, li)
                self._rs_slab[0] = self._rs_slab[1] = False
                ops.gemv(self.attn_out[:M], L["w_o"], acc0[:M])
                self._finalize(rpr, L["ffn_norm"], acc=0, gather="gather1", flag_base=F_AG1, r0=r0)
                ops.gemv(g1, L["w_gu"], self.act[:M], swiglu=True, act=self._act_code)
                ops.gemv(self.act[:M], L["w_down"], acc1[:M])
                if li != len(self.layers) - 1:
                    self._finalize(rpr, self.layers[li + 1]["attn_norm"], acc=1, gather="gather0", flag_base=F_AG0,
                                   r0=r0)
                continue
            # ---- attention block ----
            ag = self._ag_kwargs(F_AG0, T_AG0, rpr, rpr)
            gc = self._gemm_shape(M, self.wqkv, d)
            if gc["splits"] > 1 and not gc["fixup"]:
                ops.gemm(g0, L["w_qkv"], epi=ops.EPI_RED_F32, dst_ptrs=[self.qkv_acc.data_ptr()], **gc, **ag)
                qkv_kw = dict(acc_f32=self.qkv_acc)
            else:
                ops.gemm(g0, L["w_qkv"], out=self.qkv_bf16[:M], **gc, **ag)
                qkv_kw = dict(qkv_bf16=self.qkv_bf16)
            ops.qkv_rope_append(bias=L["b_qkv"], q_norm_w=L["q_norm"], k_norm_w=L["k_norm"], norm_eps=1e-6,
                                norm_w_offset=cfg.norm_weight_offset, positions=s.positions,
                                slot_mapping=s.slot_mapping, inv_freq=self.inv_freq,
                                rope_mscale=self.rope_mscale, q_out=self.q_buf, k_cache=self.k_cache[li],
                                v_cache=self.v_cache[li], m=M, hq=self.hq, hkv=self.hkv, d=self.D, **qkv_kw)
            self._attention(s, li)
            gc = self._gemm_shape(M, d, self.hq * self.D, routed=True)
            ops.gemm(self.attn_out[:M], L["w_o"], **gc, **self._red_kwargs(0, T_DONE_O, rpr, gc))
            # ---- feed-forward block ----
            if cfg.is_moe:
                self._finalize(rpr, L["ffn_norm"], acc=0, gather="", flag_base=F_MOE, r0=r0, layer=L, moe=True)
                self._moe(L, M, rpr)
            else:
                self._finalize(rpr, L["ffn_norm"], acc=0, gather="gather1", flag_base=F_AG1, r0=r0)
                ops.gemm(g1, L["w_gu"], out=self.act[:M], epi=ops.EPI_SWIGLU_BF16, act=self._act_code,
                         **self._gemm_shape(M, 2 * self.i_l, d, swiglu=True),
                         **self._ag_kwargs(F_AG1, T_AG1, rpr, rpr))
                gc = self._gemm_shape(M, d, self.i_l, routed=True)
                ops.gemm(self.act[:M], L["w_down"], **gc, **self._red_kwargs(1, T_DONE_D, rpr, gc))
            last = li == len(self.layers) - 1
            if not last:
                self._finalize(rpr, self.layers[li + 1]["attn_norm"], acc=1, gather="gather0", flag_base=F_AG0,
                               r0=r0, moe_acc=cfg.is_moe)
        if not self.pp_last:
            self._finalize(rpr, None, acc=1, gather="", flag_base=0, r0=r0, moe_acc=cfg.is_moe,
                           out_local=self.pp_out)
            return self.pp_out[:rpr]
        # ---- final norm (logit rows only) + vocab-parallel LM head ----
        n_log = max(s.n_logits, 1)  # a step without logit rows still drains the last accumulator
        row_map = s.logit_map[r0:r0 + rpr] if s.logit_map is not None else None
        self._finalize(rpr, self.out_norm, acc=1, gather="lmg", flag_base=F_LMG, r0=r0 if row_map is None else 0,
                       row_map=row_map, moe_acc=cfg.is_moe)
        lmg = self.ws.local("lmg")[:n_log]
        if gemv and n_log <= 8 and self.v_l % 2 == 0:
            ops.gemv(lmg, self.lm_head, self.logits[:n_log])
        else:
            ops.gemm(lmg, self.lm_head, out=self.logits[:n_log], epi=ops.EPI_STORE_F32,
                     **self._gemm_shape(n_log, self.v_l, d, store=True), **self._ag_kwargs(F_LMG, T_LMG, 0, rpr))
        if cfg.logit_softcap > 0:
            ops.softcap(self.logits[:n_log], cfg.logit_softcap)
        return self.logits[:n_log]

    def enable_block_mass(self) -> None:
        """From now on the decode attention of the last layer also writes `block_mass[seq, page]`, the
        softmax probability mass that the step's queries (this rank's heads) put on every KV block: the
        heavy-hitter score of H2O pruning. Call before the decode graphs are captured."""
        if self.block_mass is None:
            self.page_ml = torch.zeros(self._max_seqs, self._max_blocks_per_seq, self.hq, 2, dtype=torch.float32,
                                       device=self.device)
            self.block_mass = torch.zeros(self._max_seqs, self._max_blocks_per_seq, dtype=torch.float32,
                                          device=self.device)

    def _attention(self, s: StepInputs, li: int, q8=None) -> None:
        nd = s.n_decode
        win = self.cfg.sliding_window
        if nd > 0:
            mass = self.block_mass is not None and li == len(self.k_cache) - 1
            ops.paged_decode(self.q_buf[:nd].view(nd, self.hq, self.D), self.k_cache[li], self.v_cache[li],
                             s.block_tables, s.seq_lens, s.pages_per_split, self.part_o, self.part_ml,
                             self.attn_out[:nd], batch=nd, max_splits=self.max_splits, window=win,
                             scale=self.scale, page_ml=self.page_ml if mass else None,
                             block_mass=self.block_mass if mass else None, q8=q8)
        if s.n_prefill > 0:
            ops.paged_prefill(self.q_buf.view(-1, self.hq, self.D), self.k_cache[li], self.v_cache[li],
                              s.prefill_block_tables, s.tile_seq, s.tile_q0, s.q_start, s.q_lens, s.ctx_lens,
                              self.attn_out, n_tiles=s.n_tiles, window=win, scale=self.scale)

    def _moe(self, L: dict, M: int, rpr: int) -> None:
        cfg, tp = self.cfg, self.tp
        slab, meta = self.ws.local("slab"), self.ws.local("meta")
        cnt = self.ws.local("cnt")[:self.e_l]
        m_tiles = (M * cfg.n_experts_used + 127) // 128 + self.e_l
        if self.weight_mode == "nvfp4":
            # The quantiser is the consumer of the dispatch (it waits for every source's flag, then
            # converts the rows each expert received); both expert GEMMs run on the block-scaled fp4
            # tensor-core path with the same SwiGLU and combine epilogues as the bf16 path.
            wgu, wdn = L["w_gu"], L["w_down"]
            sq, ssf, sgs = ops.quant_act_nvfp4(slab, self._fp4_slab, cnt, **self._ag_kwargs_quant(F_MOE, T_MOE, rpr))
            ops.gemm(sq, wgu.q, out=self.act_slab, epi=ops.EPI_SWIGLU_BF16, act=self._act_code, group_counts=cnt,
                     m_tiles=m_tiles, sfa=ssf, sfb=wgu.sf, a_gscale=sgs, w_gscale=wgu.gscale)
            aq, asf, ags = ops.quant_act_nvfp4(self.act_slab, self._fp4_act, cnt)
            kw = dict(epi=ops.EPI_RED_F32, dst_ptrs=self.ws.ptrs("acc1"), group_counts=cnt, row_meta=meta,
                      m_tiles=m_tiles, done_ticket=self.tickets[T_DONE_D:T_DONE_D + 1], reset_on_done=cnt,
                      sfa=asf, sfb=wdn.sf, a_gscale=ags, w_gscale=wdn.gscale)
            if tp > 1:
                kw["arrive_ptrs"] = self._flag_ptrs(F_ARRIVE1)
            ops.gemm(aq, wdn.q, **kw)
            return
        ops.gemm(slab, L["w_gu"], out=self.act_slab, epi=ops.EPI_SWIGLU_BF16, act=self._act_code,
                 group_counts=cnt, m_tiles=m_tiles, bn=128, **self._ag_kwargs(F_MOE, T_MOE, 0, rpr))
        kw = dict(epi=ops.EPI_RED_F32, dst_ptrs=self.ws.ptrs("acc1"), group_counts=cnt, row_meta=meta,
                  m_tiles=m_tiles, bn=128, done_ticket=self.tickets[T_DONE_D:T_DONE_D + 1], reset_on_done=cnt)
        if tp > 1:
            kw["arrive_ptrs"] = self._flag_ptrs(F_ARRIVE1)
        ops.gemm(self.act_slab, L["w_down"], **kw)

    def _forward_quant(self, s: StepInputs) -> torch.Tensor:
        """tp == 1 path over packed GGUF weights (MMVQ for M <= 8, dequant + tcgen05 GEMM above)."""
        cfg = self.cfg
        M, d = s.m, cfg.d_model
        acc0, acc1 = self.ws.local("acc0"), self.ws.local("acc1")
        g0, g1 = self.ws.local("gather0")[:M], self.ws.local("gather1")[:M]
        if self.embed_q.packed:
            ops.dequant_rows(self.embed_q.code, self.embed_q.w, self.residual[:M], n_src_rows=cfg.vocab_size,
                             k=d, row_ids=s.token_ids[:M], scale=cfg.emb_scale)
        else:
            ops.embed_gather(s.token_ids[:M], self.embed_q.w, self.residual[:M], cfg.emb_scale)
        # the kernels that produce an activation row also write its int8 view for the integer GEMV
        # (finalize_norm for the normed rows, swiglu for the FFN activation): no quantiser launches
        # except for the attention output
        xq_d = self._q8_views(M, d)
        self._finalize(M, self.layers[0]["attn_norm"], acc=None, gather="gather0", flag_base=F_AG0, r0=0, first=True,
                       q8=xq_d)
        qd, kd = cfg.q_dim, cfg.kv_dim
        for li, L in enumerate(self.layers):
            xq = xq_d if xq_d is not None else self._q8(g0)
            if "attn_qkv" in L:
                self._qlinear(L["attn_qkv"], g0, self.qkv_acc[:M], xq=xq)
            elif xq is not None and L.get("qkv_mix") is not None and M <= self._mmvq_rows(L["attn_q"]):
                ops.mmvq_mixed(L["qkv_mix"], g0, self.qkv_acc[:M], k=d, xq=xq)
            else:
                self._qlinear(L["attn_q"], g0, self.qkv_acc[:M, :qd], xq=xq)
                self._qlinear(L["attn_k"], g0, self.qkv_acc[:M, qd:qd + kd], xq=xq)
                self._qlinear(L["attn_v"], g0, self.qkv_acc[:M, qd + kd:], xq=xq)
            ops.qkv_rope_append(acc_f32=self.qkv_acc, bias=L["b_qkv"], q_norm_w=L["q_norm"], k_norm_w=L["k_norm"],
                                norm_eps=1e-6, norm_w_offset=cfg.norm_weight_offset, positions=s.positions,
                                slot_mapping=s.slot_mapping, inv_freq=self.inv_freq, rope_mscale=self.rope_mscale,
                                q_out=self.q_buf, k_cache=self.k_cache[li], v_cache=self.v_cache[li], m=M,
                                hq=self.hq, hkv=self.hkv, d=self.D)
            # decode-only steps: the merge kernel of the attention writes the int8 view of its output
            xq_o = self._q8_views(M, cfg.q_dim) if (s.n_prefill == 0 and s.n_decode == M) else None
            self._attention(s, li, q8=xq_o)
            self._qlinear(L["attn_output"], self.attn_out[:M], acc0[:M],
                          xq=xq_o if xq_o is not None else self._q8(self.attn_out[:M]))
            self._finalize(M, L["ffn_norm"], acc=0, gather="gather1", flag_base=F_AG1, r0=0, q8=xq_d)
            xq = xq_d if xq_d is not None else self._q8(g1)
            if "ffn_gate_up" in L:
                self._qlinear(L["ffn_gate_up"], g1, self.gu_acc[:M], xq=xq)
            elif xq is not None and L.get("gu_mix") is not None and M <= self._mmvq_rows(L["ffn_gate"]):
                ops.mmvq_mixed(L["gu_mix"], g1, self.gu_acc[:M], k=d, xq=xq)
            else:
                self._qlinear(L["ffn_gate"], g1, self.gu_acc[:M, :self.i_l], xq=xq)
                self._qlinear(L["ffn_up"], g1, self.gu_acc[:M, self.i_l:], xq=xq)
            xq_a = self._q8_views(M, self.i_l)
            ops.swiglu(acc_f32=self.gu_acc, out=self.act, m=M, i=self.i_l, act=self._act_code, q8=xq_a)
            self._qlinear(L["ffn_down"], self.act[:M], acc1[:M], xq=xq_a if xq_a is not None else self._q8(self.act[:M]))
            if li != cfg.n_layers - 1:
                self._finalize(M, self.layers[li + 1]["attn_norm"], acc=1, gather="gather0", flag_base=F_AG0, r0=0,
                               q8=xq_d)
        n_log = max(s.n_logits, 1)
        xq_l = self._q8_views(M, d)   # indexed by the destination (logits) row, of which there are at most M
        self._finalize(M, self.out_norm, acc=1, gather="lmg", flag_base=F_LMG, r0=0, row_map=s.logit_map[:M], q8=xq_l)
        lmg = self.ws.local("lmg")[:n_log]
        self._qlinear(self.lm_head_q, lmg, self.logits[:n_log],
                      xq=xq_l if xq_l is not None else (self._q8(lmg) if n_log <= 8 else None))
        if cfg.logit_softcap > 0:
            ops.softcap(self.logits[:n_log], cfg.logit_softcap)
        return self.logits[:n_log]

    def _fp8_linear(self, w, x: torch.Tensor, out: Optional[torch.Tensor], *, ag: Optional[dict] = None,
                    rs_acc: Optional[int] = None, rs_ticket: int = 0, rpr: int = 0) -> None:
        """x @ W^T with W in block-scaled fp8: quantise the activation rows (1 x 128 scales; waits on
        the all-gather flags when the rows come from peers), then the tcgen05 f8 GEMM with per-block
        promotion. `rs_acc`: row-parallel projection whose epilogue scatters bf16 partial rows into
        the row owners' receive slabs (GEMM -> reduce-scatter)."""
        m, k = x.shape
        a8 = self.a8_flat[:m * k].view(m, k)
        sa = self.sa_flat[:(k + 127) // 128 * m].view(-1, m)
        ops.quant_act_fp8(x, a8, sa, **(ag or {}))
        if rs_acc is None:
            ops.gemm_fp8_block(a8, sa, w[0], w[1], out=out)
            return
        self._rs_slab[rs_acc] = True
        ops.gemm_fp8_block(a8, sa, w[0], w[1], slab_ptrs=self.ws.ptrs(f"slab{rs_acc}"),
                           arrive_ptrs=self._flag_ptrs(F_ARRIVE0 + rs_acc),
                           done_ticket=self.tickets[rs_ticket:rs_ticket + 1], rows_per_owner=rpr,
                           my_rank=self.rank, slab_ld=self.cfg.d_model)

    def _forward_fp8(self, s: StepInputs) -> torch.Tensor:
        """Block-scaled fp8 projections (embedding, norms and LM head stay bf16). Tensor parallel with
        the same hand-offs as the bf16 path: the activation quantiser is the consumer of the
        all-gather buffers, the fp8 GEMM's epilogue is the reduce-scatter of O and down."""
        cfg, tp, rank = self.cfg, self.tp, self.rank
        M, d = s.m, cfg.d_model
        rpr = M // tp
        r0 = rank * rpr
        g0, g1 = self.ws.local("gather0")[:M], self.ws.local("gather1")[:M]
        ops.embed_gather(s.token_ids[r0:r0 + rpr], self.embed, self.residual[:rpr], cfg.emb_scale)
        self._finalize(rpr, self.layers[0]["attn_norm"], acc=None, gather="gather0", flag_base=F_AG0, r0=r0,
                       first=True)
        proj = self.proj_bf16[:M] if tp == 1 else None

        def ag(flag_base, ticket):
            if tp == 1:
                return None
            return dict(ag_flags=self.ws.local("flags")[flag_base:flag_base + tp], ag_expected=rpr,
                        ag_rows_per_src=rpr, ag_ticket=self.tickets[ticket:ticket + 1])

        def fin(norm_w, gather, flag_base, acc, **kw):
            if tp > 1:
                self._finalize(rpr, norm_w, acc=acc, gather=gather, flag_base=flag_base, r0=kw.pop("r0", r0), **kw)
                return
            ops.finalize_norm(rows=M, n=d, rs_slab=proj, n_slabs=1, slab_stride=M * d, residual_in=self.residual,
                              residual_out=self.residual, norm_w=norm_w, eps=cfg.rms_eps,
                              w_offset=cfg.norm_weight_offset, out_ptrs=self.ws.ptrs(gather), out_flag_ptrs=[],
                              out_row_off=0, device=self.device, out_row_map=kw.get("row_map"))

        for li, L in enumerate(self.layers):
            self._fp8_linear(L["w_qkv"], g0, self.qkv_bf16[:M], ag=ag(F_AG0, T_AG0))
            ops.qkv_rope_append(qkv_bf16=self.qkv_bf16, bias=L["b_qkv"], q_norm_w=L["q_norm"], k_norm_w=L["k_norm"],
                                norm_eps=1e-6, norm_w_offset=cfg.norm_weight_offset, positions=s.positions,
                                slot_mapping=s.slot_mapping, inv_freq=self.inv_freq, rope_mscale=self.rope_mscale,
                                q_out=self.q_buf, k_cache=self.k_cache[li], v_cache=self.v_cache[li], m=M,
                                hq=self.hq, hkv=self.hkv, d=self.D)
            self._attention(s, li)
            if tp == 1:
                self._fp8_linear(L["w_o"], self.attn_out[:M], proj)
            else:
                self._fp8_linear(L["w_o"], self.attn_out[:M], None, rs_acc=0, rs_ticket=T_DONE_O, rpr=rpr)
            fin(L["ffn_norm"], "gather1", F_AG1, 0)
            self._fp8_linear(L["w_gu"], g1, self.gu_bf16[:M], ag=ag(F_AG1, T_AG1))
            ops.swiglu(gu_bf16=self.gu_bf16, out=self.act, m=M, i=self.i_l, act=self._act_code)
            if tp == 1:
                self._fp8_linear(L["w_down"], self.act[:M], proj)
            else:
                self._fp8_linear(L["w_down"], self.act[:M], None, rs_acc=1, rs_ticket=T_DONE_D, rpr=rpr)
            if li != cfg.n_layers - 1:
                fin(self.layers[li + 1]["attn_norm"], "gather0", F_AG0, 1)
        n_log = max(s.n_logits, 1)
        row_map = s.logit_map[r0:r0 + rpr] if s.logit_map is not None else None
        fin(self.out_norm, "lmg", F_LMG, 1, row_map=row_map, r0=r0 if row_map is None else 0)
        lmg = self.ws.local("lmg")[:n_log]
        ops.gemm(lmg, self.lm_head, out=self.logits[:n_log], epi=ops.EPI_STORE_F32,
                 bn=ops.pick_bn(self.v_l, (n_log + 127) // 128), **self._ag_kwargs(F_LMG, T_LMG, 0, rpr))
        if cfg.logit_softcap > 0:
            ops.softcap(self.logits[:n_log], cfg.logit_softcap)
        return self.logits[:n_log]

    # ------------------------------------------------------------------ baseline path
    def forward_baseline(self, s: StepInputs) -> torch.Tensor:
        """The comparison path: library GEMMs (torch / cuBLAS) with plain NCCL all-reduces between
        them and unfused residual / norm / activation steps; attention and the KV append still use
        this engine's kernels. Replicated activations (no sequence parallelism), dense models."""
        import torch.distributed as dist
        import torch.nn.functional as F

        cfg, tp = self.cfg, self.tp
        if cfg.is_moe or self.weight_mode != "bf16":
            raise ConfigError("the NCCL + library-GEMM baseline covers dense bf16 models")
        M = s.m
        eps, off = cfg.rms_eps, cfg.norm_weight_offset
        rowmajor = ops.untile_weight  # the fused path keeps weights tile-major; a library GEMM reads rows

        def norm(x, w):
            xf = x.float()
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + off)).to(torch.bfloat16)

        x = (self.embed[s.token_ids[:M].long()].float() * cfg.emb_scale).to(torch.bfloat16)
        for li, L in enumerate(self.layers):
            h = norm(x, L["attn_norm"])
            qkv = F.linear(h, rowmajor(L["w_qkv"]))
            ops.qkv_rope_append(qkv_bf16=qkv, bias=L["b_qkv"], q_norm_w=L["q_norm"], k_norm_w=L["k_norm"],
                                norm_eps=1e-6, norm_w_offset=off, positions=s.positions, slot_mapping=s.slot_mapping,
                                inv_freq=self.inv_freq, rope_mscale=self.rope_mscale, q_out=self.q_buf,
                                k_cache=self.k_cache[li], v_cache=self.v_cache[li], m=M, hq=self.hq, hkv=self.hkv,
                                d=self.D)
            self._attention(s, li)
            o = F.linear(self.attn_out[:M], rowmajor(L["w_o"]))
            if tp > 1:
                dist.all_reduce(o, group=self.group)
            x = x + o
            h = norm(x, L["ffn_norm"])
            gu = F.linear(h, rowmajor(L["w_gu"])).view(M, self.i_l // 32, 2, 32)
            gate, up = gu[:, :, 0].reshape(M, self.i_l), gu[:, :, 1].reshape(M, self.i_l)
            a = (F.gelu(gate.float(), approximate="tanh") if self._act_code else F.silu(gate.float())) * up.float()
            dn = F.linear(a.to(torch.bfloat16), rowmajor(L["w_down"]))
            if tp > 1:
                dist.all_reduce(dn, group=self.group)
            x = x + dn
        n_log = max(s.n_logits, 1)
        if s.n_logits == M:
            # decode bucket: every row has a logits row, in order (no host round trip, so the step
            # can be captured in a CUDA graph)
            hl = norm(x, self.out_norm)
        else:
            rows = torch.nonzero(s.logit_map[:M] >= 0).flatten()
            if rows.numel() == 0:
                rows = torch.zeros(1, dtype=torch.long, device=self.device)
            order = torch.argsort(s.logit_map[:M][rows])
            hl = norm(x[rows[order]], self.out_norm)
        logits = F.linear(hl, rowmajor(self.lm_head)).float()
        if cfg.logit_softcap > 0:
            logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
        self.logits[:logits.shape[0]] = logits
        return self.logits[:n_log]

    def reset_sync_state(self) -> None:
        """Re-arms every counter of the hand-off protocol on this rank (arrival / all-gather flags,
        tickets, split-K tickets, MoE slot counters). Used after a device wait ran out: waiters that
        gave up leave tickets part-way and a late peer may still bump a flag. Every rank of the group
        calls it between steps, with none of its kernels in flight."""
        torch.cuda.synchronize(self.device)
        self.ws.local("flags").zero_()
        if self.tp > 1:
            self.ws.local("amax").zero_()
            self.amax_slot = 1
        self.tickets.zero_()
        if self.cfg.is_moe:
            self.ws.local("cnt").zero_()
        ops.gemm_workspace(self.device)[1].zero_()
        for name in ("acc0", "acc1"):
            self.ws.local(name).zero_()
        self.qkv_acc.zero_()
        torch.cuda.synchronize(self.device)

    def close(self) -> None:
        self.ws.close()
