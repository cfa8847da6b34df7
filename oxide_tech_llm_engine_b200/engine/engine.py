"""LLMEngine: continuous-batching serving loop of one rank.

step() = C++ scheduler builds the plan -> one pinned-host -> device copy of the step descriptor
-> forward (CUDA graph replay for decode-only buckets, eager launches for steps with prefill
chunks) -> device sampler -> D2H of the sampled ids -> scheduler update -> token events.
With tp > 1 every rank runs the same deterministic scheduler on the same request stream, so no
per-step control traffic is needed; rank 0 owns the client-facing side.

Reference parity: ContinuousBatchingEngine::run_loop / step_batch_overlap
(oxide-engine/src/continuous_batching.rs:303-1395), CudaBackend::dispatch_batch_decode_step with
one graph per batch bucket (oxide-backend-cuda/src/lib.rs:3326-4114), prefix reuse
(continuous_batching.rs:406-437), typed errors and per-request failure (`:664-672`).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional

import numpy as np
import torch

from .. import ops
from .._build import host_ext
from ..config import EngineConfig
from ..errors import ConfigError, EngineError, OutOfMemory
from ..models.config import ModelConfig, preset
from ..models.llama import DeviceModel, StepInputs
from ..sampling_params import SamplingParams


@dataclass
class RequestState:
    req_id: int
    params: SamplingParams
    prompt_len: int
    t_arrival: float
    t_first_token: Optional[float] = None
    t_last_token: Optional[float] = None
    n_generated: int = 0
    host_sampler: object = None
    grammar: object = None
    on_token: Optional[Callable] = None
    output: list = field(default_factory=list)
    finished: bool = False
    finish_reason: str = ""
    spec: object = None        # AdaptiveSpeculator of this request (speculative decoding)
    n_drafted: int = 0         # drafts attached to the step in flight


@dataclass
class _Event:
    """Engine-made token event (same fields as the scheduler's TokenEvent)."""
    req_id: int
    token: int
    finished: bool
    reason: str


class _Staging:
    """One pinned host buffer and its device mirror holding every per-step array; a step is
    described to the GPU with a single H2D copy."""

    def __init__(self, fields_: dict[str, tuple[int, np.dtype]], device):
        off = 0
        self.off: dict[str, tuple[int, int, np.dtype]] = {}
        for name, (count, dt) in fields_.items():
            dt = np.dtype(dt)
            off = (off + 15) // 16 * 16
            self.off[name] = (off, count, dt)
            off += count * dt.itemsize
        self.nbytes = (off + 15) // 16 * 16
        pin = torch.cuda.is_available()
        self.host = torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        self._tdt = {np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
                     np.dtype(np.float32): torch.float32}

    def h(self, name: str) -> np.ndarray:
        o, c, dt = self.off[name]
        return self.host_np[o:o + c * dt.itemsize].view(dt)

    def d(self, name: str) -> torch.Tensor:
        o, c, dt = self.off[name]
        return self.dev[o:o + c * dt.itemsize].view(self._tdt[dt])

    def upload(self, upto: Optional[int] = None) -> int:
        n = self.nbytes if upto is None else upto
        self.dev[:n].copy_(self.host[:n], non_blocking=True)
        return n


class LLMEngine:
    def __init__(self, cfg: EngineConfig, model_cfg: Optional[ModelConfig] = None, *, weights=None,
                 rank: int = 0, world: int = 1, group=None, device: Optional[torch.device] = None,
                 random_init: bool = False, random_quant_type: Optional[str] = None, pp=None):
        self.cfg = cfg
        self.group = group
        self._decode_ctas_per_sm = int(os.environ.get("OXB_DECODE_CTAS_PER_SM", "0"))
        self.pp = pp  # parallel.pipeline.PpContext or None; rank/world/group describe the TP group of this stage
        self.rank, self.world = rank, world
        self.cpu = cfg.backend == "cpu"
        if self.cpu:
            self._init_cpu(cfg, model_cfg, weights)
            return
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        if model_cfg is None:
            if weights is not None:
                model_cfg = weights.cfg
            else:
                model_cfg = preset(cfg.model)
        self.model_cfg = model_cfg
        mc = model_cfg
        H = host_ext()
        self.block = H.TOKENS_PER_BLOCK
        max_blocks_per_seq = (min(cfg.ctx_size, mc.max_ctx) + self.block - 1) // self.block
        weight_mode = cfg.weight_mode
        if weight_mode == "auto":
            packed = weights is not None and any(
                weights.type_name(n) not in ("F32", "F16", "BF16") for n in ("blk.0.attn_q.weight",)
                if weights.has(n))
            weight_mode = "quant" if packed and world == 1 and not mc.is_moe else "bf16"
            if (mc.is_moe and weights is not None and weights.has("blk.0.ffn_gate_exps.weight")
                    and weights.type_name("blk.0.ffn_gate_exps.weight") == "NVFP4"
                    and mc.d_model % 256 == 0 and mc.ffn_dim % 256 == 0):
                weight_mode = "nvfp4"   # expert matrices stay packed and run on the fp4 tensor-core path
        self.max_tokens = max(cfg.max_num_batched_tokens, cfg.max_num_seqs)
        self.max_tokens = (self.max_tokens + world - 1) // world * world
        # packed GGUF weights may be doubled by a bf16 copy for batched steps (decided before the KV
        # pool is sized): by default when that copy is under a quarter of the free memory
        self._dense_bytes = 0
        if weight_mode == "quant" and cfg.quant_dense_copy != "off" and (weights is not None or random_init):
            need = 2 * mc.n_params()
            free_now, _ = torch.cuda.mem_get_info(self.device)
            if cfg.quant_dense_copy == "on" or need < free_now // 4:
                self._dense_bytes = need
        num_blocks = cfg.num_kv_blocks
        if num_blocks <= 0:
            num_blocks = self._auto_blocks(mc, weight_mode, random_init or weights is not None)
        self.model = DeviceModel(mc, rank=rank, world=world, group=group, device=self.device,
                                 max_tokens=self.max_tokens, max_seqs=cfg.max_num_seqs,
                                 num_blocks=num_blocks, max_blocks_per_seq=max_blocks_per_seq,
                                 max_logits=max(cfg.max_num_seqs * (1 + (cfg.draft_tokens if cfg.speculative != "off" else 0)), 64),
                                 max_splits=cfg.max_splits, weight_mode=weight_mode,
                                 tile_weights=False if (cfg.comm == "nccl" or cfg.gemm == "library") else None,
                                 layer_range=pp.layers(mc.n_layers) if pp is not None else None)
        if cfg.h2o_pruning:
            self.model.enable_block_mass()
        if pp is not None:
            self.pp_recv = torch.zeros(self.max_tokens // world, mc.d_model, dtype=torch.bfloat16, device=self.device)
            self.pp_tokens = torch.zeros(max(cfg.max_num_seqs * (1 + cfg.draft_tokens), 64), dtype=torch.int32,
                                         device=self.device)
        if weights is not None:
            self.model.load(weights)
        elif random_init and weight_mode == "quant":
            self.model.init_random_quant(random_quant_type or "Q4_K", cfg.seed)
        elif random_init:
            self.model.init_random(cfg.seed)
        if weight_mode == "quant" and (weights is not None or random_init) and cfg.quant_dense_copy != "off":
            # batched steps then run at bf16-GEMM speed, small batches keep streaming the packed blocks
            if self._dense_bytes:
                self.stats_dense_copy_bytes = self.model.make_dense_copies()
        sc = H.SchedulerConfig()
        sc.num_blocks = num_blocks
        sc.max_num_seqs = cfg.max_num_seqs
        sc.max_num_batched_tokens = cfg.max_num_batched_tokens
        sc.max_blocks_per_seq = max_blocks_per_seq
        sc.chunk_min, sc.chunk_max = cfg.chunk_min, cfg.chunk_max
        sc.sla_itl_us, sc.base_us, sc.per_token_us = cfg.sla_itl_us, cfg.base_us, cfg.per_token_us
        sc.enable_radix = cfg.enable_radix
        sc.sla_budget = cfg.sla_budget
        sc.context_shift, sc.shift_keep_tokens, sc.shift_step_tokens = (cfg.context_shift, cfg.shift_keep_tokens,
                                                                        cfg.shift_step_tokens)
        self.sched = H.Scheduler(sc)
        self._init_kv_tiers()
        self.max_blocks_per_seq = max_blocks_per_seq
        S, M = cfg.max_num_seqs, self.max_tokens
        n_tiles_max = M // 64 + S + 1
        i32, i64 = np.int32, np.int64
        self.st = _Staging({
            "token_ids": (M, i32), "positions": (M, i32), "logit_map": (M, i32), "slot_mapping": (M, i64),
            "pages_per_split": (4, i32), "seq_lens": (S, i32), "block_tables": (S * max_blocks_per_seq, i32),
            "q_start": (S, i32), "q_lens": (S, i32), "ctx_lens": (S, i32), "tile_seq": (n_tiles_max, i32),
            "tile_q0": (n_tiles_max, i32), "prefill_block_tables": (S * max_blocks_per_seq, i32),
            "cow_src": (S, i32), "cow_dst": (S, i32),
            "temperature": (self.model.max_logits, np.float32), "top_k": (self.model.max_logits, i32),
            "top_p": (self.model.max_logits, np.float32), "min_p": (self.model.max_logits, np.float32),
            "seeds": (self.model.max_logits, i64), "counters": (self.model.max_logits, i64),
        }, self.device)
        # everything up to the prefill arrays is what a decode-only step needs
        self._decode_bytes = self.st.off["q_start"][0]
        self.sampled = torch.zeros(self.model.max_logits, dtype=torch.int32, device=self.device)
        self.sampled_val = torch.zeros(self.model.max_logits, dtype=torch.float32, device=self.device)
        self.sampled_host = torch.zeros(self.model.max_logits, dtype=torch.int32,
                                        pin_memory=torch.cuda.is_available())
        # the kernels' status word rides home with the sampled ids of every step
        self.status_host = torch.zeros(1, dtype=torch.int32, pin_memory=torch.cuda.is_available())
        self.requests: dict[int, RequestState] = {}
        self._next_id = 0
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_launches: dict[int, int] = {}
        # decode bursts: K graph replays per host round trip (in-graph step advance, tokens come home
        # through a ring in mapped pinned memory)
        self._burst_k = cfg.decode_burst if (cfg.decode_burst > 1 and world == 1 and pp is None and cfg.cuda_graph
                                             and cfg.comm != "nccl" and cfg.gemm != "library") else 0
        self.burst_graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._burst_steps = 0
        if self._burst_k:
            self._burst_ring = 2 * self._burst_k
            self._burst_rows = self._bucket(max(1, cfg.burst_max_batch)) or cfg.burst_max_batch
            self._mail, self._mail_dev = ops.alloc_mapped_host(self._burst_ring * self._burst_rows)
            self._mail_np = self._mail.numpy()
            self._burst_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.stats = {"steps": 0, "decode_tokens": 0, "prefill_tokens": 0, "graph_replays": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0, "degraded": False}
        self.stop_ids_default = [mc.eos_id]
        self._drafter = None
        if cfg.speculative in ("ngram", "auto"):
            from .spec_decode import NgramDrafter

            self._drafter = NgramDrafter(cfg.draft_tokens)

    def _init_cpu(self, cfg: EngineConfig, model_cfg, weights) -> None:
        """fp32 torch backend over the same scheduler / block manager (no GPU needed)."""
        from ..models.cpu_model import CpuPagedModel
        from ..models.weights import SyntheticSource

        self.device = torch.device("cpu")
        if model_cfg is None:
            model_cfg = weights.cfg if weights is not None else preset(cfg.model)
        if weights is None:
            weights = SyntheticSource(model_cfg, seed=cfg.seed)
        self.model_cfg = mc = model_cfg
        H = host_ext()
        self.block = H.TOKENS_PER_BLOCK
        self.max_blocks_per_seq = (min(cfg.ctx_size, mc.max_ctx) + self.block - 1) // self.block
        num_blocks = cfg.num_kv_blocks if cfg.num_kv_blocks > 0 else min(
            4096, cfg.max_num_seqs * self.max_blocks_per_seq + 16)
        self.model = CpuPagedModel(mc, weights, num_blocks)
        sc = H.SchedulerConfig()
        sc.num_blocks = num_blocks
        sc.max_num_seqs = cfg.max_num_seqs
        sc.max_num_batched_tokens = cfg.max_num_batched_tokens
        sc.max_blocks_per_seq = self.max_blocks_per_seq
        sc.chunk_min, sc.chunk_max = cfg.chunk_min, cfg.chunk_max
        sc.sla_itl_us, sc.base_us, sc.per_token_us = cfg.sla_itl_us, cfg.base_us, cfg.per_token_us
        sc.enable_radix = cfg.enable_radix
        sc.sla_budget = cfg.sla_budget
        sc.context_shift, sc.shift_keep_tokens, sc.shift_step_tokens = (cfg.context_shift, cfg.shift_keep_tokens,
                                                                        cfg.shift_step_tokens)
        self.sched = H.Scheduler(sc)
        self._init_kv_tiers()
        self.requests = {}
        self._next_id = 0
        self.graphs, self.graph_launches = {}, {}
        self.stats = {"steps": 0, "decode_tokens": 0, "prefill_tokens": 0, "graph_replays": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0, "degraded": False}
        self.stop_ids_default = [mc.eos_id]
        self._drafter = None
        if cfg.speculative in ("ngram", "auto"):
            from .spec_decode import NgramDrafter

            self._drafter = NgramDrafter(cfg.draft_tokens)

    def _step_cpu(self, plan) -> np.ndarray:
        if plan.cow_src.size:
            self.model.copy_blocks(plan.cow_src, plan.cow_dst)
        logits = self.model.forward_plan(plan).numpy()
        toks = np.zeros(plan.logit_rows.size, dtype=np.int32)
        for i, rid in enumerate(plan.logit_req):
            r = self.requests.get(int(rid))
            row = logits[i]
            mask = None
            if r is not None and r.grammar is not None:
                mask = r.grammar.allow_mask(self.model_cfg.vocab_size)
            if r is None or (r.params.is_greedy() and mask is None):
                toks[i] = int(row.argmax())
                continue
            if r.host_sampler is None:
                from ..sampler import HostSampler

                r.host_sampler = HostSampler(r.params)
            hist = self.sched.request_tokens(r.req_id)
            hist = hist[r.prompt_len:] if hist is not None else np.zeros(0, np.int32)
            toks[i] = r.host_sampler.sample(row, hist, mask)
        return toks

    # ------------------------------------------------------------------ sizing
    def _auto_blocks(self, mc: ModelConfig, weight_mode: str, has_weights: bool) -> int:
        free, total = torch.cuda.mem_get_info(self.device)
        tp = self.world
        w_bytes = 0
        if has_weights:
            per = {"bf16": 2.0, "fp8": 1.02, "nvfp4": 0.7}.get(weight_mode, 0.6)
            n = mc.n_params()
            w_bytes = int((n - mc.vocab_size * mc.d_model) / tp * per + mc.vocab_size * mc.d_model * 2)
        act = self.max_tokens * (mc.d_model * 16 + (mc.q_dim + 2 * mc.kv_dim) // tp * 8 + mc.ffn_dim // tp * 4)
        act += self.cfg.max_num_seqs * (mc.vocab_size // tp) * 4 * 2
        if mc.is_moe:
            act += (mc.n_experts // tp) * self.max_tokens * (mc.d_model + mc.ffn_dim) * 2
        budget = int(free * self.cfg.gpu_memory_utilization) - w_bytes - act - (2 << 30) - getattr(self, "_dense_bytes", 0)
        per_block = 2 * mc.n_layers * (mc.n_kv_heads // tp) * 16 * mc.head_dim * 2
        n = budget // per_block
        if n < 16:
            raise OutOfMemory(f"not enough device memory for the KV pool ({budget} bytes left for blocks)")
        cap = self.cfg.max_num_seqs * ((min(self.cfg.ctx_size, mc.max_ctx) + 15) // 16) + 64
        return int(min(n, cap))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_tokens: Iterable[int], params: Optional[SamplingParams] = None,
                    on_token: Optional[Callable] = None, req_id: Optional[int] = None) -> int:
        params = params or SamplingParams()
        toks = np.asarray(list(prompt_tokens), dtype=np.int32)
        if toks.size == 0:
            raise ConfigError("empty prompt")
        rid = self._next_id if req_id is None else req_id
        self._next_id = max(self._next_id, rid) + 1
        stop = list(params.stop_token_ids) or list(self.stop_ids_default)
        if getattr(self, "kv_tier", None) is not None:
            self._promote_prefix(toks)
        self.sched.add_request(rid, toks, int(params.max_tokens), stop, bool(params.ignore_eos))
        st = RequestState(rid, params, int(toks.size), time.perf_counter(), on_token=on_token)
        if not params.is_greedy() and not params.device_ok():
            from ..sampler import HostSampler

            st.host_sampler = HostSampler(params)
        if params.grammar:
            from ..grammar import grammar_from_spec

            st.grammar = grammar_from_spec(params.grammar, getattr(self, "vocab_bytes", None))
        self.requests[rid] = st
        return rid

    def set_tokenizer(self, tokenizer) -> None:
        """Gives grammars the byte strings of the vocabulary and the engine the stop ids."""
        self.vocab_bytes = tokenizer.vocab_bytes()
        self.stop_ids_default = tokenizer.stop_ids()
        self._bytes_to_token = {}
        for i, b in enumerate(self.vocab_bytes):
            if b and b not in self._bytes_to_token:
                self._bytes_to_token[bytes(b)] = i
        self._max_token_bytes = max((len(b) for b in self._bytes_to_token), default=1)

    def cancel(self, req_id: int) -> bool:
        ok, events = self.sched.cancel(req_id)
        for e in events:
            self._deliver(e)
        return ok

    def has_work(self) -> bool:
        return self.sched.has_work()

    # ------------------------------------------------------------------ step
    def _bucket(self, n: int) -> Optional[int]:
        for b in self.cfg.graph_buckets:
            if b >= n and b % self.world == 0 and b <= self.cfg.max_num_seqs:
                return b
        return None

    def _fill(self, plan, extra_len: int = 0):
        """Writes the step descriptor and uploads it. `extra_len`: tokens the sequences will grow by
        before the next upload (decode burst); the KV split covers them."""
        st = self.st
        n, nd, npf = plan.n_tokens, plan.n_decode, plan.n_prefill
        world = self.world
        decode_only = npf == 0
        m = n
        bucket = self._bucket(nd) if (decode_only and self.cfg.cuda_graph) else None
        if bucket is not None:
            m = bucket
        m = (m + world - 1) // world * world
        h = st.h
        tok, pos, slot, lmap = h("token_ids"), h("positions"), h("slot_mapping"), h("logit_map")
        tok[:n] = plan.token_ids
        pos[:n] = plan.positions
        slot[:n] = plan.slot_mapping
        tok[n:m] = 0
        pos[n:m] = 0
        slot[n:m] = -1
        rows = plan.logit_rows
        if bucket is not None:
            lmap[:m] = np.arange(m, dtype=np.int32)  # graph buckets compute logits for every row
        else:
            lmap[:m] = -1
            lmap[rows] = np.arange(rows.size, dtype=np.int32)
        W = self.max_blocks_per_seq
        w = plan.max_blocks
        nd_pad = m if decode_only else nd
        if nd > 0:
            sl = h("seq_lens")
            sl[:nd] = plan.decode_seq_lens
            sl[nd:nd_pad] = 0
            bt = h("block_tables").reshape(-1, W)
            bt[:nd, :w] = plan.decode_block_tables.reshape(nd, w)
            max_len = int(plan.decode_seq_lens.max()) + extra_len
            pages = (max_len + 15) // 16
            # enough CTAs to fill the SMs a few times over, at least one page per warp. With several KV
            # heads per rank (single GPU, low TP) shorter page chains balance ragged lengths better:
            # measured best near 12 CTAs per SM there, near 4 with one KV head per rank (TP = 8).
            per_sm = self._decode_ctas_per_sm or (12 if self.model.hkv >= 4 else 4)
            want = -(-per_sm * getattr(self.model, "_sms", 148) // max(1, nd * self.model.hkv))
            splits = max(1, min(self.cfg.max_splits, want))
            pps = max(4, -(-pages // splits))
            pps = (pps + 3) // 4 * 4
            h("pages_per_split")[0] = pps
        n_tiles = 0
        if npf > 0:
            h("q_start")[:npf] = plan.q_start
            h("q_lens")[:npf] = plan.q_lens
            h("ctx_lens")[:npf] = plan.ctx_lens
            n_tiles = plan.tile_seq.size
            h("tile_seq")[:n_tiles] = plan.tile_seq
            h("tile_q0")[:n_tiles] = plan.tile_q0
            pbt = h("prefill_block_tables").reshape(-1, W)
            pbt[:npf, :w] = plan.prefill_block_tables.reshape(npf, w)
        n_cow = plan.cow_src.size
        if n_cow:
            h("cow_src")[:n_cow] = plan.cow_src
            h("cow_dst")[:n_cow] = plan.cow_dst
        nbytes = st.upload(self._decode_bytes if (decode_only and not n_cow) else None)
        self.stats["h2d_bytes"] += nbytes
        d = st.d
        s = StepInputs(m=m, n_decode=nd_pad if decode_only else nd, n_prefill=npf, n_tiles=n_tiles,
                       n_logits=rows.size if bucket is None else m,
                       token_ids=d("token_ids"), positions=d("positions"), slot_mapping=d("slot_mapping"),
                       seq_lens=d("seq_lens"), block_tables=d("block_tables").view(-1, W),
                       pages_per_split=d("pages_per_split"), tile_seq=d("tile_seq"), tile_q0=d("tile_q0"),
                       q_start=d("q_start"), q_lens=d("q_lens"), ctx_lens=d("ctx_lens"),
                       prefill_block_tables=d("prefill_block_tables").view(-1, W), logit_map=d("logit_map"))
        if n_cow:
            for li in range(self.model_cfg.n_layers):
                ops.kv_block_copy(self.model.k_cache[li], self.model.v_cache[li], d("cow_src")[:n_cow],
                                  d("cow_dst")[:n_cow])
        return s, bucket

    def _forward(self, s: StepInputs, bucket: Optional[int]) -> torch.Tensor:
        baseline = self.cfg.comm == "nccl" or self.cfg.gemm == "library"
        # baseline path: library GEMMs + NCCL all-reduces; decode buckets are captured in a CUDA graph
        # like the fused path (torch's graph-private pool serves its temporaries)
        fwd = self.model.forward_baseline if baseline else self.model.forward
        if bucket is None:
            return fwd(s)
        g = self.graphs.get(bucket)
        if g is None:
            # warm-up launches outside capture (lazy module init, TMA descriptor cache), then capture
            fwd(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            c0 = ops.launch_count
            with torch.cuda.graph(g):
                fwd(s)
            self.graph_launches[bucket] = ops.launch_count - c0
            self.graphs[bucket] = g
            # the capture did not execute; the warm-up run already produced this step's state
            return self.model.logits[:s.n_logits]
        g.replay()
        ops.launch_count += self.graph_launches[bucket]  # kernels inside the replayed graph
        self.stats["graph_replays"] += 1
        return self.model.logits[:s.n_logits]

    def _step_pp(self, plan, s: StepInputs, n_rows: int) -> np.ndarray:
        """One step of a pipeline stage: receive the residual rows from the previous stage (NCCL
        recv), run this stage's layers, send them on or sample; the sampled ids are broadcast down
        the pipeline column so that every stage's scheduler replica applies the same update."""
        import torch.distributed as dist

        ctx = self.pp
        rpr = s.m // self.world
        hidden = None
        if not ctx.first:
            hidden = self.pp_recv[:rpr]
            dist.recv(hidden, src=ctx.prev_rank)
        out = self.model.forward(s, hidden)
        tok = self.pp_tokens[:max(n_rows, 1)]
        if ctx.last:
            toks = self._sample(plan, out, n_rows)
            if n_rows:
                tok[:n_rows].copy_(torch.from_numpy(np.ascontiguousarray(toks, dtype=np.int32)))
        else:
            dist.send(out.contiguous(), dst=ctx.next_rank)
        dist.broadcast(tok, src=ctx.column_src, group=ctx.column_group)
        return tok[:n_rows].cpu().numpy()

    # ------------------------------------------------------------------ heavy-hitter pruning
    def _h2o_prune(self, plan) -> None:
        """Sequences that outgrew `h2o_budget_blocks` give their least attended middle blocks back to
        the pool (sink and rolling-window blocks always stay). The score of a block is the softmax
        probability mass that this step's query of the last layer put on it, summed over heads: the
        decode attention kernel records it (`DeviceModel.enable_block_mass`), so a step costs one
        all-reduce over the tensor-parallel ranks (which hold different heads) and one device -> host
        read, and only in steps where some sequence is over its budget. Same decision on every rank.
        Reference: the per-block mass accumulated in the decode kernel
        (oxide-backend-cuda/src/kernels/megakernel_ops.cu:577-617)."""
        cfg = self.cfg
        over = []
        for row, rid in enumerate(plan.decode_ids):
            info = self.sched.request_info(int(rid))
            if info is not None and info["phase"] == 2 and len(info["blocks"]) > cfg.h2o_budget_blocks:
                over.append((row, int(rid), info["blocks"]))
        if not over:
            return
        if self.cpu or self.model.block_mass is None:
            mass = None
        else:
            mass = self.model.block_mass[:len(plan.decode_ids)].clone()
            if self.world > 1:
                import torch.distributed as dist

                dist.all_reduce(mass, group=self.group)
            mass = mass.cpu().numpy()
        for row, rid, blocks in over:
            nb = len(blocks)
            scores = [0.0] * nb
            if mass is not None:
                n = min(nb, mass.shape[1])
                scores[:n] = mass[row, :n].tolist()
            keep = self.sched.prune_request(rid, scores, cfg.h2o_sink_blocks, cfg.h2o_rolling_blocks,
                                            cfg.h2o_budget_blocks)
            if keep:
                self.stats["h2o_pruned_blocks"] = self.stats.get("h2o_pruned_blocks", 0) + nb - len(keep)

    def compare_with_baseline(self, n_steps: int = 2) -> dict:
        """Runs `n_steps` decode steps twice from the same state: through the fused path and through
        the library-GEMM + NCCL all-reduce path, and compares the sampled tokens and the logits.
        The fused result is the one the scheduler advances with. Used by bench.py as evidence that
        the fused multi-rank path computes what the plain one does."""
        if self.cpu or self.model.weight_mode != "bf16" or self.model_cfg.is_moe or self.pp is not None:
            return {"steps": 0}
        same = total = 0
        worst = 0.0
        worst_rms, min_cos = 0.0, 1.0
        for _ in range(n_steps):
            plan = self.sched.schedule()
            for e in self.sched.take_events():
                self._deliver(e)
            if plan.n_tokens == 0:
                break
            s, _ = self._fill(plan)
            n_rows = plan.logit_rows.size
            logits = self.model.forward(s)
            ref_fused = logits.clone()
            tok_fused = self._sample(plan, logits, n_rows).copy()
            logits_b = self.model.forward_baseline(s)     # same inputs: the KV append rewrites equal values
            ref_base = logits_b.clone()
            tok_base = self._sample(plan, logits_b, n_rows)
            same += int((tok_fused == tok_base).sum())
            total += int(n_rows)
            scale_ = float(ref_base[:n_rows].abs().max().clamp_min(1e-6))
            worst = max(worst, float((ref_fused[:n_rows] - ref_base[:n_rows]).abs().max()) / scale_)
            # per row over this rank's vocabulary shard: relative RMS difference and cosine of the two logit vectors
            a, b = ref_fused[:n_rows].double(), ref_base[:n_rows].double()
            worst_rms = max(worst_rms, float(((a - b).pow(2).mean(-1).sqrt() / b.pow(2).mean(-1).sqrt().clamp_min(1e-12)).max()))
            min_cos = min(min_cos, float(torch.nn.functional.cosine_similarity(a, b, dim=-1).min()))
            for e in self.sched.update(plan, tok_fused):
                self._deliver(e)
            self.stats["steps"] += 1
            self.stats["decode_tokens"] += plan.n_decode
            self.stats["prefill_tokens"] += plan.prefill_tokens
        return {"steps": n_steps, "tokens_equal": same, "tokens": total, "max_logit_diff_rel": round(worst, 5),
                "max_row_rms_diff_rel": round(worst_rms, 5), "min_row_logit_cosine": round(min_cos, 6)}

    def attach_monitor(self, monitor) -> None:
        """`monitor.check()` (parallel.watchdog.RankMonitor) runs before every step: a peer that
        stopped answering is found on the host, before any kernel waits on it."""
        self.monitor = monitor

    def fail_all(self, reason: str) -> list:
        """Ends every request with `reason` and returns the KV blocks (used when the job degrades)."""
        events = []
        for rid in list(self.requests.keys()):
            ok, ev = self.sched.cancel(rid)
            for e in ev:
                self._deliver(_Event(int(e.req_id), -1, True, reason))
                events.append(e)
        self.degraded = reason
        return events

    def step(self) -> list:
        """One scheduler iteration. Returns the TokenEvents of this step."""
        t0 = time.perf_counter()
        mon = getattr(self, "monitor", None)
        if mon is not None:
            try:
                mon.check()
            except Exception as e:
                self.fail_all(f"rank_failure: {e}")
                raise
        burst = self._burst_plan() if self._burst_k_now() else 0
        plan = self.sched.schedule()
        if getattr(self, "kv_tier", None) is not None:
            self._demote_evicted()
        # requests the scheduler had to end while planning (they can never fit the KV pool)
        early = list(self.sched.take_events())
        for e in early:
            self._deliver(e)
        if plan.n_tokens == 0:
            if early or not self.sched.has_work():
                self._idle_plans = 0
                return early
            # work is queued and nothing was scheduled: one such step can happen around a
            # preemption, a run of them means the loop would spin for ever
            self._idle_plans = getattr(self, "_idle_plans", 0) + 1
            if self._idle_plans >= 4:
                raise EngineError(
                    f"scheduler made no progress for {self._idle_plans} steps with "
                    f"{self.sched.num_running()} running / {self.sched.num_waiting()} waiting requests "
                    f"and {self.sched.num_free_blocks()} free KV blocks")
            return early
        self._idle_plans = 0
        if burst > 1 and plan.n_prefill == 0 and plan.n_decode == self.sched.num_running() and not early \
                and plan.cow_src.size == 0:
            events = early + self._run_burst(plan, burst)
            if time.perf_counter() - t0 > self.cfg.step_deadline_s * burst:
                self.stats["degraded"] = True
            return events
        if self.cpu:
            tokens = self._step_cpu(plan)
        else:
            s, bucket = self._fill(plan)
            n_rows = plan.logit_rows.size
            if self.pp is not None:
                tokens = self._step_pp(plan, s, n_rows)
            else:
                logits = self._forward(s, bucket)
                tokens = self._sample(plan, logits, n_rows)
        events = early + list(self.sched.update(plan, tokens))
        self.stats["steps"] += 1
        self.stats["decode_tokens"] += plan.n_decode
        self.stats["prefill_tokens"] += plan.prefill_tokens
        for e in events[len(early):]:
            self._deliver(e)
        events += self._grammar_follow_up(events[len(early):])
        if self.cfg.h2o_pruning and plan.n_decode:
            self._h2o_prune(plan)
        if self._drafter is not None:
            self._record_acceptance(events[len(early):])
            self._attach_drafts()
        if time.perf_counter() - t0 > self.cfg.step_deadline_s:
            self.stats["degraded"] = True
        return events

    # ------------------------------------------------------------------ KV tiers
    def _kv_caches(self):
        m = self.model
        return (m.pk, m.pv) if self.cpu else (m.k_cache, m.v_cache)

    def _init_kv_tiers(self) -> None:
        """Tier 2 / 3 behind the device block pool: blocks that the prefix cache evicts are copied to
        host memory (and from there to files) keyed by the chained hash of the token prefix they
        complete; a later prompt with that prefix gets them copied back into fresh device blocks
        instead of being prefilled again. Reference: HierarchicalKvCache
        (oxide-alloc/src/hierarchical_kv.rs:27-310: demotion T1->T2->T3 :135-173, promote on hit :207-242)."""
        self.kv_tier = None
        cfg = self.cfg
        if cfg.kv_host_blocks > 0 and cfg.enable_radix and self.pp is None:
            from .kv_tiers import HierarchicalKvCache

            # every rank keeps its own shard of the KV heads: its files must not meet another rank's
            sdir = cfg.kv_storage_dir
            if sdir and self.world > 1:
                sdir = os.path.join(sdir, f"rank{self.rank}")
            self.kv_tier = HierarchicalKvCache(cfg.kv_host_blocks, cfg.kv_storage_blocks, sdir)
            self.sched.record_evictions(True)

    def _demote_evicted(self) -> None:
        """Copies the blocks the prefix cache has just given up to the host tier. Runs right after the
        scheduler planned a step and before the step's kernels are launched, so the copy is ordered
        before anything that may overwrite a block that was handed out again."""
        ev = self.sched.take_evicted()
        if not ev:
            return
        from .kv_tiers import KvBlockPayload, prefix_hashes

        ids = [b for _, _, blocks in ev for b in blocks]
        kc, vc = self._kv_caches()
        idx = torch.as_tensor(ids, dtype=torch.long, device=kc[0].device)
        k = torch.stack([c.index_select(0, idx) for c in kc], dim=1)   # [n, layers, hkv, 16, D]
        v = torch.stack([c.index_select(0, idx) for c in vc], dim=1)
        scales = None
        if self.cfg.kv_host_quant == "q8":
            # int8 codes with one scale per (block, layer, K or V), made where the blocks live: the
            # transfer and the host copy shrink to half of bf16 (reference: QuantizedKvBlock q8,
            # oxide-alloc/src/kv_advanced.rs:39-175, there one scale per tensor)
            def q8(x):
                xf = x.float()
                sc = xf.abs().amax(dim=(2, 3, 4)) / 127.0                   # [n, layers]
                codes = torch.round(xf / sc.clamp_min(1e-30)[:, :, None, None, None]).clamp_(-127, 127).to(torch.int8)
                return codes, sc
            k, ks = q8(k)
            v, vs = q8(v)
            scales = torch.stack([ks, vs], dim=1).cpu().numpy()              # [n, 2, layers]
        elif k.dtype == torch.bfloat16:                                 # carried as 16-bit patterns
            k, v = k.view(torch.int16), v.view(torch.int16)
        k, v = k.cpu().numpy(), v.cpu().numpy()
        self.stats["d2h_bytes"] += k.nbytes + v.nbytes
        i = 0
        for toks, first, blocks in ev:
            hashes = prefix_hashes(toks)
            for j in range(len(blocks)):
                b0 = (first + j) * self.block
                self.kv_tier.demote(KvBlockPayload(hashes[first + j], np.asarray(toks[b0:b0 + self.block], dtype=np.int32),
                                                   k[i], v[i], 0, None if scales is None else scales[i]))
                i += 1
        self.stats["kv_demoted_blocks"] = self.stats.get("kv_demoted_blocks", 0) + len(ids)

    def _promote_prefix(self, toks: np.ndarray) -> None:
        """Before a request is queued: if the host tiers hold blocks of its prompt beyond what the
        device prefix cache has, they go back into device blocks that the cache adopts, and the
        scheduler's own prefix match then finds them."""
        from .kv_tiers import prefix_hashes

        n_full = (int(toks.size) - 1) // self.block          # the last token is always computed
        if n_full <= 0 or not (self.kv_tier.host or self.kv_tier.storage):
            return
        have = int(self.sched.radix_cached_blocks(toks[:n_full * self.block]))
        if have >= n_full:
            return
        hashes = prefix_hashes(toks[:n_full * self.block], self.block)
        found = []
        for i in range(have, n_full):
            p = self.kv_tier.lookup(hashes[i])
            if p is None or not np.array_equal(p.tokens, toks[i * self.block:(i + 1) * self.block]):
                break
            found.append(p)
        if not found:
            return
        n_blocks = have + len(found)
        ids = list(self.sched.radix_adopt(toks[:n_blocks * self.block], n_blocks))
        if len(ids) != len(found):
            return                                            # the pool is short: the prompt is prefilled as usual
        kc, vc = self._kv_caches()
        k = torch.from_numpy(np.stack([p.k for p in found], axis=1))   # [layers, n, hkv, 16, D]
        v = torch.from_numpy(np.stack([p.v for p in found], axis=1))
        if found[0].scales is not None:                                  # int8 codes: expand where the blocks go
            sc = torch.from_numpy(np.stack([p.scales for p in found], axis=0)).to(kc[0].device)   # [n, 2, layers]
            k = (k.to(kc[0].device).float() * sc[:, 0].t()[:, :, None, None, None]).to(kc[0].dtype)
            v = (v.to(kc[0].device).float() * sc[:, 1].t()[:, :, None, None, None]).to(kc[0].dtype)
        elif kc[0].dtype == torch.bfloat16:
            k, v = k.view(torch.bfloat16), v.view(torch.bfloat16)
        k, v = k.to(kc[0].device), v.to(kc[0].device)
        idx = torch.as_tensor(ids, dtype=torch.long, device=kc[0].device)
        for li in range(len(kc)):
            kc[li].index_copy_(0, idx, k[li])
            vc[li].index_copy_(0, idx, v[li])
        self.stats["h2d_bytes"] += 2 * k.numel() * k.element_size()
        self.stats["kv_promoted_blocks"] = self.stats.get("kv_promoted_blocks", 0) + len(ids)

    # ------------------------------------------------------------------ decode bursts
    def _burst_k_now(self) -> bool:
        return bool(getattr(self, "_burst_k", 0)) and not self.cpu

    def _burst_plan(self) -> int:
        """How many decode steps the next plan may run back to back on the device: all running
        requests decode greedily with nothing that needs the host between tokens (grammar, host-side
        samplers, drafts, pruning), nothing waits for admission, and the KV blocks of all those steps
        are held now so that one block table serves them all. 0 or 1: an ordinary step."""
        n_run = self.sched.num_running()
        if not 1 <= n_run <= self.cfg.burst_max_batch or self.sched.num_waiting() != 0:
            return 0
        if self._drafter is not None or self.cfg.h2o_pruning or self.cfg.context_shift or len(self.requests) != n_run:
            return 0
        k = self._burst_k
        for rid, r in self.requests.items():
            if not r.params.is_greedy() or r.grammar is not None or r.host_sampler is not None:
                return 0
            info = self.sched.request_info(int(rid))
            if info is None or info["phase"] != 2:
                return 0
        for rid in self.requests:
            k = min(k, int(self.sched.reserve_ahead(int(rid), k)))
            if k < 2:
                return 0
        return k

    def _burst_body(self, s: StepInputs) -> None:
        logits = self.model.forward(s)
        rows = s.m
        ops.argmax(logits[:rows], self.sampled[:rows], self.sampled_val[:rows])
        ops.advance_decode_step(s, self.sampled, self._mail_dev, self._burst_counter, rows=rows,
                                ring=self._burst_ring)

    def _wait_mail(self, step: int, rows: int, nd: int) -> np.ndarray:
        """Tokens of burst step `step` (device numbering) from the mapped-host ring; bounded wait."""
        base = ((step - 1) % self._burst_ring) * rows
        mail = self._mail_np
        deadline = time.perf_counter() + max(2.0, self.cfg.step_deadline_s)
        spins = 0
        while True:
            words = mail[base:base + nd]
            if bool(np.all((words >> 32) == step)):
                return (words & 0xFFFFFFFF).astype(np.int32)
            spins += 1
            if spins > 2000:
                time.sleep(0)
                if time.perf_counter() > deadline:
                    torch.cuda.synchronize(self.device)
                    self.check_device_status()
                    raise EngineError(f"decode burst: step {step} did not post its tokens in time")

    def _run_burst(self, plan, k: int) -> list:
        """`k` decode steps with one descriptor upload: the graph of a burst step ends with the argmax
        and the in-graph step advance, so the replays run back to back; the host consumes the tokens
        from the mailbox as they land and keeps the scheduler in step (one `schedule()` /
        `update()` pair per token, with the blocks already held). Requests that end inside the burst
        leave the scheduler at once; their rows idle on the device until the burst is over, writing
        only into blocks that nothing else can own before the next launch.
        Reference: advance_decode_step_kernel + the pinned step counter the host spins on
        (oxide-backend-cuda/src/kernels/megakernel_ops.cu:331-357, oxide-backend-cuda/src/lib.rs:4150-4247)."""
        s, bucket = self._fill(plan, extra_len=k)
        rows = s.m
        g = self.burst_graphs.get(bucket)
        done = 0
        if g is None:
            self._burst_body(s)      # eager warm-up: this is burst step 1
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            c0 = ops.launch_count
            with torch.cuda.graph(g):
                self._burst_body(s)
            self.graph_launches[("burst", bucket)] = ops.launch_count - c0
            self.burst_graphs[bucket] = g
            done = 1
        for _ in range(k - done):
            g.replay()
        ops.launch_count += self.graph_launches[("burst", bucket)] * (k - done)
        self.stats["graph_replays"] += k - done
        base = self._burst_steps
        self._burst_steps += k
        row_of = {int(r): i for i, r in enumerate(plan.decode_ids)}
        nd0 = plan.n_decode
        events, cur = [], plan
        for i in range(k):
            toks_all = self._wait_mail(base + i + 1, rows, nd0)
            toks = np.asarray([toks_all[row_of[int(r)]] for r in cur.decode_ids], dtype=np.int32)
            ev = list(self.sched.update(cur, toks))
            self.stats["steps"] += 1
            self.stats["decode_tokens"] += cur.n_decode
            self.stats["burst_steps"] = self.stats.get("burst_steps", 0) + 1
            self.stats["d2h_bytes"] += 8 * cur.n_decode
            for e in ev:
                self._deliver(e)
            events += ev
            if i == k - 1 or not self.sched.has_work():
                break
            cur = self.sched.schedule()
            extra = list(self.sched.take_events())
            for e in extra:
                self._deliver(e)
            events += extra
            if cur.n_prefill or cur.n_decode == 0 or any(int(r) not in row_of for r in cur.decode_ids):
                # cannot happen with nothing waiting; the plan is dropped by ending the burst here
                raise EngineError("decode burst: the scheduler left the decode-only state")
        self.status_host.copy_(ops.status_word(self.device), non_blocking=False)
        if int(self.status_host[0]) != 0:
            self._device_fault(int(self.status_host[0]))
        return events

    # ------------------------------------------------------------------ sampling
    def _sample(self, plan, logits: torch.Tensor, n_rows: int) -> np.ndarray:
        reqs = [self.requests.get(int(r)) for r in plan.logit_req]
        all_greedy = all(r is None or (r.params.is_greedy() and r.grammar is None) for r in reqs)
        n_log = logits.shape[0]
        if self.world > 1:
            logits = self._gather_logits(logits, all_greedy, n_log)
            if logits is None:  # greedy fast path finished on the device
                return self._fetch(n_rows)
        if all_greedy:
            ops.argmax(logits, self.sampled[:n_log], self.sampled_val[:n_log])
            return self._fetch(n_rows)
        st = self.st
        h = st.h
        need_host = []
        mask = None
        for i, r in enumerate(reqs):
            p = r.params if r is not None else SamplingParams(greedy=True)
            h("temperature")[i] = 0.0 if p.is_greedy() else p.temperature
            h("top_k")[i] = p.top_k
            h("top_p")[i] = p.top_p
            h("min_p")[i] = p.min_p
            h("seeds")[i] = p.seed
            h("counters")[i] = r.n_generated if r is not None else 0
            if r is not None and (r.host_sampler is not None):
                need_host.append(i)
            if r is not None and r.grammar is not None:
                if mask is None:
                    words = (self.model_cfg.vocab_size + 31) // 32
                    mask = np.full((n_log, words), -1, dtype=np.int32)
                mask[i] = r.grammar.allow_mask(self.model_cfg.vocab_size)
        for name in ("temperature", "top_k", "top_p", "min_p", "seeds", "counters"):
            o, c, dt = st.off[name]
            nb = n_rows * dt.itemsize
            st.dev[o:o + nb].copy_(st.host[o:o + nb], non_blocking=True)
        mask_t = torch.from_numpy(mask).to(self.device) if mask is not None else None
        ops.sample(logits, self.sampled[:n_log], temperature=st.d("temperature")[:n_log],
                   top_k=st.d("top_k")[:n_log], top_p=st.d("top_p")[:n_log], min_p=st.d("min_p")[:n_log],
                   seeds=st.d("seeds")[:n_log], counters=st.d("counters")[:n_log], allow_mask=mask_t)
        toks = self._fetch(n_rows)
        if need_host:
            rows = logits[need_host].float().cpu().numpy()
            for j, i in enumerate(need_host):
                r = reqs[i]
                hist = self.sched.request_tokens(r.req_id)
                hist = hist[r.prompt_len:] if hist is not None else np.zeros(0, np.int32)
                toks[i] = r.host_sampler.sample(rows[j], hist)
        return toks

    def _gather_logits(self, logits, all_greedy: bool, n_log: int):
        import torch.distributed as dist

        if all_greedy and self.pp is None and os.environ.get("OXB_NCCL_ARGMAX", "0") == "0":
            # every rank pushes its shard's (value, index) into every rank's table over peer memory and
            # combines locally: no library collective in a decode step
            m = self.model
            m.amax_slot ^= 1
            ops.argmax_exchange(logits, self.sampled[:n_log], vocab_start=self.rank * m.v_l,
                                tab_ptrs=m.ws.ptrs("amax"), max_rows=m.max_logits, my_rank=self.rank,
                                slot=m.amax_slot)
            return None
        if all_greedy:
            ops.argmax(logits, self.sampled[:n_log], self.sampled_val[:n_log])
            idx = self.sampled[:n_log] + self.rank * self.model.v_l
            vals = torch.empty(self.world, n_log, dtype=torch.float32, device=self.device)
            idxs = torch.empty(self.world, n_log, dtype=torch.int32, device=self.device)
            dist.all_gather_into_tensor(vals, self.sampled_val[:n_log].contiguous(), group=self.group)
            dist.all_gather_into_tensor(idxs, idx.contiguous(), group=self.group)
            ops.argmax_combine(vals, idxs, self.sampled[:n_log])
            return None
        full = torch.empty(self.world, n_log, self.model.v_l, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(full, logits.contiguous(), group=self.group)
        return full.permute(1, 0, 2).reshape(n_log, -1).contiguous()

    def _fetch(self, n_rows: int) -> np.ndarray:
        self.sampled_host[:n_rows].copy_(self.sampled[:n_rows], non_blocking=True)
        self.status_host.copy_(ops.status_word(self.device), non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        self.stats["d2h_bytes"] += 4 * n_rows + 4
        if int(self.status_host[0]) != 0:
            self._device_fault(int(self.status_host[0]))
        return self.sampled_host[:n_rows].numpy().copy()

    def _device_fault(self, code: int) -> None:
        """A kernel's bounded wait ran out (a peer never arrived) or an index check failed: the
        step's tokens cannot be trusted. Every request ends with a typed reason, all KV blocks go
        back to the pool, the hand-off counters are re-armed and the engine is marked degraded; the
        error is raised to the caller (the context stays usable, new requests may be served)."""
        from ..errors import CollectiveTimeout

        ops.status_word(self.device).zero_()
        if getattr(self, "_burst_k", 0):
            torch.cuda.synchronize(self.device)
            self._burst_counter.zero_()
            self._burst_steps = 0
            self._mail_np[:] = 0
        reason = "collective_timeout" if code == 4 else f"device_error_{code}"
        self.fail_all(reason)
        self.model.reset_sync_state()
        self.stats["degraded"] = True
        self.stats["device_faults"] = self.stats.get("device_faults", 0) + 1
        msg = ops.STATUS_NAMES.get(code, f"code {code}")
        if code == 4:
            raise CollectiveTimeout(f"device wait expired during a step: {msg}")
        raise EngineError(f"kernel reported during a step: {msg}")

    # ------------------------------------------------------------------ events
    def _deliver(self, e) -> None:
        r = self.requests.get(int(e.req_id))
        if r is None:
            return
        now = time.perf_counter()
        if e.token >= 0:
            if r.t_first_token is None:
                r.t_first_token = now
            r.t_last_token = now
            r.n_generated += 1
            r.output.append(int(e.token))
            if r.grammar is not None:
                r.grammar.advance(int(e.token))
        if e.finished:
            r.finished = True
            r.finish_reason = e.reason
        if r.on_token is not None:
            r.on_token(r, e)

    def _grammar_follow_up(self, events: list) -> list:
        """After the tokens of this step: a grammar that reached an accepting state ends its request
        with "stop"; a grammar whose next bytes are forced has them appended without sampling
        (jump-forward, continuous_batching.rs:475,807,1328): the scheduler computes them as one
        prefill chunk in the next step."""
        extra: list = []
        for e in events:
            r = self.requests.get(int(e.req_id))
            if r is None or r.grammar is None or r.finished or e.token < 0:
                continue
            if r.grammar.done():
                ok, _ = self.sched.cancel(r.req_id)
                if ok:
                    ev = _Event(r.req_id, -1, True, "stop")
                    self._deliver(ev)
                    extra.append(ev)
                continue
            forced = self._forced_tokens(r)
            if forced:
                self.stats["jump_forward_tokens"] = self.stats.get("jump_forward_tokens", 0) + len(forced)
                for ev in self.sched.append_forced(r.req_id, forced):
                    self._deliver(ev)
                    extra.append(ev)
        return extra

    def _forced_tokens(self, r: RequestState) -> list:
        """Greedy longest-match tokenisation of the bytes the grammar forces next."""
        lookup = getattr(self, "_bytes_to_token", None)
        if not lookup or not self.cfg.jump_forward:
            return []
        data = r.grammar.jump_forward()
        out = []
        while data:
            for n in range(min(len(data), self._max_token_bytes), 0, -1):
                t = lookup.get(data[:n])
                if t is not None:
                    out.append(t)
                    data = data[n:]
                    break
            else:
                break
        return out

    def _attach_drafts(self) -> None:
        for rid in self.sched.running_ids():
            r = self.requests.get(int(rid))
            if r is None or r.finished or not r.params.is_greedy():
                continue
            hist = self.sched.request_tokens(rid)
            if hist is None:
                continue
            if r.spec is None:
                from .spec_decode import AdaptiveSpeculator

                r.spec = AdaptiveSpeculator(k_min=1, k_max=max(1, self.cfg.draft_tokens))
            # the draft length follows the request's own rolling acceptance rate
            d = self._drafter.propose(hist)[:r.spec.k]
            r.n_drafted = len(d)
            if d:
                self.sched.set_drafts(rid, d)

    def _record_acceptance(self, events) -> None:
        """After a verify step: a request that had n drafts attached and got t tokens back accepted t - 1
        of them (the last token is the model's own choice after the accepted prefix)."""
        got: dict = {}
        for e in events:
            if int(e.token) >= 0:
                got[int(e.req_id)] = got.get(int(e.req_id), 0) + 1
        for rid, n in got.items():
            r = self.requests.get(rid)
            if r is None or r.spec is None or r.n_drafted <= 0:
                continue
            acc = min(max(n - 1, 0), r.n_drafted)
            r.spec.record(r.n_drafted, acc)
            self.stats["spec_proposed"] = self.stats.get("spec_proposed", 0) + r.n_drafted
            self.stats["spec_accepted"] = self.stats.get("spec_accepted", 0) + acc
            r.n_drafted = 0

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: list, params: Optional[SamplingParams] = None, max_steps: int = 1 << 30):
        """Runs the given prompts to completion; returns the generated token lists in order."""
        ids = [self.add_request(p, params) for p in prompts]
        steps = 0
        while self.has_work() and steps < max_steps:
            self.step()
            steps += 1
        return [self.requests[i].output for i in ids]

    def check_device_status(self) -> None:
        if not self.cpu:
            ops.check_status(self.device)

    def close(self) -> None:
        self.graphs.clear()
        if getattr(self, "burst_graphs", None):
            self.burst_graphs.clear()
        if not self.cpu:
            self.model.close()
