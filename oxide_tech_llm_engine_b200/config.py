"""Engine configuration: one dataclass filled from CLI flags (the reference's names) and from
`OXB_*` environment variables, printed at start-up.

Reference parity: clap flag set of oxide-cli/src/lib.rs:203-216,359-515 and the scheduler
constants ChunkedPrefillConfig{32, 512, 2048, 25000us, 2000us, 25us/token}
(oxide-engine/src/continuous_batching.rs:88-99), TOKENS_PER_PAGE = 16 (oxide-alloc/src/paged_kv.rs:12),
graph buckets {1..128} (oxide-backend-cuda/src/lib.rs:3356-3365), env flags OXIDE_CUDA_GRAPH,
OXIDE_H2O_PRUNING, OXIDE_H2O_BUDGET (cuda lib.rs:378-399).
"""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Optional


@dataclass
class EngineConfig:
    model: str = "tiny"                 # preset name or path to a .gguf / safetensors checkpoint
    alias: Optional[str] = None
    models_dir: Optional[str] = None
    weight_mode: str = "auto"           # auto | bf16 | quant | fp8  (quant: GGUF blocks packed in HBM; fp8: 128x128 block-scaled e4m3)
    tp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1
    cp: int = 1
    ctx_size: int = 8192                # -c / --ctx-size: per-sequence context limit
    max_num_seqs: int = 64              # --max-slots
    max_num_batched_tokens: int = 2048
    num_kv_blocks: int = 0              # 0 = size from free memory
    gpu_memory_utilization: float = 0.90
    chunk_min: int = 32
    chunk_max: int = 512
    sla_itl_us: float = 25000.0
    base_us: float = 2000.0
    per_token_us: float = 25.0
    sla_budget: bool = True
    enable_radix: bool = True
    kv_host_blocks: int = 0             # > 0: blocks the prefix cache evicts are kept in host memory (tier 2) and promoted back on a hit
    kv_storage_blocks: int = 0          # ... and from there to files under kv_storage_dir (tier 3)
    kv_storage_dir: Optional[str] = None
    kv_host_quant: str = "none"         # none | q8: demoted blocks are kept as int8 codes with one scale per layer and tensor
    cuda_graph: bool = True
    graph_buckets: tuple = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    max_splits: int = 16
    comm: str = "fused"                 # fused | nccl  (nccl + library GEMMs is the baseline path)
    gemm: str = "tcgen05"               # tcgen05 | library
    speculative: str = "off"            # off | ngram | auto
    draft_tokens: int = 5
    jump_forward: bool = True           # grammar-forced bytes are appended without sampling
    quant_dense_copy: str = "auto"    # auto | on | off: keep a bf16 copy of packed weights for steps with > 8 rows
    h2o_pruning: bool = False
    h2o_budget_blocks: int = 128        # blocks a sequence may keep (sink + rolling window + heavy hitters)
    h2o_sink_blocks: int = 1
    h2o_rolling_blocks: int = 16
    context_shift: bool = False         # at the context limit keep the prefix and drop the oldest tokens instead of ending
    shift_keep_tokens: int = 4
    shift_step_tokens: int = 256
    decode_burst: int = 0               # > 1: greedy decode-only batches run this many steps per host round trip (in-graph step advance + pinned mailbox)
    burst_max_batch: int = 8            # ... when at most this many sequences are decoding and nothing waits
    native_worker: bool = False         # run engine steps on the C++ StepWorker thread (core pin: worker_pin_core)
    worker_pin_core: int = -1
    seed: int = 42
    backend: str = "cuda"               # cuda | cpu
    step_deadline_s: float = 30.0       # watchdog: a step that takes longer marks the engine degraded

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    @classmethod
    def from_env(cls, **overrides) -> "EngineConfig":
        """Defaults <- OXB_* / OXIDE_* environment <- explicit overrides."""
        kw: dict[str, Any] = {}
        for f in fields(cls):
            env = os.environ.get("OXB_" + f.name.upper())
            if env is None:
                continue
            if f.type in ("int", int):
                kw[f.name] = int(env)
            elif f.type in ("float", float):
                kw[f.name] = float(env)
            elif f.type in ("bool", bool):
                kw[f.name] = env not in ("0", "false", "False", "")
            elif f.name == "graph_buckets":
                kw[f.name] = tuple(int(x) for x in env.split(","))
            else:
                kw[f.name] = env
        if "OXIDE_CUDA_GRAPH" in os.environ:
            kw["cuda_graph"] = os.environ["OXIDE_CUDA_GRAPH"] not in ("0", "false")
        if "OXIDE_H2O_PRUNING" in os.environ:
            kw["h2o_pruning"] = os.environ["OXIDE_H2O_PRUNING"] not in ("0", "false")
        if "OXIDE_H2O_BUDGET" in os.environ:
            kw["h2o_budget_blocks"] = int(os.environ["OXIDE_H2O_BUDGET"])
        kw.update({k: v for k, v in overrides.items() if v is not None})
        return cls(**kw)

    def describe(self) -> str:
        return "EngineConfig(" + ", ".join(f"{k}={v}" for k, v in self.to_dict().items()) + ")"
