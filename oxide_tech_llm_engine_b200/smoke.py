"""One tiny prefill + decode of the flagship Llama path on cuda:0 (driver smoke test)."""
from __future__ import annotations

import numpy as np
import torch


def run_smoke() -> None:
    from . import ops
    from .config import EngineConfig
    from .engine.engine import LLMEngine
    from .models.config import preset
    from .models.weights import SyntheticSource
    from .sampling_params import SamplingParams

    if not torch.cuda.is_available():
        raise RuntimeError("smoke() needs a CUDA device")
    torch.cuda.set_device(0)
    mc = preset("tiny")
    cfg = EngineConfig(model="tiny", max_num_seqs=8, max_num_batched_tokens=256, num_kv_blocks=128,
                       ctx_size=512, graph_buckets=(1, 2, 4, 8))
    eng = LLMEngine(cfg, mc, weights=SyntheticSource(mc, seed=3, std=0.08))
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (5, 37, 70)]
    outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=8, ignore_eos=True))
    torch.cuda.synchronize()
    eng.check_device_status()
    assert all(len(o) == 8 for o in outs), outs
    assert ops.launch_count > 0
    print(f"smoke ok: {ops.launch_count} kernel launches, graph replays {eng.stats['graph_replays']}, "
          f"tokens {outs[0]}")
    eng.close()
