"""Worker of the multi-GPU tests (launched under torchrun, one rank per GPU): runs the tiny dense
and MoE models tensor/expert parallel through the fused peer-memory path and checks the tokens
against the fp32 oracle on rank 0."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    from _util import assert_consistent
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ok = True
    for name in sys.argv[1:] or ["tiny", "tiny-moe", "tiny-fp8", "tiny-h2o", "tiny-b160", "tiny-moe-fp4"]:
        fp4 = name.endswith("-fp4")    # expert matrices on the block-scaled fp4 path, experts sharded over the ranks
        if fp4:
            name_base = name[:-4]
        fp8 = name.endswith("-fp8")
        h2o = name.endswith("-h2o")
        big = name.endswith("-b160")   # 160 sequences decode together: the 256-row GEMM tiles with in-kernel split-K
        base = name[:-4] if (fp8 or h2o or fp4) else (name[:-5] if big else name)
        if fp4:
            mc = preset(base, n_heads=8, n_kv_heads=8, d_model=256, ffn_dim=512, head_dim=64)
        elif big:
            mc = preset(base, n_heads=8, n_kv_heads=8, d_model=512, ffn_dim=1024, head_dim=64)
        elif world > 2:
            mc = preset(base, n_heads=8, n_kv_heads=8, d_model=256, ffn_dim=512, head_dim=64)
        elif fp8:
            mc = preset(base, d_model=256, ffn_dim=512, head_dim=64)
        else:
            mc = preset(base)
        src = SyntheticSource(mc, seed=3, std=0.08)
        cfg = EngineConfig(tp=world, max_num_seqs=192 if big else 8, max_num_batched_tokens=2048 if big else 256,
                           num_kv_blocks=1024 if big else 256, sla_budget=not big,
                           ctx_size=1024, graph_buckets=(192,) if big else (8,), cuda_graph=True,
                           weight_mode="fp8" if fp8 else ("nvfp4" if fp4 else "auto"),
                           **(dict(h2o_pruning=True, h2o_budget_blocks=5, h2o_sink_blocks=1, h2o_rolling_blocks=2,
                                   enable_radix=False) if h2o else {}))
        eng = LLMEngine(cfg, mc, weights=src, rank=rank, world=world, device=dev)
        rng = np.random.default_rng(1)
        lens = rng.integers(3, 24, size=160).tolist() if big else (4, 33, 100, 17)
        prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in lens]
        outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=6 if big else 12, ignore_eos=True))
        torch.cuda.synchronize()
        eng.check_device_status()
        gathered = [None] * world
        dist.all_gather_object(gathered, outs)
        if rank == 0:
            same = all(g == outs for g in gathered)
            try:
                assert same, "ranks disagree on the generated tokens"
                if h2o:   # pruned KV: only agreement between ranks, completion and the pruning itself are checked
                    assert all(len(o) == 12 for o in outs) and eng.stats.get("h2o_pruned_blocks", 0) > 0
                else:
                    assert_consistent(mc, src, prompts, outs, **(dict(tol=0.6, min_exact=0.5) if fp8 else
                                                                 dict(tol=2.0, min_exact=0.4) if fp4 else {}))
                if big:
                    assert eng.stats["graph_replays"] >= 3, "the 160-row decode steps did not run as graph replays"
                print(f"TP_CHECK {name} world={world} OK replays={eng.stats['graph_replays']}", flush=True)
            except AssertionError as e:
                ok = False
                print(f"TP_CHECK {name} world={world} FAIL {e} {outs}", flush=True)
        eng.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and not ok:
        sys.exit(1)


if __name__ == "__main__":
    main()
