"""Worker of the pipeline-parallel GPU test (torchrun, one rank per GPU): pp stages x tp ranks of the
tiny model, hidden rows handed over by NCCL send/recv, tokens checked against the fp32 oracle."""
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
    from oxide_tech_llm_engine_b200.parallel.pipeline import build_pp_context
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    pp = int(sys.argv[1]) if len(sys.argv) > 1 else 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = build_pp_context(rank, world, pp)
    mc = preset("tiny", n_layers=5)
    src = SyntheticSource(mc, seed=3, std=0.08)
    cfg = EngineConfig(tp=ctx.tp, pp=pp, max_num_seqs=8, max_num_batched_tokens=256, num_kv_blocks=256,
                       ctx_size=1024, cuda_graph=False, enable_radix=False)
    eng = LLMEngine(cfg, mc, weights=src, rank=ctx.tp_rank, world=ctx.tp, group=ctx.tp_group, device=dev, pp=ctx)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (4, 33, 100, 17)]
    outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=12, ignore_eos=True))
    torch.cuda.synchronize()
    eng.check_device_status()
    gathered = [None] * world
    dist.all_gather_object(gathered, outs)
    ok = True
    if rank == 0:
        try:
            assert all(g == outs for g in gathered), "stages disagree on the generated tokens"
            assert_consistent(mc, src, prompts, outs)
            assert len(eng.model.layers) == 3 and eng.model.pp_first and not eng.model.pp_last
            print(f"PP_CHECK pp={pp} tp={ctx.tp} OK", flush=True)
        except AssertionError as e:
            ok = False
            print(f"PP_CHECK FAIL {e} {outs}", flush=True)
    eng.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and not ok:
        sys.exit(1)


if __name__ == "__main__":
    main()
