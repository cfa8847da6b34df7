"""Serving workloads of the five benchmark configurations, run through `LLMEngine`.

    python -m oxide_tech_llm_engine_b200.bench_serving --config 1            (CPU plumbing run)
    python -m oxide_tech_llm_engine_b200.bench_serving --config 2 [--weights q4k|fp8]
    torchrun --nproc-per-node N ... -m oxide_tech_llm_engine_b200.bench_serving --config 3|4|5

Config 1: 22-layer 2048-wide Llama as a Q4_0 GGUF (Q8_0 embeddings) on the CPU backend, 300-token prompt,
128 greedy tokens, checked against the fp32 oracle. Config 2: Llama-3-8B shape, 64 requests, prompts
U[128,1024], outputs U[64,512]. Config 3: Llama-3-70B shape TP=N, 256 requests, prompts U[128,4096],
512 outputs. Config 4: Mixtral-8x7B shape EP=N, 128 requests, prompts U[256,2048], 256 outputs.
Config 5: Llama-3-8B TP=N, 64 groups x 16 requests sharing a 2048-token prefix (+128 unique), then
8 prompts of 32768 tokens with 256 outputs.

All requests of a workload arrive at t=0 (closed-loop saturation). Reported per workload: generated
tokens/s over the whole run, p50/p99 time to first token, p50 time per output token, prefix-hit rate,
prefill tokens/s, and for the long prompts the attention TFLOP/s implied by the prefill time share.
Times are host wall clock around `engine.step()` (each step ends with the D2H read of the sampled ids);
multi-GPU values are the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

import numpy as np


def _pct(xs, q):
    return float(np.percentile(np.asarray(xs, dtype=np.float64), q)) if len(xs) else None


def run_workload(eng, prompts, out_lens, *, greedy=True, label=""):
    from .sampling_params import SamplingParams

    t0 = time.perf_counter()
    ids = []
    for p, n in zip(prompts, out_lens):
        ids.append(eng.add_request(p, SamplingParams(greedy=greedy, max_tokens=int(n), ignore_eos=True)))
    pre0 = eng.stats["prefill_tokens"]
    steps = 0
    while eng.has_work():
        eng.step()
        steps += 1
    wall = time.perf_counter() - t0
    reqs = [eng.requests[i] for i in ids]
    ttft = [r.t_first_token - t0 for r in reqs if r.t_first_token is not None]
    tpot = [(r.t_last_token - r.t_first_token) / (r.n_generated - 1) for r in reqs
            if r.n_generated > 1 and r.t_first_token is not None]
    gen = sum(r.n_generated for r in reqs)
    out = {"workload": label, "requests": len(reqs), "generated_tokens": gen, "wall_s": round(wall, 3),
           "tokens_per_s": round(gen / wall, 1), "steps": steps,
           "ttft_p50_ms": round(_pct(ttft, 50) * 1e3, 2), "ttft_p99_ms": round(_pct(ttft, 99) * 1e3, 2),
           "tpot_p50_ms": round(_pct(tpot, 50) * 1e3, 3) if tpot else None,
           "prefill_tokens": int(eng.stats["prefill_tokens"] - pre0)}
    # Prefill arithmetic of the whole job (all ranks), when every prompt token was computed (no prefix hits):
    # causal attention 4 * D * Hq * L^2 / 2 per layer and prompt, projections 2 * active parameters per token.
    # Divided by the time until the last first token, which also contains the decode steps that were
    # interleaved with the prefill chunks: a lower bound of the sustained prefill rate.
    mc = getattr(eng, "model_cfg", None)
    lens = [len(p) for p in prompts]
    if mc is not None and ttft and out["prefill_tokens"] == sum(lens):
        attn = sum(2.0 * mc.head_dim * mc.n_heads * mc.n_layers * float(n) * n for n in lens)
        proj = 2.0 * mc.active_params() * sum(lens)
        t_pre = max(ttft)
        out["prompt_attention_tflop"] = round(attn / 1e12, 2)
        out["prefill_attention_tflops_lower_bound"] = round(attn / 1e12 / t_pre, 1)
        out["prefill_model_tflops_lower_bound"] = round((attn + proj) / 1e12 / t_pre, 1)
    return out


def config1(args) -> dict:
    import torch

    from .config import EngineConfig
    from .engine.engine import LLMEngine
    from .models.config import preset
    from .models.reference import ReferenceModel
    from .models.weights import open_weights, write_synthetic_gguf
    from .sampling_params import SamplingParams

    mc = preset("tinyllama-1.1b")
    if args.layers:
        mc.n_layers = args.layers
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, mc.vocab_size, size=args.prompt_len or 300).tolist()
    n_out = args.output_len or 128
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        t0 = time.perf_counter()
        write_synthetic_gguf(path, mc, seed=1, weight_type="Q4_0", embed_type="Q8_0", std=0.02)
        t_write = time.perf_counter() - t0
        t0 = time.perf_counter()
        src = open_weights(path)
        eng = LLMEngine(EngineConfig(model=path, backend="cpu", max_num_seqs=1, ctx_size=512, num_kv_blocks=64,
                                     enable_radix=False), src.cfg, weights=src)
        t_load = time.perf_counter() - t0
        t0 = time.perf_counter()
        out = eng.generate([prompt], SamplingParams(greedy=True, max_tokens=n_out, ignore_eos=True))[0]
        t_gen = time.perf_counter() - t0
        # fp32 oracle over the same dequantised weights, teacher-forced on the engine's tokens
        ref = ReferenceModel(src.cfg, src)
        logits = ref.forward(prompt + out[:-1], all_logits=True)[len(prompt) - 1:]
        gaps = [float((logits[i].max() - logits[i][t]) / logits[i].std()) for i, t in enumerate(out)]
        eng.close()
    return {"config": 1, "model": f"{mc.name} Q4_0 GGUF ({mc.n_layers}L)", "backend": "cpu", "prompt_len": len(prompt),
            "generated": len(out), "tokens_per_s": round(len(out) / t_gen, 2), "gguf_write_s": round(t_write, 1),
            "load_s": round(t_load, 2), "oracle_exact_match": round(float(np.mean(np.asarray(gaps) == 0)), 3),
            "oracle_max_gap_sigma": round(max(gaps), 4), "threads": torch.get_num_threads()}


def gpu_config(args) -> dict:
    import torch
    import torch.distributed as dist

    from .config import EngineConfig
    from .engine.engine import LLMEngine
    from .models.config import preset

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    c = args.config
    model = {2: "llama3-8b", 3: "llama3-70b", 4: "mixtral-8x7b", 5: "llama3-8b"}[c]
    mc = preset(model)
    if args.layers:
        mc.n_layers = args.layers
    rng = np.random.default_rng(7)
    scale = args.scale
    workloads = []
    if c == 2:
        n = max(1, int(64 * scale))
        workloads.append(("64 req, prompts U[128,1024], outputs U[64,512]",
                          [rng.integers(0, mc.vocab_size, size=int(rng.integers(128, 1025))).tolist() for _ in range(n)],
                          rng.integers(64, 513, size=n).tolist()))
        ctx, seqs = 1024 + 512 + 16, n
    elif c == 3:
        n = max(1, int(256 * scale))
        workloads.append(("256 req, prompts U[128,4096], 512 outputs",
                          [rng.integers(0, mc.vocab_size, size=int(rng.integers(128, 4097))).tolist() for _ in range(n)],
                          [args.output_len or 512] * n))
        ctx, seqs = 4096 + 512 + 16, n
    elif c == 4:
        n = max(1, int(128 * scale))
        workloads.append(("128 req, prompts U[256,2048], 256 outputs",
                          [rng.integers(0, mc.vocab_size, size=int(rng.integers(256, 2049))).tolist() for _ in range(n)],
                          [args.output_len or 256] * n))
        ctx, seqs = 2048 + 256 + 16, n
    else:
        groups, per = max(1, int(64 * scale)), 16
        prefixes = [rng.integers(0, mc.vocab_size, size=2048).tolist() for _ in range(groups)]
        ps = []
        for j in range(per):            # interleaved across groups
            for g in range(groups):
                ps.append(prefixes[g] + rng.integers(0, mc.vocab_size, size=128).tolist())
        workloads.append((f"{groups} groups x {per} requests, 2048-token shared prefix + 128 unique", ps,
                          [args.output_len or 32] * len(ps)))
        n_long = max(1, int(8 * scale))
        workloads.append((f"{n_long} prompts of 32768 tokens, 256 outputs",
                          [rng.integers(0, mc.vocab_size, size=32768).tolist() for _ in range(n_long)],
                          [256] * n_long))
        ctx, seqs = 32768 + 256 + 16, 256
    wm = {"bf16": "bf16", "fp8": "fp8", "q4k": "quant", "q4km": "quant", "nvfp4": "nvfp4"}[args.weights]
    cfg = EngineConfig(model=model, tp=world, ctx_size=ctx, max_num_seqs=min(seqs, 256),
                       max_num_batched_tokens=args.max_batched_tokens, gpu_memory_utilization=0.92,
                       sla_budget=False, chunk_max=args.max_batched_tokens, enable_radix=(c == 5),
                       weight_mode=wm, cuda_graph=True, decode_burst=args.burst, burst_max_batch=8,
                       quant_dense_copy=args.dense_copy,
                       graph_buckets=tuple(b for b in (1, 8, 16, 32, 64, 128, 192, 256) if b <= max(min(seqs, 256), 1)) or (8,))
    eng = LLMEngine(cfg, mc, rank=rank, world=world, device=dev, random_init=True,
                    **({"random_quant_type": {"q4k": "Q4_K", "q4km": "Q4_K_M"}[args.weights]}
                       if args.weights in ("q4k", "q4km") else {}))
    results = []
    for label, prompts, outs in workloads:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        r = run_workload(eng, prompts, outs, label=label)
        if c == 5:
            st = eng.sched.radix_stats()
            r["prefix_hit_rate"] = round(st["hit_tokens"] / max(st["lookup_tokens"], 1), 4)
            r["prefix_hit_tokens"] = int(st["hit_tokens"])
        if "32768" in label:
            # causal attention FLOPs of the prompts: 4 * D * Hq * T^2 / 2 per layer
            T = 32768
            fl = len(prompts) * mc.n_layers * 4 * mc.head_dim * mc.n_heads * T * T / 2
            r["prefill_attention_tflop_total"] = round(fl / 1e12, 1)
            r["note"] = "attention TFLOP/s in isolation: see bench_kernels --prefill (profiles/prefill_tc_*.md)"
        vals = torch.tensor([r["wall_s"], r["ttft_p50_ms"], r["ttft_p99_ms"], r["tpot_p50_ms"] or 0.0],
                            dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            r["wall_s"], r["ttft_p50_ms"], r["ttft_p99_ms"] = [round(float(v), 3) for v in vals[:3]]
            r["tpot_p50_ms"] = round(float(vals[3]), 3)
            r["tokens_per_s"] = round(r["generated_tokens"] / r["wall_s"], 1)
        results.append(r)
    eng.check_device_status()
    out = {"config": c, "model": f"{mc.name} ({mc.n_layers}L)", "weights": args.weights, "n_gpus": world,
           "parallelism": ("ep" if mc.is_moe else "tp") + str(world), "kv_blocks": eng.model.num_blocks,
           "data": "synthetic random tokens, random-init weights", "workloads": results}
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out if rank == 0 else {}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, required=True, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--dense-copy", default="auto", choices=["auto", "on", "off"],
                    help="packed GGUF weights: keep a bf16 copy for steps with more than 8 rows (off: the GEMM unpacks the blocks itself)")
    ap.add_argument("--burst", type=int, default=0,
                    help="decode steps per host round trip for small greedy batches (in-graph step advance)")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "fp8", "q4k", "q4km", "nvfp4"])
    ap.add_argument("--scale", type=float, default=1.0, help="fraction of the request count (quick runs)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (marks the run as reduced)")
    ap.add_argument("--prompt-len", type=int, default=0)
    ap.add_argument("--output-len", type=int, default=0)
    ap.add_argument("--max-batched-tokens", type=int, default=8192)
    args = ap.parse_args()
    out = config1(args) if args.config == 1 else gpu_config(args)
    if out:
        out["reduced"] = bool(args.layers or args.scale != 1.0 or args.output_len or args.prompt_len)
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    main()
