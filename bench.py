#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of continuous-batching serving, Llama-3-70B shape, TP = N.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)

Workload (the tensor-parallel serving configuration): 256 requests with random-token prompts of
uniform length in [128, 4096] and 512 output tokens, random-init bf16 weights, paged KV with
16-token blocks. The engine admits as many requests as the KV pool holds, prefills them (untimed),
then W warm-up and exactly K timed decode steps run through `LLMEngine.step()`: scheduler ->
pinned-host H2D of the step descriptor -> forward -> device sampler -> D2H of the sampled ids.
`value` is tokens/s from CUDA-event device time of the K steps (max over ranks); `e2e.value` is the
same K steps by wall clock through the public API. Weights (>= 17 GB per GPU) are far larger than
L2, so nothing is served from cache between steps.

Around the timed region, untimed: an open-loop phase (a few requests arriving as a Poisson process
at a stated rate on the idle engine: p50 / p99 time to first token without queueing behind 255
other prompts), and a check of the fused path against the library-GEMM + NCCL all-reduce path on
the same state (`tokens_match_baseline`).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = ("reference is a Rust workspace: no cargo/rustc in this image, pip finds no "
                         "Python project in it, and it has no multi-GPU / TP code path")


def reference_arm() -> None:
    print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="oxb_clocks_", suffix=".csv")
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx.append(float(p[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=4096)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--max-batched-tokens", type=int, default=8192)
    ap.add_argument("--mem-util", type=float, default=0.96,
                    help="fraction of the free device memory the engine may plan with (weights + KV pool + activations); "
                         "0.96 leaves about 7 GB of a B200 unplanned at the 70B single-GPU shape")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "fp8", "q4k", "q4km"],
                    help="fp8: block-scaled e4m3 projections (1x128 / 128x128 scales); a separate configuration, "
                         "the headline number is bf16")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="nccl: comparison path with library GEMMs and NCCL all-reduces")
    ap.add_argument("--open-loop", type=int, default=12, help="requests of the open-loop TTFT phase (0 = skip)")
    ap.add_argument("--check-steps", type=int, default=2, help="decode steps compared against the baseline path (0 = skip)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from oxide_tech_llm_engine_b200 import ops
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset(args.model)
    valid = True
    if args.layers:
        mc.n_layers = args.layers
        valid = False
    ctx = args.prompt_max + args.output_len + 16
    cfg = EngineConfig(model=args.model, tp=world, ctx_size=ctx, max_num_seqs=args.requests,
                       max_num_batched_tokens=args.max_batched_tokens, gpu_memory_utilization=args.mem_util,
                       sla_budget=False, chunk_max=args.max_batched_tokens, enable_radix=False,
                       cuda_graph=not args.no_graph, comm=args.comm, weight_mode={"q4k": "quant", "q4km": "quant"}.get(args.weights, args.weights), gemm="library" if args.comm == "nccl" else "tcgen05",
                       graph_buckets=tuple(b for b in (8, 16, 32, 64, 128, 192, 256) if b <= args.requests) or (args.requests,))
    t_build = time.perf_counter()
    eng = LLMEngine(cfg, mc, rank=rank, world=world, device=dev, random_init=True,
                    random_quant_type={"q4k": "Q4_K", "q4km": "Q4_K_M"}.get(args.weights))
    torch.cuda.synchronize()
    rng = np.random.default_rng(1234)  # same request stream on every rank
    sp = SamplingParams(greedy=True, max_tokens=args.output_len, ignore_eos=True)

    # ---- untimed: open-loop time to first token on the idle engine ----
    # Poisson arrivals at `rate` requests/s (same seeded schedule on every rank; arrival times are
    # compared with rank 0's clock, broadcast each iteration, so every rank admits the same requests
    # before the same step). Each request decodes 4 tokens and leaves.
    open_loop = None
    if args.open_loop > 0:
        rate = min(4.0, 0.5 * world)
        gaps = rng.exponential(1.0 / rate, size=args.open_loop)
        arrivals = np.cumsum(gaps)
        prompts = [rng.integers(0, mc.vocab_size, size=int(rng.integers(args.prompt_min, args.prompt_max + 1)),
                                dtype=np.int64).tolist() for _ in range(args.open_loop)]
        sp_ol = SamplingParams(greedy=True, max_tokens=4, ignore_eos=True)
        clock = torch.zeros(1, dtype=torch.float64, device=dev)
        t_start = time.perf_counter()
        nxt, ids, sched_at = 0, [], {}
        while nxt < args.open_loop or eng.has_work():
            now = time.perf_counter() - t_start
            if world > 1:
                clock[0] = now
                dist.broadcast(clock, src=0)
                now = float(clock[0])
            while nxt < args.open_loop and arrivals[nxt] <= now:
                rid = eng.add_request(prompts[nxt], sp_ol)
                sched_at[rid] = arrivals[nxt]
                ids.append(rid)
                nxt += 1
            if eng.has_work():
                eng.step()
            else:
                time.sleep(min(0.002, max(0.0, arrivals[nxt] - now)))
        # TTFT against the scheduled arrival time (includes the wait for the step in flight)
        ol = sorted((eng.requests[r].t_first_token - t_start - sched_at[r]) * 1e3 for r in ids
                    if eng.requests[r].t_first_token is not None)
        open_loop = {"requests": len(ol), "rate_req_per_s": rate,
                     "ttft_p50_ms": round(ol[len(ol) // 2], 1) if ol else None,
                     "ttft_p99_ms": round(ol[min(len(ol) - 1, int(len(ol) * 0.99))], 1) if ol else None}
        for r in ids:
            eng.requests.pop(r, None)
        eng.stats["prefill_tokens"] = 0
        eng.stats["decode_tokens"] = 0

    t_submit = time.perf_counter()
    for _ in range(args.requests):
        n = int(rng.integers(args.prompt_min, args.prompt_max + 1))
        eng.add_request(rng.integers(0, mc.vocab_size, size=n, dtype=np.int64).tolist(), sp)
    # ---- untimed: prefill until every admitted request is decoding ----
    t_prefill = time.perf_counter()
    prefill_steps = 0
    while True:
        before = eng.stats["prefill_tokens"]
        eng.step()
        prefill_steps += 1
        if eng.stats["prefill_tokens"] == before:
            break
        if prefill_steps > 100000:
            raise SystemExit("prefill did not converge")
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t_prefill
    prefill_tokens = eng.stats["prefill_tokens"]
    for _ in range(args.warmup):
        eng.step()
    eng.check_device_status()
    # ---- untimed: the fused path against library GEMMs + NCCL all-reduces on the same state ----
    check = eng.compare_with_baseline(args.check_steps) if (args.check_steps > 0 and args.comm == "fused") else {"steps": 0}
    torch.cuda.empty_cache()
    for _ in range(2):
        eng.step()  # back to steady state (the comparison ran its steps outside the graphs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    batch_sizes = []
    h2d0, d2h0, launches0 = eng.stats["h2d_bytes"], eng.stats["d2h_bytes"], ops.launch_count
    barrier()
    if sampler:
        sampler.start()
    t0 = time.perf_counter()
    for i in range(args.steps):
        ev[i][0].record()
        events = eng.step()
        ev[i][1].record()
        batch_sizes.append(len(events))
    barrier()
    wall = time.perf_counter() - t0
    whole_wall = time.perf_counter() - t_submit
    clocks = sampler.stop() if sampler else {}
    eng.check_device_status()
    # latency view of the same run: time to first token of every admitted request (all arrive at
    # t=0, so it includes queueing behind the other prompts) and time per output token
    reqs = [r for r in eng.requests.values() if r.t_first_token is not None]
    ttft = sorted((r.t_first_token - r.t_arrival) * 1e3 for r in reqs)
    dev_ms = sum(a.elapsed_time(b) for a, b in ev)
    tokens = sum(batch_sizes)
    t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = float(t[0]), float(t[1])
    launches = ops.launch_count - launches0
    if rank == 0:
        value = tokens / (dev_ms / 1e3)
        e2e = tokens / (wall_ms / 1e3)
        out = {
            "metric": "decode tokens/sec (box, max over ranks)",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": {"bf16": "bf16", "fp8": "fp8 block-scaled weights, bf16 activations/KV",
                      "q4k": "GGUF Q4_K packed weights, bf16 activations/KV",
                      "q4km": "GGUF Q4_K_M layout (Q4_K + Q6_K) packed weights, bf16 activations/KV"}[args.weights],
            "data": "synthetic random-token prompts, random-init N(0,0.02) weights",
            "impl": "ours" if args.comm == "fused" else "ours-baseline-path", "valid": valid,
            "config": {
                "model": f"{mc.name} ({mc.n_layers}L d{mc.d_model} {mc.n_heads}q/{mc.n_kv_heads}kv ffn{mc.ffn_dim} v{mc.vocab_size})",
                "parallelism": f"tp{world}", "requests_submitted": args.requests,
                "concurrent_decoding": int(statistics.median(batch_sizes)) if batch_sizes else 0,
                "global_batch": int(statistics.median(batch_sizes)) if batch_sizes else 0,
                "prompt_len": f"uniform[{args.prompt_min},{args.prompt_max}]", "output_len": args.output_len,
                "seq_len": ctx, "kv_blocks": eng.model.num_blocks, "kv_block_tokens": 16,
                "mem_free_gb_end": round(torch.cuda.mem_get_info(dev)[0] / 2**30, 2),
                "mem_peak_reserved_gb": round(torch.cuda.max_memory_reserved(dev) / 2**30, 2),
                "cache_note": "per-step inputs (weights + KV, >= 17 GB per GPU) exceed the 126 MB L2",
                "cuda_graph": cfg.cuda_graph, "comm": ("nccl all-reduce + library GEMMs (baseline path)" if args.comm == "nccl" else
                         "fused peer-memory kernels" if world > 1 else "single GPU"),
                "prefill_tokens": int(prefill_tokens), "prefill_seconds": round(prefill_s, 2),
                "prefill_tok_per_s": round(prefill_tokens / max(prefill_s, 1e-9), 1),
                "build_seconds": round(t_prefill - t_build, 2),
                "ttft_p50_ms": round(ttft[len(ttft) // 2], 1) if ttft else None,
                "ttft_p99_ms": round(ttft[min(len(ttft) - 1, int(len(ttft) * 0.99))], 1) if ttft else None,
                "tpot_p50_ms": round(statistics.median(a.elapsed_time(b) for a, b in ev), 3),
                "ttft_note": "ttft_p50/p99 above are closed-loop: all requests arrive at t=0 and queue behind each other",
                "open_loop": open_loop,
                # from the first submission to the end of the timed steps: prefill, warm-up, the baseline check and decode
                "whole_run": {"wall_s": round(whole_wall, 2), "prompt_tokens": int(prefill_tokens),
                              "generated_tokens": int(sum(r.n_generated for r in eng.requests.values())),
                              "generated_tok_per_s": round(sum(r.n_generated for r in eng.requests.values()) / whole_wall, 1)},
                "tokens_match_baseline": (f"{check['tokens_equal']}/{check['tokens']}" if check.get("tokens") else None),
                "baseline_check": check,
            },
            "clocks": clocks,
            "e2e": {"value": round(e2e, 2), "unit": "tokens/s", "ms_per_step": round(wall_ms / args.steps, 4),
                    "h2d_bytes_per_step": int((eng.stats["h2d_bytes"] - h2d0) / args.steps),
                    "d2h_bytes_per_step": int((eng.stats["d2h_bytes"] - d2h0) / args.steps)},
            "gpu_launches": int(launches),
        }
        conc = out["config"]["concurrent_decoding"]
        if conc < args.requests:
            out["n1_note"] = (f"the KV pool beside the weights holds {conc} of the {args.requests} requests at once on "
                              f"{world} GPU(s); runs on more GPUs decode all {args.requests} together, so throughput ratios "
                              f"against this run compare different batch sizes")
        print(json.dumps(out), flush=True)
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
