"""Per-kernel time breakdown of one decode (or prefill) step of the device model.

    python -m oxide_tech_llm_engine_b200.bench_kernels --model llama3-70b --shard-of 8 --layers 8 \
        --batch 256 --ctx-min 128 --ctx-max 4608 --breakdown

Builds the model of one rank (``--shard-of N`` gives the per-rank shapes of an N-way tensor-parallel
run on a single GPU, without the peers), fills the paged KV pool with random data, and times
``DeviceModel.forward`` with CUDA events. ``--breakdown`` wraps every kernel front-end in
``ops`` with its own event pair and prints the share of each kernel (per GEMM shape), which is
what the launch list of a profiler would give, without a profiler.

Reference parity: the `bench_kernels` binary (oxide-cli/src/bin/bench_kernels.rs:412-486), which
times each kernel with a stream synchronise and prints a per-op microsecond table.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict
from dataclasses import replace

import numpy as np
import torch


def shard_config(mc, n: int):
    """Per-rank shapes of an n-way TP/EP shard, expressed as a stand-alone tp=1 model."""
    if n <= 1:
        return mc
    kw = dict(n_heads=mc.n_heads // n, n_kv_heads=max(mc.n_kv_heads // n, 1), vocab_size=mc.vocab_size // n)
    if mc.is_moe:
        kw["n_experts"] = mc.n_experts // n
        kw["n_experts_used"] = min(mc.n_experts_used, kw["n_experts"])
    else:
        kw["ffn_dim"] = mc.ffn_dim // n
    return replace(mc, **kw)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-70b")
    ap.add_argument("--shard-of", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--ctx-min", type=int, default=128)
    ap.add_argument("--ctx-max", type=int, default=4608)
    ap.add_argument("--prefill", type=int, default=0, help="time a prefill step of this many tokens instead")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--breakdown", action="store_true")
    ap.add_argument("--trace", action="store_true", help="kernel table from torch.profiler (CUPTI) over the timed steps")
    ap.add_argument("--max-splits", type=int, default=16)
    ap.add_argument("--pps", type=int, default=0, help="pages per KV split (0 = engine heuristic)")
    ap.add_argument("--no-attn", action="store_true",
                    help="skip the attention kernels: times the GEMM / collective / norm chain only")
    args = ap.parse_args()

    from . import ops
    from .models.config import preset
    from .models.llama import DeviceModel, StepInputs

    import os

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    mc = shard_config(preset(args.model), args.shard_of)
    if args.layers:
        mc = replace(mc, n_layers=args.layers)
    rng = np.random.default_rng(0)
    B = args.batch
    if args.prefill:
        n_seq = max(1, args.prefill // 2048)
        q_lens = [args.prefill // n_seq] * n_seq
        ctx = list(q_lens)
        M = sum(q_lens)
    else:
        ctx = rng.integers(args.ctx_min, args.ctx_max + 1, size=B).tolist()
        M = B
    blocks_per_seq = [(c + 15) // 16 for c in ctx]
    num_blocks = sum(blocks_per_seq) + 8
    W = max(blocks_per_seq)
    model = DeviceModel(mc, rank=rank, world=world, device=dev, max_tokens=max(M, 64), max_seqs=max(len(ctx), 8),
                        num_blocks=num_blocks, max_blocks_per_seq=W, max_logits=max(len(ctx), 64),
                        max_splits=args.max_splits)
    model.init_random(0)
    if args.no_attn:
        model._attention = lambda s, li: None
    for li in range(mc.n_layers):
        model.k_cache[li].normal_()
        model.v_cache[li].normal_()
    bt = np.zeros((len(ctx), W), dtype=np.int32)
    nxt = 0
    for i, nb in enumerate(blocks_per_seq):
        bt[i, :nb] = np.arange(nxt, nxt + nb)
        nxt += nb
    ti = lambda a, dt=torch.int32: torch.as_tensor(np.asarray(a), dtype=dt, device=dev)
    if args.prefill:
        q_start = np.cumsum([0] + q_lens[:-1])
        pos = np.concatenate([np.arange(q) for q in q_lens])
        slots = np.concatenate([bt[i, np.arange(q) // 16] * 16 + np.arange(q) % 16 for i, q in enumerate(q_lens)])
        tile_seq, tile_q0 = [], []
        for s, q in enumerate(q_lens):
            for q0 in range(0, q, 128):
                tile_seq.append(s)
                tile_q0.append(q0)
        lmap = np.full(M, -1, dtype=np.int32)
        lmap[q_start + np.asarray(q_lens) - 1] = np.arange(len(q_lens))
        s_in = StepInputs(m=M, n_decode=0, n_prefill=len(q_lens), n_tiles=len(tile_seq), n_logits=len(q_lens),
                          token_ids=ti(rng.integers(0, mc.vocab_size, size=M)), positions=ti(pos),
                          slot_mapping=ti(slots, torch.int64), seq_lens=ti([0]), block_tables=ti(bt),
                          pages_per_split=ti([4]), tile_seq=ti(tile_seq), tile_q0=ti(tile_q0), q_start=ti(q_start),
                          q_lens=ti(q_lens), ctx_lens=ti(ctx), prefill_block_tables=ti(bt), logit_map=ti(lmap))
    else:
        pos = np.asarray(ctx) - 1
        slots = bt[np.arange(B), pos // 16].astype(np.int64) * 16 + pos % 16
        pages = (max(ctx) + 15) // 16
        if args.pps:
            pps = args.pps
        else:
            per_sm = 12 if model.hkv >= 4 else 4   # the engine's rule (engine/engine.py, _fill)
            want = -(-per_sm * model._sms // max(1, B * model.hkv))
            splits = max(1, min(args.max_splits, want))
            pps = (max(4, -(-pages // splits)) + 3) // 4 * 4
        s_in = StepInputs(m=M, n_decode=B, n_prefill=0, n_tiles=0, n_logits=B,
                          token_ids=ti(rng.integers(0, mc.vocab_size, size=M)), positions=ti(pos),
                          slot_mapping=ti(slots, torch.int64), seq_lens=ti(ctx), block_tables=ti(bt),
                          pages_per_split=ti([pps]), logit_map=ti(np.arange(M)))

    times: dict[str, list[float]] = defaultdict(list)
    if args.breakdown:
        def wrap(name, fn, keyf=None):
            def inner(*a, **k):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                r = fn(*a, **k)
                e.record()
                key = name + (keyf(*a, **k) if keyf else "")
                times[key].append((s, e))
                return r
            return inner
        ops.gemm = wrap("gemm", ops.gemm, lambda a, w, **k: f"[M{a.shape[-2]} N{w.shape[-2]} K{w.shape[-1]} epi{k.get('epi', 0)} bn{k.get('bn', 0)} s{k.get('splits', 1)}]")
        for n in ("paged_decode", "paged_prefill", "finalize_norm", "qkv_rope_append", "embed_gather", "swiglu"):
            setattr(ops, n, wrap(n, getattr(ops, n)))

    for _ in range(args.warmup):
        model.forward(s_in)
    torch.cuda.synchronize()
    ops.check_status()
    times.clear()
    graph = None
    if args.graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            model.forward(s_in)
        times.clear()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    prof = None
    if args.trace:
        from torch.profiler import ProfilerActivity, profile

        prof = profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU])
        prof.__enter__()
    for a, b in ev:
        a.record()
        if graph is not None:
            graph.replay()
        else:
            model.forward(s_in)
        b.record()
    torch.cuda.synchronize()
    if prof is not None:
        prof.__exit__(None, None, None)
    if prof is not None and rank == 0:
        agg = defaultdict(lambda: [0.0, 0])
        for e in prof.events():
            if e.device_type is not None and str(e.device_type).endswith("CUDA") and e.name and "Memcpy" not in e.name:
                agg[e.name[:90]][0] += e.device_time if hasattr(e, "device_time") else e.cuda_time
                agg[e.name[:90]][1] += 1
        tot = sum(v[0] for v in agg.values())
        print(f"{'us/step':>10} {'calls':>6} {'avg us':>8} {'share':>7}  kernel (in-situ durations, profiler attached)")
        for k, v in sorted(agg.items(), key=lambda kv: -kv[1][0]):
            print(f"{v[0] / args.steps:10.2f} {v[1] // args.steps:6d} {v[0] / max(v[1], 1):8.2f} {100 * v[0] / max(tot, 1e-9):6.1f}%  {k}")
        print(f"{tot / args.steps:10.2f} us of kernel time per step")
        evs = sorted((e for e in prof.events() if e.device_type is not None and str(e.device_type).endswith("CUDA")
                      and e.name and "Memcpy" not in e.name), key=lambda e: e.time_range.start)
        per_step = len(evs) // args.steps
        print("launch sequence of the last step (us):")
        for e in evs[-per_step:][: 4 + 2 * 12]:
            dur = e.device_time if hasattr(e, "device_time") else e.cuda_time
            print(f"  {dur:8.2f}  {e.name.split('(')[0][-48:]}")
    ops.check_status()
    ms = sorted(a.elapsed_time(b) for a, b in ev)
    med = ms[len(ms) // 2]
    if world > 1:
        t = torch.tensor([med, ms[0]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every multi-GPU number is the max over ranks
        med, ms[0] = float(t[0]), float(t[1])
    out = {"model": mc.name, "shard_of": args.shard_of, "tp": world, "layers": mc.n_layers, "rows": M,
           "mean_ctx": float(np.mean(ctx)), "ms_per_step_median": round(med, 4), "ms_min": round(ms[0], 4),
           "graph": bool(args.graph), "attention": not args.no_attn}
    if args.no_attn and not mc.is_moe:
        # roofline of the fused GEMM + collective chain: per GEMM the slower of FLOPs / measured
        # sustained GEMM peak and NVLink bytes / measured 770 GB/s per direction
        from .utils.roofline import load_measured_peaks

        pk = load_measured_peaks()
        peak = pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) * 1e12
        link = 770e9
        tp, d = world, mc.d_model
        qd, kvd, ff = mc.q_dim // tp, mc.kv_dim // tp, mc.ffn_dim // tp
        frac = (tp - 1) / tp
        terms = {
            "ag_gemm_qkv": (2.0 * M * (qd + 2 * kvd) * d / peak, M * d * 2 * frac / link),
            "gemm_rs_o": (2.0 * M * d * qd / peak, M * d * 2 * frac / link),
            "ag_gemm_gate_up": (2.0 * M * 2 * ff * d / peak, M * d * 2 * frac / link),
            "gemm_rs_down": (2.0 * M * d * ff / peak, M * d * 2 * frac / link),
        }
        ideal_ms = mc.n_layers * sum(max(c, l) for c, l in terms.values()) * 1e3
        out["roofline"] = {"ideal_ms": round(ideal_ms, 4), "achieved_over_roofline": round(ideal_ms / med, 3),
                           "peaks": f"{peak / 1e12:.0f} TFLOP/s sustained ({pk.get('source', 'measured')}), 770 GB/s NVLink per direction",
                           "per_layer_us": {k: {"compute": round(c * 1e6, 2), "link": round(l * 1e6, 2)}
                                            for k, (c, l) in terms.items()}}
    if rank == 0:
        print(json.dumps(out))
    if rank != 0:
        args.breakdown = args.trace = False
    if args.breakdown and graph is None:
        rows = []
        for k, v in times.items():
            tot = sum(s.elapsed_time(e) for s, e in v)
            rows.append((tot / args.steps, len(v) // args.steps, k))
        total = sum(r[0] for r in rows)
        print(f"{'ms/step':>10} {'calls':>6} {'share':>7}  kernel")
        for t, c, k in sorted(rows, reverse=True):
            print(f"{t:10.4f} {c:6d} {100 * t / total:6.1f}%  {k}")
        print(f"{total:10.4f} total of event-timed kernels")
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

