"""Micro-benchmark of the small-batch weight-streaming kernels: the quantised GEMV (`ops.mmvq`, with
and without int8 activations) and the bf16 GEMV (`ops.gemv`).

    python -m oxide_tech_llm_engine_b200.bench_gemv [--rows 1,4,8] [--iters 10]

Shapes are the projections of a Llama-3-8B layer plus its LM head. Every launch is timed with CUDA
events after a 256 MB write that evicts L2, and reported as microseconds and GB/s of weight bytes.
"""
from __future__ import annotations

import argparse
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="1,4,8")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="", help="substring filter on the case name")
    args = ap.parse_args()
    from . import ops
    from .models.llama import random_quant_linear
    from .utils.roofline import load_measured_peaks

    peaks = load_measured_peaks()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    cases = [("Q4_K", 6144, 4096), ("Q4_K", 4096, 4096), ("Q4_K", 28672, 4096), ("Q4_K", 4096, 14336),
             ("Q8_0", 128256, 4096), ("Q6_K", 4096, 14336), ("Q6_K", 128256, 4096), ("Q4_0", 4096, 4096),
             ("mixed Q4_K|Q4_K|Q6_K", 6144, 4096), ("bf16", 6144, 4096), ("bf16", 28672, 4096), ("bf16", 4096, 14336)]
    for typ, N, K in cases:
        name = f"{typ} N={N} K={K}"
        if args.only and args.only not in name:
            continue
        for M in [int(r) for r in args.rows.split(",")]:
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            y = torch.empty(M, N, device=dev, dtype=torch.float32)
            if typ == "bf16":
                w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
                wt = ops.tile_weight(w)
                us = timed(lambda: ops.gemv(x, wt, y))
                wbytes = w.numel() * 2
                row = {"kernel": "gemv_bf16 (tile-major weights)"}
            elif typ.startswith("mixed"):
                # Q | K | V of an 8B model in a Q4_K_M file: one launch over three matrices of two types
                lins = [random_quant_linear(t, n, K, dev, g) for t, n in (("Q4_K", 4096), ("Q4_K", 1024), ("Q6_K", 1024))]
                parts = [(l.code, l.w, l.n) for l in lins]
                xq = ops.quant_q8_1(x)
                us = timed(lambda: ops.mmvq_mixed(parts, x, y, k=K, xq=xq))

                def three():
                    o = 0
                    for l in lins:
                        ops.mmvq(l.code, l.w, x, y[:, o:o + l.n], n=l.n, k=K, xq=xq)
                        o += l.n
                us_f = timed(three)
                wbytes = sum(l.w.numel() for l in lins)
                row = {"kernel": "mmvq_mixed (one launch)", "us_three_launches": round(us_f, 2)}
            else:
                lin = random_quant_linear(typ, N, K, dev, g)
                xq = ops.quant_q8_1(x)
                us = timed(lambda: ops.mmvq(lin.code, lin.w, x, y, n=N, k=K, xq=xq))
                us_f = timed(lambda: ops.mmvq(lin.code, lin.w, x, y, n=N, k=K))
                wbytes = lin.w.numel()
                row = {"kernel": "mmvq int8 activations (dp4a)", "us_fp32_activations": round(us_f, 2)}
            row.update({"case": name, "rows": M, "us": round(us, 2), "weights_gb_s": round(wbytes / us / 1e3, 1),
                        "frac_hbm_of_measured": round(wbytes / us / 1e3 / peaks["hbm_gbs"], 3)})
            print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
