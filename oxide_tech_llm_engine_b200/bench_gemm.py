"""Micro-benchmark of the tcgen05 GEMM over tile / split / epilogue choices.

    python -m oxide_tech_llm_engine_b200.bench_gemm --m 256 --n 7168 --k 8192 --epi 3

Each configuration is timed with CUDA events over `--iters` launches, with a buffer larger than
L2 written between launches so that weights come from HBM, and reported as microseconds,
weight-stream GB/s and TFLOP/s next to the measured peaks of this machine.
"""
from __future__ import annotations

import argparse
import itertools
import json

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=256)
    ap.add_argument("--n", type=int, default=7168)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--epi", type=int, default=0)
    ap.add_argument("--bn", default="64,128,256")
    ap.add_argument("--splits", default="1")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--tiled", default="0", help="comma list of 0/1: weights stored tile-major")
    ap.add_argument("--mt", default="1", help="comma list of 1/2: 128-row halves per tile (2 = all 256 rows with one CTA)")
    ap.add_argument("--graph", action="store_true", help="time a CUDA-graph replay of the launch (no host launch path in the number)")
    ap.add_argument("--trace", action="store_true", help="print the per-CTA timeline (medians over CTAs, microseconds from kernel entry)")
    ap.add_argument("--narrow-boxes", action="store_true", help="mt = 2: two 16 KB TMA boxes per operand and stage instead of one 32 KB box")
    ap.add_argument("--auto", action="store_true", help="time the (bn, mt, splits) that ops.pick_decode_cfg chooses")
    ap.add_argument("--nvfp4", action="store_true", help="time the NVFP4 block-scaled GEMM (and its activation quantiser)")
    ap.add_argument("--packed", default="", help="GGUF block type (Q4_K, Q6_K, Q8_0, Q4_0): time the GEMM that unpacks the weights in the kernel")
    ap.add_argument("--fp8", action="store_true", help="time the block-scaled fp8 GEMM (and its activation quantiser)")
    args = ap.parse_args()
    from . import ops
    from .utils.roofline import load_measured_peaks

    peaks = load_measured_peaks()
    dev = torch.device("cuda", 0)
    a = torch.randn(args.m, args.k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16) * 0.02
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    n_out = args.n // 2 if args.epi == ops.EPI_SWIGLU_BF16 else args.n
    out_bf = torch.empty(args.m, n_out, device=dev, dtype=torch.bfloat16)
    out_f32 = torch.zeros(args.m, args.n, device=dev, dtype=torch.float32)
    flops = 2.0 * args.m * args.n * args.k
    wbytes = 2.0 * args.n * args.k
    w_tiled = ops.tile_weight(w)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.iters):
            if not args.no_flush:
                flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    if args.fp8:
        w8, sw = ops.quant_weight_fp8_block(w)
        a8, sa = ops.quant_act_fp8(a)
        out8 = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)

        us = timed(lambda: ops.gemm_fp8_block(a8, sa, w8, sw, out=out8))
        uq = timed(lambda: ops.quant_act_fp8(a, a8, sa))
        ops.check_status()
        print(json.dumps({"kernel": "gemm_fp8_block", "m": args.m, "n": args.n, "k": args.k, "us": round(us, 2),
                          "weights_gb_s": round(wbytes / 2 / us / 1e3, 1), "tflops": round(flops / us / 1e6, 1),
                          "frac_hbm_of_measured": round(wbytes / 2 / us / 1e3 / peaks["hbm_gbs"], 3),
                          "x_bf16_peak_of_measured": round(flops / us / 1e6 / peaks["bf16_tflops"], 3),
                          "quant_act_us": round(uq, 2)}), flush=True)
        return
    if args.nvfp4:
        # NVFP4 x NVFP4 (block scales of 16, e4m3) on the fp4 tensor-core path; the activation quantiser apart
        wq = ops.Nvfp4Weight.from_float(w.float())
        aq, sfa, ags = ops.quant_act_nvfp4(a)
        out4 = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
        us = timed(lambda: ops.gemm(aq, wq.q, out=out4, sfa=sfa, sfb=wq.sf, a_gscale=ags, w_gscale=wq.gscale))
        uq = timed(lambda: ops.quant_act_nvfp4(a))
        ops.check_status()
        print(json.dumps({"kernel": "gemm nvfp4 (kind::mxf4nvf4.block_scale)", "m": args.m, "n": args.n, "k": args.k,
                          "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                          "weights_gb_s": round(wbytes / 4 / us / 1e3, 1),
                          "x_bf16_peak_of_measured": round(flops / us / 1e6 / peaks["bf16_tflops"], 3),
                          "quant_act_us": round(uq, 2)}), flush=True)
        return
    if args.packed:
        # bf16 activations x GGUF-packed weights unpacked inside the GEMM, against the same GEMM on a bf16 copy
        from .models.llama import random_quant_linear

        gen = torch.Generator(device=dev)
        gen.manual_seed(0)
        lin = random_quant_linear(args.packed, args.n, args.k, dev, gen)
        mt = 2 if args.m > 128 else 1
        sp = max(1, min(ops.sm_count(dev) // (-(-args.n // 128) * -(-args.m // (128 * mt))), args.k // 256, 16))
        us = timed(lambda: ops.gemm_packed(a, lin.code, lin.w, args.n, out_f32, epi=ops.EPI_RED_F32, mt=mt, splits=sp))
        ud = timed(lambda: ops.gemm(a, w, epi=ops.EPI_RED_F32, dst_ptrs=[out_f32.data_ptr()], bn=128, mt=mt, splits=sp))
        ops.check_status()
        print(json.dumps({"kernel": f"gemm_packed {args.packed}", "m": args.m, "n": args.n, "k": args.k, "mt": mt,
                          "splits": sp, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                          "us_same_gemm_on_bf16_weights": round(ud, 2),
                          "weights_gb_s": round(lin.w.numel() / us / 1e3, 1)}), flush=True)
        return
    combos = list(itertools.product([int(x) for x in args.bn.split(",")], [int(x) for x in args.splits.split(",")],
                                    [int(x) for x in args.tiled.split(",")], [int(x) for x in args.mt.split(",")]))
    if args.auto:
        bn, mt, sp = ops.pick_decode_cfg(args.m, args.n, args.k, swiglu=args.epi == ops.EPI_SWIGLU_BF16,
                                         sms=ops.sm_count(dev))
        combos = [(bn, sp, int(args.tiled.split(",")[0]), mt)]
    for bn, sp, stag, mt in combos:
        if args.epi == ops.EPI_SWIGLU_BF16 and args.n % bn:
            continue
        tiles = -(-args.n // bn) * -(-args.m // (128 * mt))
        if sp > 1 and args.epi != ops.EPI_RED_F32 and tiles * sp > ops.sm_count(dev):
            continue
        kw = dict(bn=bn, splits=sp, mt=mt, wide_boxes=not args.narrow_boxes)
        ww = w_tiled if stag else w
        if args.epi == ops.EPI_RED_F32:
            kw.update(epi=ops.EPI_RED_F32, dst_ptrs=[out_f32.data_ptr()])
        elif args.epi == ops.EPI_STORE_F32:
            kw.update(epi=ops.EPI_STORE_F32, out=out_f32)
        else:
            kw.update(epi=args.epi, out=out_bf)
        trace = torch.zeros(8 * ops.sm_count(dev), dtype=torch.int64, device=dev) if args.trace else None
        if trace is not None:
            kw["trace"] = trace
        for _ in range(3):
            ops.gemm(a, ww, **kw)
        torch.cuda.synchronize()
        launch = lambda: ops.gemm(a, ww, **kw)
        if args.graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                ops.gemm(a, ww, **kw)
            launch = g.replay
        ts = []
        for _ in range(args.iters):
            if not args.no_flush:
                flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            launch()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        ops.check_status()
        ts.sort()
        us = ts[len(ts) // 2]
        if trace is not None:
            t = trace.view(-1, 8).cpu().numpy().astype("int64")
            t = t[t[:, 0] > 0]
            t0 = t[:, 0].min()
            names = ["entry", "acc_ready", "partial_stored", "splits_met", "epilogue_done", "exit"]
            med = {n: round(float(__import__("numpy").median(t[:, i][t[:, i] > 0] - t0)) / 1e3, 2) if (t[:, i] > 0).any() else None
                   for i, n in enumerate(names)}
            mx = {n: round(float((t[:, i][t[:, i] > 0] - t0).max()) / 1e3, 2) if (t[:, i] > 0).any() else None
                  for i, n in enumerate(names)}
            print(json.dumps({"trace_us_median": med, "trace_us_max": mx, "ctas": int(t.shape[0])}), flush=True)
        print(json.dumps({"m": args.m, "n": args.n, "k": args.k, "epi": args.epi, "bn": bn, "mt": mt, "splits": sp,
                          "tiled": stag, "us": round(us, 2), "weights_gb_s": round(wbytes / us / 1e3, 1),
                          "tflops": round(flops / us / 1e6, 1),
                          "frac_hbm_of_measured": round(wbytes / us / 1e3 / peaks["hbm_gbs"], 3),
                          "frac_tflops_of_measured": round(flops / us / 1e6 / peaks["bf16_tflops"], 3)}), flush=True)


if __name__ == "__main__":
    main()
