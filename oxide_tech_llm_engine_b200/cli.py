"""Command line front-end with the reference's flag names.

    oxide [-m MODEL] [-p PROMPT] [-n N] ...        one-shot generation or interactive chat (-i)
    oxide chat  ...                                 REPL with /model /models /list /info /help /exit
    oxide server --host H --port P ...              OpenAI-compatible HTTP server
    oxide bench ...                                 decode loop -> roofline receipt (JSON)
    oxide verify / roofline / quantize ...          16 greedy tokens / copy-bandwidth probe / GGUF re-quantiser

Reference parity: Cli / Commands of oxide-cli/src/lib.rs:203-216,359-515,542-670 (flags -m/--model,
--alias, --models-dir, -c/--ctx-size, -ngl, -b/--backend, --max-slots, -p, -n, -t, -i, --temp,
--top-p, --min-p, --repeat-penalty, --repeat-last-n, --top-k, --seed, --greedy, --speculative,
--draft-tokens, --system, --chat-format, --continuous-batching), `-ngl` / `-md` single-dash
normalisation (:672-701), REPL commands (:1097-1135), aux binaries oxide-bench, oxide-verify,
oxide-roofline, oxide-quantize (oxide-cli/src/bin/*.rs). Only the `cuda` and `cpu` backends exist
here; `img`, `lab` and `gpu-unlock` are recognised and refused.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Optional

from .config import EngineConfig
from .errors import ConfigError, EngineError

BACKENDS_ACCEPTED = ("cuda", "cpu", "auto")
BACKENDS_KNOWN = ("rocm", "metal", "tpu", "intel", "qualcomm", "rknn", "hailo", "vulkan", "opencl", "hybrid")


def normalize_argv(argv: list[str]) -> list[str]:
    """llama.cpp-style single-dash long flags: -ngl N -> --n-gpu-layers N, -md M -> --draft-model M."""
    out = []
    for a in argv:
        if a == "-ngl":
            out.append("--n-gpu-layers")
        elif a.startswith("-ngl="):
            out += ["--n-gpu-layers", a.split("=", 1)[1]]
        elif a == "-md":
            out.append("--draft-model")
        elif a == "--cb":
            out.append("--continuous-batching")
        else:
            out.append(a)
    return out


def add_common(p: argparse.ArgumentParser) -> None:
    p.add_argument("-m", "--model", default=os.environ.get("OXIDE_MODEL", "tiny"))
    p.add_argument("--alias")
    p.add_argument("--models-dir")
    p.add_argument("-c", "--ctx-size", type=int, default=8192)
    p.add_argument("--n-gpu-layers", type=int, default=-1)
    p.add_argument("-b", "--backend", default="auto")
    p.add_argument("--weights", default="auto", choices=["auto", "bf16", "quant", "fp8"])
    p.add_argument("--max-slots", type=int, default=64)
    p.add_argument("--gpu", type=int, default=0)
    p.add_argument("-p", "--prompt")
    p.add_argument("-n", "--max-tokens", type=int, default=512)
    p.add_argument("-t", "--threads", type=int, default=8)
    p.add_argument("-i", "--interactive", action="store_true")
    p.add_argument("--kv-device-blocks", type=int, default=0)
    p.add_argument("--kv-host-blocks", type=int, default=8192)
    p.add_argument("--kv-storage-blocks", type=int, default=32768)
    p.add_argument("--kv-storage-dir", default=None, help="directory of the file tier behind the host KV tier (none: host tier only)")
    p.add_argument("--kv-host-quant", default="none", choices=["none", "q8"], help="keep demoted KV blocks as int8 codes")
    p.add_argument("--decode-burst", type=int, default=0, help="decode steps per host round trip for small greedy batches")
    p.add_argument("--temp", type=float, default=0.7)
    p.add_argument("--top-p", type=float, default=0.95)
    p.add_argument("--min-p", type=float, default=0.05)
    p.add_argument("--repeat-penalty", type=float, default=1.1)
    p.add_argument("--repeat-last-n", type=int, default=64)
    p.add_argument("--top-k", type=int, default=40)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--greedy", action="store_true")
    p.add_argument("--speculative", default="auto")
    p.add_argument("--draft-tokens", type=int, default=5)
    p.add_argument("--draft-model")
    p.add_argument("--system")
    p.add_argument("--chat-format", default="auto")
    p.add_argument("--continuous-batching", action="store_true")
    p.add_argument("--tp", type=int, default=1, help="tensor / expert parallel ranks (one process per GPU, started through torch.distributed.run)")
    p.add_argument("--dp", type=int, default=1, help="data-parallel engine replicas behind one front (tp = 1: one GPU each, in this process)")
    p.add_argument("--max-batched-tokens", type=int, default=2048)
    p.add_argument("--no-cuda-graph", action="store_true")
    p.add_argument("--no-radix", action="store_true")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="oxide", description="B200-native Oxide LLM engine")
    add_common(ap)
    ap.add_argument("--serve", action="store_true")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    sub = ap.add_subparsers(dest="command")
    c = sub.add_parser("chat")
    add_common(c)
    s = sub.add_parser("server")
    add_common(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8080)
    b = sub.add_parser("bench")
    add_common(b)
    b.add_argument("--steps", type=int, default=64)
    b.add_argument("--batch", type=int, default=1)
    b.add_argument("--prompt-len", type=int, default=128)
    b.add_argument("--assert-mbu-min", type=float, default=0.0)
    v = sub.add_parser("verify")
    add_common(v)
    r = sub.add_parser("roofline")
    r.add_argument("--gpu", type=int, default=0)
    r.add_argument("--mib", type=int, default=1024)
    q = sub.add_parser("quantize")
    q.add_argument("input")
    q.add_argument("output")
    q.add_argument("--type", default="Q4_K")
    q.add_argument("--embed-type", default="Q8_0")
    for name in ("img", "lab", "gpu-unlock"):
        sub.add_parser(name)
    return ap


def parse_args(argv: Optional[list[str]] = None) -> argparse.Namespace:
    argv = normalize_argv(list(sys.argv[1:] if argv is None else argv))
    args = build_parser().parse_args(argv)
    be = (args.backend if hasattr(args, "backend") else "auto").lower()
    if be in BACKENDS_KNOWN:
        raise ConfigError(f"backend {be!r} is not built in this engine (only cuda and cpu)")
    if be not in BACKENDS_ACCEPTED:
        raise ConfigError(f"unknown backend {be!r}")
    return args


def engine_config_from_args(args) -> EngineConfig:
    import torch

    be = args.backend.lower()
    if be == "auto":
        be = "cuda" if torch.cuda.is_available() else "cpu"
    spec = args.speculative
    if spec == "auto":
        spec = "ngram" if args.greedy else "off"
    return EngineConfig.from_env(
        model=args.model, alias=args.alias, models_dir=args.models_dir, ctx_size=args.ctx_size,
        max_num_seqs=args.max_slots, num_kv_blocks=args.kv_device_blocks, seed=args.seed, backend=be,
        weight_mode=args.weights, speculative=spec, draft_tokens=args.draft_tokens, tp=args.tp, dp=args.dp,
        max_num_batched_tokens=args.max_batched_tokens, cuda_graph=not args.no_cuda_graph,
        enable_radix=not args.no_radix, kv_host_blocks=args.kv_host_blocks, kv_storage_blocks=args.kv_storage_blocks,
        kv_storage_dir=args.kv_storage_dir, kv_host_quant=args.kv_host_quant, decode_burst=args.decode_burst)


def sampling_from_args(args):
    from .sampling_params import SamplingParams

    return SamplingParams(temperature=0.0 if args.greedy else args.temp, top_k=args.top_k, top_p=args.top_p,
                          min_p=args.min_p, repeat_penalty=args.repeat_penalty, repeat_last_n=args.repeat_last_n,
                          seed=args.seed, max_tokens=args.max_tokens, greedy=args.greedy)


class Job:
    """What this process is in a multi-rank serving job (`--tp N` under torch.distributed.run):
    rank, world, the NCCL (or gloo, CPU backend) group of the engine ranks, the gloo control group
    that carries the commands, the job store and this rank's heartbeat."""

    def __init__(self, backend: str):
        import torch
        import torch.distributed as dist

        from .parallel import front
        from .parallel.watchdog import Heartbeat

        self.rank, self.world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if backend == "cuda":
            torch.cuda.set_device(self.local)
            self.device = torch.device("cuda", self.local)
            dist.init_process_group("nccl", device_id=self.device)
        else:
            self.device = torch.device("cpu")
            dist.init_process_group("gloo")
        self.group = dist.group.WORLD
        self.ctl = front.make_control_group()
        self.store = front.job_store()
        self.heartbeat = Heartbeat(self.store, self.rank, period_s=0.2).start()

    def close(self) -> None:
        import torch.distributed as dist

        self.heartbeat.stop()
        if dist.is_initialized():
            dist.destroy_process_group()


_job: Optional[Job] = None


def load_model(name: str, path: Optional[str], cfg: EngineConfig):
    """Builds engine + tokenizer + handle for a checkpoint path or a catalog preset. In a
    multi-rank job (see `Job`) every rank builds its shard; rank 0 gets the handle that broadcasts
    commands, the others get a plain handle-less record and run `front.follower_loop`. With
    `dp > 1` (and tp = 1) one engine per GPU is built in this process behind a `DpHandle`."""
    from .engine.engine import LLMEngine
    from .engine.handle import EngineHandle
    from .engine.model_manager import LoadedModel
    from .models.config import preset
    from .models.weights import SyntheticSource, open_weights
    from .tokenizer import Tokenizer

    if path is not None:
        src = open_weights(path)
        mc = src.cfg
        tok = None
        if hasattr(src, "file") and "tokenizer.ggml.tokens" in src.file.metadata:
            tok = Tokenizer.from_gguf(src.file)
    else:
        mc = preset(name)
        src = SyntheticSource(mc, seed=cfg.seed)
        tok = None
    if tok is None:
        tok = Tokenizer.ascii_fallback(mc.vocab_size)
    if _job is not None:
        from .parallel.front import DistributedEngineHandle
        from .parallel.watchdog import RankMonitor

        if getattr(_job, "model_loaded", False):
            raise ConfigError("a multi-rank job serves the model it was started with (no hot swap: the "
                              "follower ranks only follow rank 0's request stream)")
        _job.model_loaded = True

        eng = LLMEngine(cfg, mc, weights=src, rank=_job.rank, world=1 if cfg.backend == "cpu" else _job.world,
                        group=_job.group, device=_job.device if cfg.backend != "cpu" else None)
        eng.set_tokenizer(tok)
        if _job.rank != 0:
            return LoadedModel(name, path, None, tok, mc), eng
        monitor = RankMonitor(_job.store, 0, _job.world, timeout_s=5.0)
        handle = DistributedEngineHandle(eng, _job.ctl, _job.world, monitor=monitor, heartbeat=_job.heartbeat,
                                         store=_job.store)
        return LoadedModel(name, path, handle, tok, mc)
    if cfg.dp > 1:
        import torch

        from .parallel.dp_router import DpHandle

        if cfg.tp != 1:
            raise ConfigError("--dp replicas are built for tp = 1 (one GPU per replica in this process)")
        import dataclasses
        import os

        handles = []
        for i in range(cfg.dp):
            # every replica keeps its own KV file tier (same prefixes, different block pools and lifetimes)
            rcfg = cfg if not cfg.kv_storage_dir else dataclasses.replace(
                cfg, kv_storage_dir=os.path.join(cfg.kv_storage_dir, f"replica{i}"))
            if cfg.backend == "cpu":
                eng = LLMEngine(rcfg, mc, weights=src)
            else:
                if i >= torch.cuda.device_count():
                    raise ConfigError(f"--dp {cfg.dp} needs {cfg.dp} GPUs, {torch.cuda.device_count()} visible")
                with torch.cuda.device(i):
                    eng = LLMEngine(rcfg, mc, weights=src, device=torch.device("cuda", i))
            eng.set_tokenizer(tok)
            handles.append(EngineHandle(eng))
        return LoadedModel(name, path, DpHandle(handles), tok, mc)
    eng = LLMEngine(cfg, mc, weights=src)
    eng.set_tokenizer(tok)
    return LoadedModel(name, path, EngineHandle(eng), tok, mc)


def run_follower(cfg: EngineConfig) -> int:
    """A rank other than 0 of a multi-rank job: builds its shard of the default model and follows
    rank 0's command stream until shut-down."""
    from .engine.model_manager import ModelManager
    from .parallel.front import follower_loop

    mgr = ModelManager(lambda n, p: None, cfg.models_dir)
    path = mgr.resolve_path(cfg.model)
    _, eng = load_model(cfg.model, path, cfg)
    try:
        follower_loop(eng, _job.ctl, heartbeat=_job.heartbeat, store=_job.store, rank=_job.rank)
    finally:
        eng.close()
    return 0


def relaunch_under_torchrun(argv: list[str], n: int) -> int:
    """`--tp N` outside a launcher: start N ranks of this same command line on this node."""
    import socket
    import subprocess

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "oxide_tech_llm_engine_b200", *argv]
    return subprocess.call(cmd)


def make_manager(cfg: EngineConfig):
    from .engine.model_manager import ModelManager

    mgr = ModelManager(lambda n, p: load_model(n, p, cfg), cfg.models_dir)
    mgr.load(cfg.model, cfg.alias)
    return mgr


def run_chat(args, mgr) -> int:
    from .chat_template import parse_format, render_chat

    m = mgr.get(None)
    sp = sampling_from_args(args)
    sp.stop_token_ids = m.tokenizer.stop_ids()
    fmt = parse_format(args.chat_format, m.model_cfg.arch, m.model_cfg.name)
    history = [{"role": "system", "content": args.system}] if args.system else []

    def generate(user: str) -> str:
        history.append({"role": "user", "content": user})
        toks = m.tokenizer.encode(render_chat(history, fmt))
        t0 = time.perf_counter()
        st = m.handle.submit(toks, sp)
        out, t_first = [], None
        while True:
            ev = st.get(timeout=600)
            if ev.token >= 0 and not (ev.finished and ev.reason == "stop"):
                if t_first is None:
                    t_first = time.perf_counter()
                out.append(ev.token)
                sys.stdout.write(m.tokenizer.decode_token(ev.token))
                sys.stdout.flush()
            if ev.finished:
                break
        dt = time.perf_counter() - (t_first or t0)
        sys.stderr.write(f"\n[ttft {1e3 * ((t_first or t0) - t0):.1f} ms, {len(out) / max(dt, 1e-9):.1f} tok/s]\n")
        text = m.tokenizer.decode(out)
        history.append({"role": "assistant", "content": text})
        return text

    if args.prompt and not args.interactive:
        generate(args.prompt)
        print()
        return 0
    print("oxide chat - /help for commands")
    while True:
        try:
            line = input("> ").strip()
        except EOFError:
            break
        if not line:
            continue
        if line in ("/exit", "/quit"):
            break
        if line == "/help":
            print("/model NAME  /models  /list  /info  /help  /exit  /quit")
        elif line in ("/models", "/list"):
            print("\n".join(mgr.list()))
        elif line == "/info":
            print(json.dumps(m.model_cfg.to_dict(), indent=1))
        elif line.startswith("/model "):
            m = mgr.load(line.split(None, 1)[1])
            history.clear()
        else:
            generate(line)
            print()
    return 0


def run_server(args, mgr) -> int:
    import uvicorn

    from .server.app import create_app

    app = create_app(mgr)
    uvicorn.run(app, host=args.host, port=args.port, log_level="info")  # handles SIGINT/SIGTERM
    for m in list(mgr.models.values()):
        m.handle.shutdown()
    return 0


def run_bench(args, mgr) -> int:
    """Decode loop at a fixed batch -> RooflineReceipt JSON (reference: oxide-bench)."""
    import numpy as np

    from .sampling_params import SamplingParams
    from .utils.roofline import RooflineReceipt, load_measured_peaks

    m = mgr.get(None)
    eng = m.handle.engine
    m.handle.shutdown()  # drive the engine directly
    rng = np.random.default_rng(args.seed)
    sp = SamplingParams(greedy=True, max_tokens=args.steps + 8, ignore_eos=True)
    for _ in range(args.batch):
        eng.add_request(rng.integers(3, m.model_cfg.vocab_size, size=args.prompt_len).tolist(), sp)
    while eng.stats["decode_tokens"] == 0:
        eng.step()
    for _ in range(3):
        eng.step()
    t0 = time.perf_counter()
    n0 = eng.stats["decode_tokens"]
    for _ in range(args.steps):
        eng.step()
    dt = time.perf_counter() - t0
    tok_s = (eng.stats["decode_tokens"] - n0) / dt
    peaks = load_measured_peaks()
    rec = RooflineReceipt.from_run(m.model_cfg, tokens_per_s=tok_s, batch=args.batch, peaks=peaks,
                                   weight_bytes_per_param=2.0, context=args.prompt_len)
    print(json.dumps(rec.to_dict()))
    if args.assert_mbu_min > 0 and rec.mbu < args.assert_mbu_min:
        print(f"MBU {rec.mbu:.3f} below the required {args.assert_mbu_min}", file=sys.stderr)
        return 2
    return 0


def run_verify(args, mgr) -> int:
    """16 greedy tokens from a fixed prompt, printed as ids and text (reference: oxide-verify)."""
    from .sampling_params import SamplingParams

    m = mgr.get(None)
    toks = m.tokenizer.encode(args.prompt or "The quick brown fox")
    out, reason = m.handle.generate(toks, SamplingParams(greedy=True, max_tokens=16, stop_token_ids=m.tokenizer.stop_ids()))
    print(json.dumps({"prompt_tokens": toks, "tokens": out, "text": m.tokenizer.decode(out), "finish_reason": reason}))
    return 0


def run_roofline(args) -> int:
    """Device copy-bandwidth probe (reference: oxide-roofline's memcpy probe)."""
    import torch

    n = args.mib * (1 << 20) // 2
    a = torch.empty(n, dtype=torch.bfloat16, device=f"cuda:{args.gpu}").normal_()
    b = torch.empty_like(a)
    best = 0.0
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        b.copy_(a)
        e.record()
        torch.cuda.synchronize()
        best = max(best, 2 * n * 2 / (s.elapsed_time(e) * 1e-3) / 1e9)
    print(json.dumps({"copy_gb_s": round(best, 1), "mib": args.mib}))
    return 0


def run_quantize(args) -> int:
    """Re-encode the matrices of a GGUF / SafeTensors checkpoint to another block type."""
    from .formats import quants
    from .formats.gguf import GgufWriter
    from .models.config import gguf_metadata
    from .models.weights import open_weights

    src = open_weights(args.input)
    md = gguf_metadata(src.cfg)
    if hasattr(src, "file"):
        md.update({k: v for k, v in src.file.metadata.items() if k.startswith("tokenizer.") or k.startswith("general.")})
    w = GgufWriter(args.output, md)
    for name in src.names():
        arr = src.f32(name)
        if arr.ndim == 1 or name.endswith("ffn_gate_inp.weight"):
            t = "F32"
        elif name in ("token_embd.weight", "output.weight"):
            t = args.embed_type
        else:
            t = args.type
        if arr.shape[-1] % quants.TYPES[t].block:
            t = "F16"
        w.add_tensor(name, arr, t)
    w.write()
    print(f"wrote {args.output}")
    return 0


def main(argv: Optional[list[str]] = None) -> int:
    try:
        args = parse_args(argv)
    except ConfigError as ex:
        print(f"error: {ex}", file=sys.stderr)
        return 2
    if args.command in ("img", "lab"):
        print(f"error: the `{args.command}` subcommand is not part of this engine", file=sys.stderr)
        return 2
    if args.command == "gpu-unlock":
        print("error: gpu-unlock changes device state and is never built here", file=sys.stderr)
        return 2
    if args.command == "roofline":
        return run_roofline(args)
    if args.command == "quantize":
        return run_quantize(args)
    cfg = engine_config_from_args(args)
    global _job
    if cfg.tp > 1:
        if args.command != "server" and not getattr(args, "serve", False):
            print("error: --tp > 1 is for the server (chat / bench / verify drive one GPU)", file=sys.stderr)
            return 2
        if "RANK" not in os.environ:
            return relaunch_under_torchrun(normalize_argv(list(sys.argv[1:] if argv is None else argv)), cfg.tp)
        if int(os.environ["WORLD_SIZE"]) != cfg.tp:
            print(f"error: --tp {cfg.tp} but the launcher started {os.environ['WORLD_SIZE']} ranks", file=sys.stderr)
            return 2
        _job = Job(cfg.backend)
        if _job.rank != 0:
            try:
                return run_follower(cfg)
            finally:
                _job.close()
    if _job is None or _job.rank == 0:
        print(cfg.describe(), file=sys.stderr)
    try:
        mgr = make_manager(cfg)
    except EngineError as ex:
        print(f"error: {ex}", file=sys.stderr)
        return 1
    try:
        if args.command == "server" or getattr(args, "serve", False):
            return run_server(args, mgr)
        if args.command == "bench":
            return run_bench(args, mgr)
        if args.command == "verify":
            return run_verify(args, mgr)
        return run_chat(args, mgr)
    finally:
        for m in list(mgr.models.values()):
            m.handle.shutdown(timeout=2.0)
        if _job is not None:
            _job.close()


if __name__ == "__main__":
    sys.exit(main())
