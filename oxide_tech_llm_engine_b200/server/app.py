"""OpenAI-compatible HTTP server (+ Anthropic messages, embeddings, rerank, metrics).

Routes and wire format follow the reference router (oxide-server/src/lib.rs:304-319):
GET /health ("Oxide-Tech-LLM-Engine OK"), GET /metrics (Prometheus gauges oxide_up,
oxide_active_inference_slots, oxide_max_inference_slots + engine gauges), GET /v1/models,
POST /v1/models/load, POST /v1/chat/completions (SSE `chat.completion.chunk` with the role on the
first delta and a terminal `data: [DONE]`, lib.rs:455-485), POST /v1/completions,
POST /v1/embeddings (mean of token-embedding rows, L2 normalised, lib.rs:831-876),
POST /v1/rerank (cosine, lib.rs:928-1002), POST /v1/vision/detect (501), POST /v1/messages
(Anthropic events, anthropic.rs:140-269). Defaults max_tokens=64, temperature=0.7, top_p=0.9; ids
`chatcmpl-oxide-N`, `cmpl-oxide-N`, `msg_oxide_N`; `created` = 1728000000; 503 body of lib.rs:531-541.
Unlike the reference, every request goes through the GPU continuous-batching engine, and
/v1/completions streams too.
"""
from __future__ import annotations

import asyncio
import itertools
import json
import time
from typing import Any, Optional

import numpy as np
from fastapi import FastAPI, Request
from fastapi.middleware.cors import CORSMiddleware
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..chat_template import ChatFormat, render_chat
from ..errors import EngineError, ModelLoadError, SlotsExhausted
from ..sampling_params import SamplingParams
from .parsers import split_reasoning, parse_tool_calls  # noqa: F401  (re-exported for clients)

CREATED = 1728000000
_req_counter = itertools.count(1)
_rerank_counter = itertools.count(1)


def _busy() -> JSONResponse:
    return JSONResponse(status_code=503, content={"error": {
        "message": "All inference slots busy (concurrency limit reached)", "type": "server_error", "code": 503}})


def _error(status: int, msg: str, typ: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse(status_code=status, content={"error": {"message": msg, "type": typ, "code": status}})


class Metrics:
    def __init__(self):
        self.requests = 0
        self.prompt_tokens = 0
        self.completion_tokens = 0
        self.ttft: list[float] = []
        self.tpot: list[float] = []

    def observe(self, prompt: int, completion: int, ttft: Optional[float], tpot: Optional[float]) -> None:
        self.requests += 1
        self.prompt_tokens += prompt
        self.completion_tokens += completion
        if ttft is not None:
            self.ttft = (self.ttft + [ttft])[-1024:]
        if tpot is not None:
            self.tpot = (self.tpot + [tpot])[-1024:]

    @staticmethod
    def pct(v: list[float], p: float) -> float:
        return float(np.percentile(v, p)) if v else 0.0


def create_app(manager, *, allow_queueing: bool = True) -> FastAPI:
    """`manager` is an engine.model_manager.ModelManager with at least one registered model."""
    app = FastAPI(title="Oxide-Tech-LLM-Engine (B200)")
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_methods=["*"], allow_headers=["*"])
    metrics = Metrics()
    app.state.metrics = metrics
    app.state.manager = manager

    def resolve(model: Optional[str]):
        try:
            return manager.get(model)
        except ModelLoadError:
            return manager.load(model) if model else None

    def sampling(body: dict, m) -> SamplingParams:
        temperature = float(body.get("temperature", 0.7) if body.get("temperature") is not None else 0.7)
        sp = SamplingParams(temperature=temperature, top_p=float(body.get("top_p") or 0.9),
                            top_k=int(body.get("top_k") or 40), min_p=float(body.get("min_p") or 0.0),
                            max_tokens=int(body.get("max_tokens") or 64), seed=int(body.get("seed") or 42),
                            greedy=temperature <= 0.0,
                            repeat_penalty=float(body.get("repeat_penalty") or 1.0),
                            frequency_penalty=float(body.get("frequency_penalty") or 0.0),
                            presence_penalty=float(body.get("presence_penalty") or 0.0),
                            stop_token_ids=m.tokenizer.stop_ids())
        if body.get("json_schema") or (body.get("response_format") or {}).get("type") in ("json_object", "json_schema"):
            sp.grammar = "json"
        return sp

    async def collect(m, stream, t0):
        toks, reason, t_first = [], "length", None
        while True:
            ev = await stream.aget()
            if ev.token >= 0:
                if t_first is None:
                    t_first = time.perf_counter()
                if not (ev.finished and ev.reason == "stop"):
                    toks.append(ev.token)
            if ev.finished:
                reason = ev.reason or "stop"
                break
        t1 = time.perf_counter()
        n = max(len(toks), 1)
        metrics.observe(stream.prompt_tokens, len(toks), (t_first - t0) if t_first else None,
                        (t1 - t_first) / max(n - 1, 1) if t_first else None)
        return toks, reason

    def submit(m, prompt_tokens, sp):
        loop = asyncio.get_running_loop()
        return m.handle.submit(prompt_tokens, sp, loop=loop, queue_if_full=allow_queueing)

    async def sse_chat(m, stream, rid: str, model_name: str, t0: float):
        first = True
        n, t_first, done = 0, None, False
        try:
            while True:
                ev = await stream.aget()
                finish = None
                text = None
                if ev.token >= 0 and not (ev.finished and ev.reason == "stop"):
                    text = m.tokenizer.decode_token(ev.token)
                    n += 1
                    if t_first is None:
                        t_first = time.perf_counter()
                if ev.finished:
                    finish = ev.reason or "stop"
                chunk = {"id": rid, "object": "chat.completion.chunk", "created": CREATED, "model": model_name,
                         "choices": [{"index": 0, "delta": {"content": text, "role": "assistant" if first else None},
                                      "finish_reason": finish}]}
                first = False
                yield f"data: {json.dumps(chunk)}\n\n"
                if ev.finished:
                    done = True
                    break
            yield "data: [DONE]\n\n"
        finally:
            if not done:  # the client went away mid-generation: give the slot and the blocks back
                stream.closed = True
                m.handle.cancel(stream.req_id)
            t1 = time.perf_counter()
            metrics.observe(stream.prompt_tokens, n, (t_first - t0) if t_first else None,
                            (t1 - t_first) / max(n - 1, 1) if t_first else None)

    # ------------------------------------------------------------------ basic routes
    @app.get("/health")
    async def health():
        ok = all(m.handle.healthy for m in manager.models.values())
        return PlainTextResponse("Oxide-Tech-LLM-Engine OK" if ok else "Oxide-Tech-LLM-Engine DEGRADED",
                                 status_code=200 if ok else 503)

    @app.get("/metrics")
    async def metrics_route():
        active = sum(m.handle.active_slots() for m in manager.models.values())
        max_slots = sum(m.handle.max_slots for m in manager.models.values())
        lines = [
            "# HELP oxide_up Server operational status", "# TYPE oxide_up gauge", "oxide_up 1",
            "# HELP oxide_active_inference_slots Number of currently leased inference slots",
            "# TYPE oxide_active_inference_slots gauge", f"oxide_active_inference_slots {active}",
            "# HELP oxide_max_inference_slots Maximum configured continuous batching slots",
            "# TYPE oxide_max_inference_slots gauge", f"oxide_max_inference_slots {max_slots}",
        ]
        for name, m in manager.models.items():
            eng = m.handle.engine
            rs = eng.sched.radix_stats()
            lab = f'{{model="{name}"}}'
            lines += [
                f"oxide_queue_depth{lab} {eng.sched.num_waiting()}",
                f"oxide_running_sequences{lab} {eng.sched.num_running()}",
                f"oxide_kv_blocks_free{lab} {eng.sched.num_free_blocks()}",
                f"oxide_prefix_hit_tokens{lab} {rs['hit_tokens']}",
                f"oxide_prefix_lookup_tokens{lab} {rs['lookup_tokens']}",
                f"oxide_prefix_lookups{lab} {rs['lookups']}",
                f"oxide_decode_tokens_total{lab} {eng.stats['decode_tokens']}",
                f"oxide_prefill_tokens_total{lab} {eng.stats['prefill_tokens']}",
                f"oxide_engine_steps_total{lab} {eng.stats['steps']}",
                f"oxide_preemptions_total{lab} {eng.sched.preemptions()}",
                f"oxide_graph_replays_total{lab} {eng.stats.get('graph_replays', 0)}",
                f"oxide_burst_steps_total{lab} {eng.stats.get('burst_steps', 0)}",
                f"oxide_spec_proposed_total{lab} {eng.stats.get('spec_proposed', 0)}",
                f"oxide_spec_accepted_total{lab} {eng.stats.get('spec_accepted', 0)}",
                f"oxide_h2o_pruned_blocks_total{lab} {eng.stats.get('h2o_pruned_blocks', 0)}",
                f"oxide_context_shifts_total{lab} {eng.sched.context_shifts()}",
                f"oxide_kv_demoted_blocks_total{lab} {eng.stats.get('kv_demoted_blocks', 0)}",
                f"oxide_kv_promoted_blocks_total{lab} {eng.stats.get('kv_promoted_blocks', 0)}",
                f"oxide_device_faults_total{lab} {eng.stats.get('device_faults', 0)}",
            ]
            tier = getattr(eng, "kv_tier", None)
            if tier is not None:
                lines += [f"oxide_kv_tier_host_blocks{lab} {len(tier.host)}",
                          f"oxide_kv_tier_storage_blocks{lab} {len(tier.storage)}",
                          f"oxide_kv_tier_host_hits_total{lab} {tier.stats['host_hits']}",
                          f"oxide_kv_tier_storage_hits_total{lab} {tier.stats['storage_hits']}"]
        lines += [
            f"oxide_requests_total {metrics.requests}",
            f"oxide_ttft_seconds_p50 {Metrics.pct(metrics.ttft, 50):.6f}",
            f"oxide_ttft_seconds_p99 {Metrics.pct(metrics.ttft, 99):.6f}",
            f"oxide_tpot_seconds_p50 {Metrics.pct(metrics.tpot, 50):.6f}",
            f"oxide_tpot_seconds_p99 {Metrics.pct(metrics.tpot, 99):.6f}",
        ]
        return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": n, "object": "model", "created": CREATED, "owned_by": "oxide-engine"}
                                           for n in manager.list()]}

    @app.post("/v1/models/load")
    async def models_load(req: Request):
        body = await req.json()
        name = body.get("model")
        if not name:
            return _error(400, "model is required")
        try:
            await asyncio.get_running_loop().run_in_executor(None, manager.load, name, body.get("alias"))
        except (ModelLoadError, EngineError, OSError) as ex:
            return JSONResponse(status_code=400, content={"success": False, "model": name, "message": str(ex)})
        return {"success": True, "model": name, "message": f"model {name} loaded"}

    # ------------------------------------------------------------------ completions
    @app.post("/v1/chat/completions")
    async def chat_completions(req: Request):
        body = await req.json()
        try:
            m = resolve(body.get("model"))
        except (ModelLoadError, EngineError) as ex:
            return _error(404, str(ex))
        if body.get("messages"):
            prompt = render_chat(body["messages"], ChatFormat.CHATML)
        else:
            prompt = body.get("prompt") or ""
        toks = m.tokenizer.encode(prompt)
        sp = sampling(body, m)
        t0 = time.perf_counter()
        try:
            stream = submit(m, toks, sp)
        except SlotsExhausted:
            return _busy()
        except EngineError as ex:  # the engine group is down (a rank left): no request can be served
            return _error(503, str(ex), "server_error")
        rid = f"chatcmpl-oxide-{next(_req_counter)}"
        name = body.get("model") or m.name
        if body.get("stream"):
            return StreamingResponse(sse_chat(m, stream, rid, name, t0), media_type="text/event-stream")
        out, reason = await collect(m, stream, t0)
        text = m.tokenizer.decode(out)
        return {"id": rid, "object": "chat.completion", "created": CREATED, "model": name,
                "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": reason}],
                "usage": {"prompt_tokens": len(toks), "completion_tokens": len(out), "total_tokens": len(toks) + len(out)}}

    @app.post("/v1/completions")
    async def completions(req: Request):
        body = await req.json()
        try:
            m = resolve(body.get("model"))
        except (ModelLoadError, EngineError) as ex:
            return _error(404, str(ex))
        prompt = body.get("prompt") or ""
        if isinstance(prompt, list):
            prompt = prompt[0] if prompt else ""
        toks = m.tokenizer.encode(prompt)
        sp = sampling(body, m)
        t0 = time.perf_counter()
        try:
            stream = submit(m, toks, sp)
        except SlotsExhausted:
            return _busy()
        except EngineError as ex:  # the engine group is down (a rank left): no request can be served
            return _error(503, str(ex), "server_error")
        rid = f"cmpl-oxide-{next(_req_counter)}"
        name = body.get("model") or m.name
        if body.get("stream"):
            async def gen():
                while True:
                    ev = await stream.aget()
                    text = ""
                    if ev.token >= 0 and not (ev.finished and ev.reason == "stop"):
                        text = m.tokenizer.decode_token(ev.token)
                    chunk = {"id": rid, "object": "text_completion", "created": CREATED, "model": name,
                             "choices": [{"text": text, "index": 0,
                                          "finish_reason": (ev.reason or "stop") if ev.finished else None}]}
                    yield f"data: {json.dumps(chunk)}\n\n"
                    if ev.finished:
                        break
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        out, reason = await collect(m, stream, t0)
        return {"id": rid, "object": "text_completion", "created": CREATED, "model": name,
                "choices": [{"text": m.tokenizer.decode(out), "index": 0, "finish_reason": reason}],
                "usage": {"prompt_tokens": len(toks), "completion_tokens": len(out), "total_tokens": len(toks) + len(out)}}

    # ------------------------------------------------------------------ embeddings / rerank
    def embed_text(m, text: str) -> tuple[np.ndarray, int]:
        toks = m.tokenizer.encode(text, add_bos=False) or [0]
        rows = m.embedding_rows(np.asarray(toks, dtype=np.int64))
        v = rows.mean(0)
        n = float(np.linalg.norm(v))
        return (v / n if n > 0 else v), len(toks)

    @app.post("/v1/embeddings")
    async def embeddings(req: Request):
        body = await req.json()
        m = resolve(body.get("model"))
        inp = body.get("input")
        texts = [inp] if isinstance(inp, str) else list(inp or [])
        data, total = [], 0
        for i, t in enumerate(texts):
            v, n = embed_text(m, str(t))
            total += n
            data.append({"object": "embedding", "index": i, "embedding": [float(x) for x in v]})
        return {"object": "list", "data": data, "model": body.get("model") or m.name,
                "usage": {"prompt_tokens": total, "completion_tokens": 0, "total_tokens": total}}

    @app.post("/v1/rerank")
    async def rerank(req: Request):
        body = await req.json()
        m = resolve(body.get("model"))
        q, nq = embed_text(m, body.get("query", ""))
        docs = list(body.get("documents") or [])
        res, total = [], nq
        for i, d in enumerate(docs):
            v, n = embed_text(m, str(d))
            total += n
            item: dict[str, Any] = {"index": i, "relevance_score": float(np.dot(q, v))}
            if body.get("return_documents"):
                item["document"] = {"text": str(d)}
            res.append(item)
        res.sort(key=lambda r: -r["relevance_score"])
        top_n = body.get("top_n")
        if top_n:
            res = res[: int(top_n)]
        return {"id": f"rerank-{next(_rerank_counter):08x}", "results": res,
                "meta": {"api_version": {"version": "1"}, "billed_units": {"search_units": 1, "total_tokens": total}}}

    @app.post("/v1/vision/detect")
    async def vision_detect():
        return _error(501, "vision detection is not served by this engine", "not_implemented")

    # ------------------------------------------------------------------ Anthropic messages
    @app.post("/v1/messages")
    async def messages(req: Request):
        body = await req.json()
        try:
            m = resolve(body.get("model"))
        except (ModelLoadError, EngineError) as ex:
            return JSONResponse(status_code=404, content={"type": "error", "error": {"type": "not_found_error", "message": str(ex)}})
        parts = []
        system = body.get("system")
        if isinstance(system, list):
            system = "".join(b.get("text", "") for b in system if isinstance(b, dict))
        if system:
            parts.append(f"{system}\n")
        for msg in body.get("messages", []):
            c = msg.get("content")
            if isinstance(c, list):
                c = "".join(b.get("text", "") for b in c if isinstance(b, dict))
            parts.append(f"{msg.get('role', 'user')}: {c}\n")
        parts.append("Assistant: ")
        toks = m.tokenizer.encode("".join(parts))
        b2 = dict(body)
        b2["max_tokens"] = min(int(body.get("max_tokens") or 1024), 4096)
        sp = sampling(b2, m)
        t0 = time.perf_counter()
        try:
            stream = submit(m, toks, sp)
        except SlotsExhausted:
            return JSONResponse(status_code=529, content={"type": "error", "error": {"type": "overloaded_error", "message": "All inference slots busy"}})
        except EngineError as ex:
            return JSONResponse(status_code=503, content={"type": "error", "error": {"type": "api_error", "message": str(ex)}})
        mid = f"msg_oxide_{next(_req_counter)}"
        name = body.get("model") or m.name
        if body.get("stream"):
            async def gen():
                def ev_(name_, data):
                    return f"event: {name_}\ndata: {json.dumps(data)}\n\n"
                yield ev_("message_start", {"type": "message_start", "message": {
                    "id": mid, "type": "message", "role": "assistant", "content": [], "model": name,
                    "stop_reason": None, "usage": {"input_tokens": len(toks), "output_tokens": 0}}})
                yield ev_("content_block_start", {"type": "content_block_start", "index": 0,
                                                  "content_block": {"type": "text", "text": ""}})
                n = 0
                while True:
                    e = await stream.aget()
                    if e.token >= 0 and not (e.finished and e.reason == "stop"):
                        n += 1
                        yield ev_("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                          "delta": {"type": "text_delta", "text": m.tokenizer.decode_token(e.token)}})
                    if e.finished:
                        reason = "end_turn" if e.reason == "stop" else "max_tokens"
                        break
                yield ev_("content_block_stop", {"type": "content_block_stop", "index": 0})
                yield ev_("message_delta", {"type": "message_delta", "delta": {"stop_reason": reason},
                                            "usage": {"output_tokens": n}})
                yield ev_("message_stop", {"type": "message_stop"})
            return StreamingResponse(gen(), media_type="text/event-stream")
        out, reason = await collect(m, stream, t0)
        return {"id": mid, "type": "message", "role": "assistant", "model": name,
                "content": [{"type": "text", "text": m.tokenizer.decode(out)}],
                "stop_reason": "end_turn" if reason == "stop" else "max_tokens",
                "usage": {"input_tokens": len(toks), "output_tokens": len(out)}}

    return app
