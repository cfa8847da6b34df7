"""HTTP API on the CPU backend through an in-process client (no sockets, no GPU)."""
import json

import pytest
from starlette.testclient import TestClient

from oxide_tech_llm_engine_b200.cli import load_model
from oxide_tech_llm_engine_b200.config import EngineConfig
from oxide_tech_llm_engine_b200.engine.model_manager import ModelManager
from oxide_tech_llm_engine_b200.server.app import create_app
from oxide_tech_llm_engine_b200.server.parsers import parse_tool_calls, split_reasoning


@pytest.fixture(scope="module")
def client():
    cfg = EngineConfig(backend="cpu", model="tiny", max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=128,
                       ctx_size=512)
    mgr = ModelManager(lambda n, p: load_model(n, p, cfg))
    mgr.load("tiny", alias="default-model")
    with TestClient(create_app(mgr)) as c:
        yield c
    for m in list(mgr.models.values()):
        m.handle.shutdown()


def test_health_metrics_models(client):
    r = client.get("/health")
    assert r.status_code == 200 and r.text == "Oxide-Tech-LLM-Engine OK"
    m = client.get("/metrics")
    assert m.headers["content-type"].startswith("text/plain")
    for g in ("oxide_up 1", "oxide_active_inference_slots 0", "oxide_max_inference_slots 4", "oxide_kv_blocks_free",
              "oxide_context_shifts_total", "oxide_spec_accepted_total", "oxide_kv_promoted_blocks_total",
              "oxide_burst_steps_total", "oxide_device_faults_total"):
        assert g in m.text
    ids = [d["id"] for d in client.get("/v1/models").json()["data"]]
    assert "tiny" in ids and "default-model" in ids


def test_chat_completion_non_stream(client):
    r = client.post("/v1/chat/completions", json={"model": "tiny", "messages": [{"role": "user", "content": "hi"}],
                                                  "max_tokens": 5, "temperature": 0})
    j = r.json()
    assert r.status_code == 200 and j["object"] == "chat.completion" and j["id"].startswith("chatcmpl-oxide-")
    assert j["created"] == 1728000000 and j["choices"][0]["message"]["role"] == "assistant"
    assert j["choices"][0]["finish_reason"] in ("length", "stop")
    u = j["usage"]
    assert u["completion_tokens"] <= 5 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]


def test_chat_completion_stream_sse(client):
    with client.stream("POST", "/v1/chat/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 4,
                                                              "temperature": 0, "stream": True}) as r:
        assert r.headers["content-type"].startswith("text/event-stream")
        lines = [l for l in r.iter_lines() if l]
    assert lines[-1] == "data: [DONE]" and all(l.startswith("data: ") for l in lines)
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["object"] == "chat.completion.chunk" and chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[1]["choices"][0]["delta"]["role"] is None
    assert chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop") and len(chunks) == 4


def test_completions_and_determinism(client):
    body = {"model": "tiny", "prompt": "hello", "max_tokens": 6, "temperature": 0}
    a = client.post("/v1/completions", json=body).json()
    b = client.post("/v1/completions", json=body).json()
    assert a["object"] == "text_completion" and a["id"].startswith("cmpl-oxide-")
    assert a["choices"][0]["text"] == b["choices"][0]["text"]
    with client.stream("POST", "/v1/completions", json=dict(body, stream=True)) as r:
        lines = [l for l in r.iter_lines() if l]
    assert lines[-1] == "data: [DONE]"


def test_embeddings_and_rerank(client):
    e = client.post("/v1/embeddings", json={"model": "tiny", "input": ["abc", "abd"]}).json()
    v = e["data"][0]["embedding"]
    assert len(e["data"]) == 2 and abs(sum(x * x for x in v) - 1.0) < 1e-4
    r = client.post("/v1/rerank", json={"model": "tiny", "query": "abc", "documents": ["xyz", "abc", "abq"],
                                         "top_n": 2, "return_documents": True}).json()
    assert r["id"].startswith("rerank-") and len(r["results"]) == 2 and r["results"][0]["index"] == 1
    assert r["results"][0]["document"]["text"] == "abc" and r["meta"]["billed_units"]["search_units"] == 1


def test_anthropic_messages(client):
    body = {"model": "tiny", "max_tokens": 4, "system": "s", "messages": [{"role": "user", "content": "hi"}],
            "temperature": 0}
    j = client.post("/v1/messages", json=body).json()
    assert j["type"] == "message" and j["id"].startswith("msg_oxide_") and j["content"][0]["type"] == "text"
    with client.stream("POST", "/v1/messages", json=dict(body, stream=True)) as r:
        names = [l[7:] for l in r.iter_lines() if l.startswith("event: ")]
    assert names[:2] == ["message_start", "content_block_start"]
    assert names[-3:] == ["content_block_stop", "message_delta", "message_stop"] and "content_block_delta" in names


def test_model_hot_load_and_errors(client):
    r = client.post("/v1/models/load", json={"model": "tiny-moe", "alias": "moe"})
    assert r.status_code == 200 and r.json()["success"]
    j = client.post("/v1/completions", json={"model": "moe", "prompt": "x", "max_tokens": 2, "temperature": 0}).json()
    assert j["usage"]["completion_tokens"] <= 2
    bad = client.post("/v1/models/load", json={"model": "/no/such/file.gguf"})
    assert bad.status_code == 400 and not bad.json()["success"]
    assert client.post("/v1/vision/detect", json={}).status_code == 501


def test_slots_busy_returns_503():
    cfg = EngineConfig(backend="cpu", model="tiny", max_num_seqs=1, max_num_batched_tokens=32, num_kv_blocks=64,
                       ctx_size=256)
    mgr = ModelManager(lambda n, p: load_model(n, p, cfg))
    m = mgr.load("tiny")
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    with TestClient(create_app(mgr, allow_queueing=False)) as c:
        st = m.handle.submit(list(range(5, 30)), SamplingParams(greedy=True, max_tokens=200, ignore_eos=True))
        r = c.post("/v1/chat/completions", json={"model": "tiny", "prompt": "x", "max_tokens": 2})
        assert r.status_code == 503 and r.json()["error"]["code"] == 503
        assert "slots busy" in r.json()["error"]["message"]
        m.handle.cancel(st.req_id)
    m.handle.shutdown()


def test_reasoning_and_tool_parsers():
    assert split_reasoning("<think>plan</think>answer") == ("plan", "answer")
    assert split_reasoning("plain") == ("", "plain")
    calls = parse_tool_calls('<tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>')
    assert calls[0].name == "f" and calls[0].arguments == {"x": 1}
    assert parse_tool_calls('{"name": "g", "parameters": "{\\"y\\": 2}"}')[0].arguments == {"y": 2}
