"""Worker of the multi-rank serving-front tests (launched under torchrun with 2 CPU ranks over gloo):
rank 0 serves HTTP through the distributed handle, rank 1 follows its command stream.

    mp_front_check.py stream   both ranks serve a streamed chat completion and a cancelled request
    mp_front_check.py leave    rank 1 leaves between steps; rank 0 ends the requests with a typed reason
"""
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from oxide_tech_llm_engine_b200 import cli
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.model_manager import ModelManager
    from oxide_tech_llm_engine_b200.parallel.front import follower_loop

    mode = sys.argv[1]
    cfg = EngineConfig(backend="cpu", model="tiny", tp=2, max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=128,
                       ctx_size=512, enable_radix=False)
    cli._job = job = cli.Job("cpu")
    if job.rank != 0:
        _, eng = cli.load_model("tiny", None, cfg)
        steps = follower_loop(eng, job.ctl, heartbeat=job.heartbeat, store=job.store, rank=job.rank,
                              leave_after_steps=3 if mode == "leave" else None)
        free = eng.sched.num_free_blocks()
        print(f"FOLLOWER steps={steps} free_blocks={free} running={eng.sched.num_running()}", flush=True)
        if mode == "leave":
            time.sleep(3.0)   # the host of the rank stays up for a while; it just no longer takes part
        job.heartbeat.stop()
        return
    from starlette.testclient import TestClient

    from oxide_tech_llm_engine_b200.server.app import create_app

    mgr = ModelManager(lambda n, p: cli.load_model(n, p, cfg))
    mgr.load("tiny", alias="default-model")
    handle = mgr.get(None).handle
    eng = handle.engine
    free0 = eng.sched.num_free_blocks()
    with TestClient(create_app(mgr)) as c:
        if mode == "stream":
            body = {"model": "tiny", "messages": [{"role": "user", "content": "hello there"}], "max_tokens": 12,
                    "temperature": 0, "stream": True}
            chunks = []
            with c.stream("POST", "/v1/chat/completions", json=body) as r:
                assert r.status_code == 200 and r.headers["content-type"].startswith("text/event-stream")
                for line in r.iter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        chunks.append(json.loads(line[6:]))
            text = "".join(ch["choices"][0]["delta"].get("content", "") for ch in chunks)
            assert chunks[0]["choices"][0]["delta"].get("role") == "assistant" and chunks[-1]["choices"][0]["finish_reason"]
            # the same request without streaming gives the same text (greedy)
            r2 = c.post("/v1/chat/completions", json=dict(body, stream=False)).json()
            assert r2["choices"][0]["message"]["content"] == text, (text, r2)
            # several clients at once, then everything is back in the pool
            outs = [c.post("/v1/completions", json={"model": "tiny", "prompt": "abc" * (i + 1), "max_tokens": 6,
                                                      "temperature": 0}).json() for i in range(3)]
            assert all(o["usage"]["completion_tokens"] == 6 for o in outs)
            assert c.get("/health").status_code == 200
            print(f"FRONT stream OK text={text!r}", flush=True)
        else:
            from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

            st = handle.submit(list(range(3, 40)), SamplingParams(greedy=True, max_tokens=400, ignore_eos=True))
            got, reason = 0, ""
            while True:
                ev = st.get(timeout=60)
                got += ev.token >= 0
                if ev.finished:
                    reason = ev.reason
                    break
            assert reason.startswith("rank_failure"), reason
            assert got < 400 and handle.dead is not None and not handle.healthy
            deadline = time.time() + 5
            while eng.sched.num_free_blocks() != free0 and time.time() < deadline:
                time.sleep(0.01)
            assert eng.sched.num_free_blocks() == free0 and not eng.has_work()
            r = c.post("/v1/completions", json={"model": "tiny", "prompt": "abc", "max_tokens": 3, "temperature": 0})
            assert r.status_code in (500, 503), r.status_code
            print(f"FRONT leave OK reason={reason!r} tokens_before={got}", flush=True)
    for m in list(mgr.models.values()):
        m.handle.shutdown(timeout=5.0)
    job.heartbeat.stop()
    free = eng.sched.num_free_blocks()
    assert free == free0, (free, free0)
    print(f"FRONT done free_blocks={free}", flush=True)


if __name__ == "__main__":
    main()
    os._exit(0)   # gloo teardown of a group whose peer left may block; the checks above are what counts
