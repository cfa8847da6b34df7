"""Multi-GPU tier: the fused GEMM->reduce-scatter / all-gather->GEMM / MoE dispatch-combine path
on 2+ GPUs (one process per GPU, plain peer loads and stores; NVLS is switched off)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_tp_and_ep_match_oracle():
    n = min(torch.cuda.device_count(), 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.join(here, "mp_tp_check.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_CHECK tiny world=%d OK" % n in r.stdout
    assert "TP_CHECK tiny-moe world=%d OK" % n in r.stdout
    assert "TP_CHECK tiny-fp8 world=%d OK" % n in r.stdout
    assert "TP_CHECK tiny-h2o world=%d OK" % n in r.stdout
    assert "TP_CHECK tiny-b160 world=%d OK" % n in r.stdout
    assert "TP_CHECK tiny-moe-fp4 world=%d OK" % n in r.stdout


def test_pipeline_parallel_stages_match_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs (one pipeline stage per GPU)")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29512", os.path.join(here, "mp_pp_check.py"), "2"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "PP_CHECK pp=2 tp=1 OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("what,token", [("ring", "RING_OK"), ("ulysses", "ULYSSES_OK")])
def test_context_parallel_attention_over_nccl_matches_full_attention(what, token):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs (one context-parallel rank per GPU)")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", OXB_RING_GPU="1")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29513", os.path.join(here, "mp_cpu_parallel.py"), what]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and token in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_http_server_over_a_tensor_parallel_engine():
    """`server --tp 2`: the CLI starts two ranks (one per GPU), rank 0 serves HTTP and broadcasts the
    admitted requests to rank 1 over gloo; a streamed chat completion equals the non-streamed one."""
    import json
    import signal
    import socket
    import time
    import urllib.request

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=root)
    proc = subprocess.Popen([sys.executable, "-m", "oxide_tech_llm_engine_b200", "server", "-m", "tiny", "--tp", "2",
                             "--port", str(port), "--max-slots", "8", "-c", "512", "--kv-device-blocks", "256"],
                            env=env, cwd=root, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            start_new_session=True)
    base = f"http://127.0.0.1:{port}"
    try:
        up = False
        for _ in range(240):
            if proc.poll() is not None:
                break
            try:
                up = urllib.request.urlopen(base + "/health", timeout=1).status == 200
                if up:
                    break
            except Exception:
                time.sleep(0.5)
        assert up, "server did not come up: " + (proc.stdout.read()[-3000:] if proc.poll() is not None else "")
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 10, "temperature": 0}

        def post(b):
            req = urllib.request.Request(base + "/v1/chat/completions", data=json.dumps(b).encode(),
                                         headers={"Content-Type": "application/json"})
            return urllib.request.urlopen(req, timeout=120).read().decode()
        first = json.loads(post(body))
        whole = first["choices"][0]["message"]["content"]
        assert first["usage"]["completion_tokens"] == 10     # random weights: the text itself may be unprintable
        text, chunks = "", []
        for line in post(dict(body, stream=True)).splitlines():
            if line.startswith("data: ") and line != "data: [DONE]":
                chunks.append(json.loads(line[6:]))
                text += chunks[-1]["choices"][0]["delta"].get("content", "")
        assert text == whole and chunks and chunks[-1]["choices"][0]["finish_reason"] == "length"
        m = urllib.request.urlopen(base + "/metrics", timeout=5).read().decode()
        assert "oxide_up 1" in m
    finally:
        try:
            os.killpg(proc.pid, signal.SIGTERM)   # the process group this test started, nothing else
        except ProcessLookupError:
            pass
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
