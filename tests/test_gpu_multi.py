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
