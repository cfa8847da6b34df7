"""Multi-process host-side parallelism on CPU ranks (gloo): pipeline hand-off, ring attention,
data-parallel routing."""
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _torchrun(n, what, port):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_cpu_parallel.py"), what]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_parallel_decoding_matches_oracle(world):
    r = _torchrun(world, "pipeline", 29610 + world)
    assert r.returncode == 0 and "PP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_ring_attention_matches_full_attention():
    r = _torchrun(2, "ring", 29620)
    assert r.returncode == 0 and "RING_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_stage_plans_and_ngl():
    from oxide_tech_llm_engine_b200.parallel.pipeline import StagePlan, plan_n_gpu_layers

    assert [StagePlan(3, s, 80).layers for s in range(3)] == [(0, 27), (27, 54), (54, 80)]
    assert StagePlan(3, 0, 80).first and StagePlan(3, 2, 80).last
    host, dev = plan_n_gpu_layers(32, 20)
    assert list(host) == list(range(12)) and list(dev) == list(range(12, 32))
    assert len(plan_n_gpu_layers(32, -1)[0]) == 0


def test_dp_router_prefix_affinity_and_balance():
    from oxide_tech_llm_engine_b200.parallel.dp_router import DpRouter

    class Rep:
        def __init__(self): self.n = 0
        def active_slots(self): return self.n
        def submit(self, toks, params, **kw):
            self.n += 1
            return self.n
    reps = [Rep(), Rep(), Rep()]
    r = DpRouter(reps, affinity_tokens=8, imbalance=2)
    a = list(range(100))
    b = list(range(50, 150))
    ia, _ = r.submit(a, None)
    ib, _ = r.submit(b, None)
    assert ia != ib
    assert r.submit(a + [7], None)[0] == ia           # same prefix -> same replica (radix hit)
    for _ in range(4):
        r.submit(a, None)
    assert reps[ia].n <= 5 and sum(rep.n for rep in reps) == 7
    assert max(rep.n for rep in reps) - min(rep.n for rep in reps) <= 5
    spill = r.pick(a)
    assert spill != ia                                  # the hot replica is too far ahead: spill over
