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


def test_ulysses_attention_matches_full_attention():
    r = _torchrun(2, "ulysses", 29625)
    assert r.returncode == 0 and "ULYSSES_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


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


def test_rank_exit_is_detected_on_the_host_and_resources_return():
    r = _torchrun(3, "rank_exit", 29630)
    assert r.returncode == 0 and r.stdout.count("RANK_EXIT_OK") == 2, r.stdout[-2000:] + r.stderr[-3000:]


def test_rank_monitor_with_fake_store_and_clock():
    from oxide_tech_llm_engine_b200.parallel.watchdog import Heartbeat, RankFailure, RankMonitor

    class Store(dict):
        def set(self, k, v): self[k] = v
        def get(self, k): return self[k]
        def check(self, ks): return all(k in self for k in ks)
    st, now = Store(), [0.0]
    hb1 = Heartbeat(st, 1)
    mon = RankMonitor(st, 0, 3, timeout_s=1.0, clock=lambda: now[0])
    now[0] = 0.5
    assert mon.poll() == {}
    hb1.beat()
    now[0] = 1.2
    gone = mon.poll()                      # rank 2 never wrote a heartbeat: it never joined
    assert list(gone) == [2] and "missed" in gone[2]
    now[0] = 1.9
    assert 1 not in mon.poll()             # rank 1 beat at 0.5..1.2
    now[0] = 3.0
    with pytest.raises(RankFailure) as ei:
        mon.check()
    assert ei.value.rank == 1
    hb1.leave()
    mon2 = RankMonitor(st, 0, 2, timeout_s=10.0, clock=lambda: now[0])
    assert mon2.poll() == {1: "left the job"}


@pytest.mark.filterwarnings("ignore::pytest.PytestUnraisableExceptionWarning")
def test_step_worker_runs_commands_in_order_and_idles_in_three_phases():
    import time

    from oxide_tech_llm_engine_b200._build import host_ext

    H = host_ext()
    assert H.STEP_COMMAND_BYTES == 64 and H.STEP_COMPLETION_BYTES == 64
    seen = []

    def handler(kind, a0, a1):
        seen.append((kind, a0, a1))
        if a0 == 13:
            raise RuntimeError("boom")
        return 0, a0 * 2
    w = H.StepWorker(handler, capacity=8, pin_core=-1, spin_limit=50, yield_limit=200, park_us=50)
    hb0 = w.heartbeat()
    for i in range(20):
        while not w.submit(i, 0, i, 1000 + i):
            c = w.wait(1000)
            assert c is not None
        if i == 5:
            time.sleep(0.02)               # let the worker reach the park phase
    got = []
    while len(got) + 0 < 20:
        c = w.wait(2000)
        if c is None:
            break
        got.append(c)
    # completions drained inside the submit loop are not in `got`; order is still monotonic
    seqs = [c[0] for c in got]
    assert seqs == sorted(seqs) and seqs[-1] == 19
    assert [s[1] for s in seen] == list(range(20))
    assert any(c[1] == -1 for c in got if c[0] == 13) or 13 not in seqs   # handler exception -> status -1
    st = w.idle_stats()
    assert st["commands"] == 20 and st["spins"] > 0 and st["yields"] > 0 and st["parks"] > 0, st
    assert w.heartbeat() > hb0
    w.stop()


def test_dp_handle_serves_over_two_cpu_replicas():
    """Two complete CPU engines behind one handle: same tokens as a single engine, both replicas used,
    repeated prompts stick to their replica (prefix affinity)."""
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.engine.handle import EngineHandle
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
    from oxide_tech_llm_engine_b200.parallel.dp_router import DpHandle
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny")
    src = SyntheticSource(mc, seed=2, std=0.08)
    mk = lambda: EngineHandle(LLMEngine(EngineConfig(model="tiny", backend="cpu", max_num_seqs=4, num_kv_blocks=64,
                                                     ctx_size=256), mc, weights=src))
    dp = DpHandle([mk(), mk()], affinity_tokens=8)
    single = mk()
    sp = SamplingParams(greedy=True, max_tokens=6, ignore_eos=True)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(3, 900, size=n).tolist() for n in (12, 20, 33, 15)]
    try:
        streams = [dp.submit(p, sp) for p in prompts]
        outs = []
        for st in streams:
            toks = []
            while True:
                ev = st.get(timeout=60)
                if ev.token >= 0:
                    toks.append(ev.token)
                if ev.finished:
                    break
            outs.append(toks)
        ref = [single.generate(p, sp)[0] for p in prompts]
        assert outs == ref
        assert min(dp.router.routed) >= 1 and sum(dp.router.routed) == 4
        first = streams[0].replica
        assert dp.submit(prompts[0], sp).replica == first
        assert dp.max_slots == 8 and dp.healthy
    finally:
        dp.shutdown()
        single.shutdown()


@pytest.mark.parametrize("mode", ["stream", "leave"])
def test_http_front_over_two_engine_ranks(mode):
    """`server --tp 2` on CPU ranks: rank 0 serves HTTP and broadcasts the admitted requests over gloo,
    rank 1 follows; a rank that leaves between steps ends the requests with `rank_failure` and every
    KV block returns to the pool."""
    import os
    import socket
    import subprocess
    import sys

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(here, "mp_front_check.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2"))
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-4000:]
    assert f"FRONT {mode} OK" in out and "FRONT done" in out, out[-4000:]
    assert "FOLLOWER steps=" in out
    if mode == "stream":
        assert "running=0" in out
