"""Worker of the CPU multi-process tests (gloo ranks): pipeline-parallel decoding and ring
attention, each compared against the single-process oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_pipeline(rank, world):
    from oxide_tech_llm_engine_b200._build import host_ext
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.cpu_model import CpuPagedModel
    from oxide_tech_llm_engine_b200.models.reference import ReferenceModel
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
    from oxide_tech_llm_engine_b200.parallel.pipeline import (PipelineComm, StagePlan, broadcast_tokens,
                                                              run_stage_microbatched)

    mc = preset("tiny", n_layers=5)
    src = SyntheticSource(mc, seed=3, std=0.08)
    H = host_ext()
    sc = H.SchedulerConfig()
    sc.num_blocks, sc.max_num_seqs, sc.enable_radix = 64, 4, False
    sched = H.Scheduler(sc)            # replicated: every stage schedules the same requests
    model = CpuPagedModel(mc, src, 64)  # each stage only touches the KV of its own layers
    plan_ = StagePlan(world, rank, mc.n_layers)
    comm = PipelineComm(rank - 1 if rank > 0 else None, rank + 1 if rank < world - 1 else None)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 1000, size=n).tolist() for n in (9, 30)]
    for i, p in enumerate(prompts):
        sched.add_request(i, np.asarray(p, dtype=np.int32), 6, [], True)
    outs = {0: [], 1: []}
    while sched.has_work():
        plan = sched.schedule()
        n_rows = plan.logit_rows.size
        res = run_stage_microbatched(
            plan_, comm, [plan],
            first_fn=lambda mb: model.forward_plan(mb, layer_range=plan_.layers, return_hidden=not plan_.last),
            mid_fn=lambda mb, h: model.forward_plan(mb, layer_range=plan_.layers, x_in=h, return_hidden=not plan_.last),
            hidden_like=lambda mb: torch.empty(mb.n_tokens, mc.d_model))
        toks = torch.zeros(n_rows, dtype=torch.int32)
        if plan_.last:
            toks = res[0].argmax(-1).to(torch.int32)
        broadcast_tokens(toks, world - 1)
        for e in sched.update(plan, toks.numpy()):
            outs[e.req_id].append(e.token)
    if rank == 0:
        ref = [ReferenceModel(mc, src).generate_greedy(p, 6) for p in prompts]
        assert [outs[0], outs[1]] == ref, (outs, ref)
        assert plan_.layers == (0, 3) if world == 2 else True
        print("PP_OK", flush=True)


def run_ring(rank, world):
    from oxide_tech_llm_engine_b200.parallel.ring_attention import partial_attention, ring_attention, zigzag_chunks

    torch.manual_seed(0)
    T, H, Hkv, D = 64 * world, 4, 2, 16
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if os.environ.get("OXB_RING_GPU") else "cpu"
    q, k, v = (torch.randn(T, H, D).to(dev), torch.randn(T, Hkv, D).to(dev), torch.randn(T, Hkv, D).to(dev))
    pos = torch.arange(T, device=dev)
    chunk = T // (2 * world)
    a, b = zigzag_chunks(world, rank)
    idx = torch.cat([pos[a * chunk:(a + 1) * chunk], pos[b * chunk:(b + 1) * chunk]])
    o = ring_attention(q[idx], k[idx], v[idx], idx, idx, rank=rank, cp=world)
    full, _ = partial_attention(q, k, v, pos, pos, 1.0 / D ** 0.5)
    err = (o - full[idx]).abs().max().item()
    assert err < 1e-4, err
    # causal work is balanced: every rank holds one early and one late chunk
    assert a + b == 2 * world - 1
    dist.barrier()
    if rank == 0:
        print("RING_OK", flush=True)


def run_rank_exit(rank, world):
    """Rank `world-1` leaves between steps; the others learn of it on the host before their next
    collective, fail their in-flight requests with a typed error and return every KV block."""
    import time
    from datetime import timedelta

    from oxide_tech_llm_engine_b200._build import host_ext
    from oxide_tech_llm_engine_b200.parallel.watchdog import Heartbeat, RankFailure, RankMonitor

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, rank == 0,
                          timeout=timedelta(seconds=30))
    hb = Heartbeat(store, rank, period_s=0.02).start()
    mon = RankMonitor(store, rank, world, timeout_s=0.5)
    H = host_ext()
    sc = H.SchedulerConfig()
    sc.num_blocks, sc.max_num_seqs, sc.enable_radix = 64, 4, False
    sched = H.Scheduler(sc)
    free0 = sched.num_free_blocks()
    sched.add_request(0, np.arange(3, 40, dtype=np.int32), 50, [], True)
    victim = world - 1
    steps, failure = 0, None
    x = torch.ones(4)
    t0 = time.monotonic()
    while sched.has_work() and time.monotonic() - t0 < 20:
        if rank == victim and steps == 3:
            hb.leave()          # between steps, nothing in flight
            break
        try:
            mon.check()         # host-side check BEFORE the collective
        except RankFailure as e:
            failure = e
            break
        plan = sched.schedule()
        if rank != victim or steps < 3:
            # the "collective" of the step among ranks that are still in the job
            dist.all_reduce(x) if steps < 3 else None
        toks = np.full(plan.logit_rows.size, 7, dtype=np.int32)
        sched.update(plan, toks)
        steps += 1
        time.sleep(0.05)
    if rank != victim:
        assert failure is not None and failure.rank == victim, (rank, failure, steps)
        ok, ev = sched.cancel(0)
        assert ok and ev and ev[0].finished
        assert sched.num_free_blocks() == free0
        hb.stop()
        print(f"RANK_EXIT_OK rank={rank} steps={steps} reason={failure.reason}", flush=True)
        store.set(f"done/{rank}", "1")
    else:
        # keep the store's client alive until the survivors have finished reading it
        for r in range(world - 1):
            store.wait([f"done/{r}"], timedelta(seconds=20))
    if rank == 0:
        time.sleep(0.3)


def run_ulysses(rank, world):
    from oxide_tech_llm_engine_b200.parallel.ring_attention import partial_attention
    from oxide_tech_llm_engine_b200.parallel.ulysses import ulysses_attention

    torch.manual_seed(0)
    T, H, Hkv, D = 48 * world, 4 * world, 2 * world, 16
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if os.environ.get("OXB_RING_GPU") else "cpu"
    q, k, v = (torch.randn(T, H, D).to(dev), torch.randn(T, Hkv, D).to(dev), torch.randn(T, Hkv, D).to(dev))
    tl = T // world
    sl = slice(rank * tl, (rank + 1) * tl)
    o = ulysses_attention(q[sl], k[sl], v[sl], rank=rank, cp=world)
    pos = torch.arange(T, device=dev)
    full, _ = partial_attention(q, k, v, pos, pos, 1.0 / D ** 0.5)
    err = (o - full[sl]).abs().max().item()
    assert o.shape == (tl, H, D) and err < 1e-4, err
    dist.barrier()
    if rank == 0:
        print("ULYSSES_OK", flush=True)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if os.environ.get("OXB_RING_GPU"):
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
        {"ring": run_ring, "ulysses": run_ulysses}[sys.argv[1]](rank, world)
        dist.barrier()
        dist.destroy_process_group()
        return
    if sys.argv[1] == "rank_exit":
        dist.init_process_group("gloo")
        run_rank_exit(rank, world)
        os._exit(0)  # survivors do not run a collective teardown with a rank that is gone
    dist.init_process_group("gloo")
    {"pipeline": run_pipeline, "ring": run_ring, "ulysses": run_ulysses}[sys.argv[1]](rank, world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
