"""C++ host runtime: block pool, sequence block tables, radix prefix cache, scheduler core (CPU)."""
import threading

import numpy as np
import pytest

from oxide_tech_llm_engine_b200._build import host_ext


@pytest.fixture(scope="module")
def H():
    return host_ext()


def test_block_pool_refcounts(H):
    p = H.BlockPool(4)
    a, b = p.allocate(), p.allocate()
    assert p.num_free() == 2 and p.ref_count(a) == 1
    p.retain(a)
    assert not p.release(a) and p.ref_count(a) == 1
    assert p.release(a) and p.num_free() == 3
    with pytest.raises(RuntimeError):
        p.release(a)
    c, d, e = p.allocate(), p.allocate(), p.allocate()
    assert p.allocate() == -1 and {b, c, d, e} == {0, 1, 2, 3}


def test_block_pool_threaded_soak(H):
    # fork/release storm from 8 threads: every block must come home
    p = H.BlockPool(64)
    def work():
        for _ in range(2000):
            b = p.allocate()
            if b >= 0:
                p.retain(b)
                p.release(b)
                p.release(b)
    ts = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert p.num_free() == 64


def test_sequence_table_advance_rewind_cow(H):
    p = H.BlockPool(8)
    t = H.SequenceBlockTable(p)
    ok, cow = t.advance(20)
    assert ok and len(t.blocks()) == 2 and not cow
    t.commit()
    ok, _ = t.advance(30)  # speculative growth
    assert len(t.blocks()) == 4 and t.num_tokens() == 50
    t.rollback()
    assert t.num_tokens() == 20 and len(t.blocks()) == 2 and p.num_free() == 6
    # a second table adopts the (partial) prefix; writing into the shared tail block forks it
    u = H.SequenceBlockTable(p)
    u.adopt_prefix(t.blocks(), 20)
    assert p.ref_count(t.blocks()[1]) == 2
    ok, cow = u.advance(1)
    assert ok and cow == [(t.blocks()[1], u.blocks()[1])] and u.blocks()[0] == t.blocks()[0]
    # exhaustion leaves the table untouched
    big = H.SequenceBlockTable(p)
    ok, _ = big.advance(16 * 100)
    assert not ok and big.num_tokens() == 0
    u.release_all(); t.release_all()
    assert p.num_free() == 8


def test_h2o_prune_keeps_sinks_heavy_hitters_and_tail(H):
    p = H.BlockPool(64)
    t = H.SequenceBlockTable(p)
    t.advance(16 * 20 - 5)
    scores = [0.0] * 20
    scores[7], scores[11] = 9.0, 5.0
    kept = t.prune_heavy_hitters(scores, sink_blocks=2, rolling_blocks=3, budget_blocks=7)
    assert kept == [0, 1, 7, 11, 17, 18, 19]
    assert t.num_tokens() == 16 * 6 + 11 and p.num_free() == 64 - 7


def test_radix_match_insert_split_evict(H):
    p = H.BlockPool(32)
    r = H.RadixCache(p)
    toks = np.arange(64, dtype=np.int32)
    blocks = [p.allocate() for _ in range(4)]
    assert r.insert(toks, blocks) == 4 and r.cached_blocks() == 4
    got, n = r.match(toks, True)
    assert n == 48 and got == blocks[:3]          # never the whole prompt
    got, n = r.match(np.concatenate([toks, [1, 2]]).astype(np.int32), True)
    assert n == 64 and got == blocks
    # diverge inside the second block: only the first block matches; inserting splits the node
    other = toks.copy(); other[20] = 999
    got, n = r.match(other, True)
    assert n == 16 and got == blocks[:1]
    ob = [blocks[0]] + [p.allocate() for _ in range(3)]
    assert r.insert(other, ob) == 3 and r.num_nodes() == 3
    # blocks still referenced by a sequence cannot be evicted
    assert r.evict(100) == 0
    for b in blocks + ob[1:]:
        p.release(b)
    assert r.evict(3) >= 3
    freed_total = 7 - r.cached_blocks()
    assert p.num_free() == 32 - 7 + freed_total
    r.clear()
    assert p.num_free() == 32 and r.cached_blocks() == 0


def test_prefill_budget_formula(H):
    c = H.SchedulerConfig()
    c.num_blocks = 64
    s = H.Scheduler(c)
    # clamp(min((25000 - (2000 + 350 B)) / 25, 2048 - B), 32, 512)
    assert s.prefill_budget(0) == 512
    assert s.prefill_budget(40) == int((25000 - (2000 + 350 * 40)) / 25)
    assert s.prefill_budget(64) == 32       # SLA exhausted -> floor
    assert s.prefill_budget(2048) == 0
    c.sla_budget = False
    assert H.Scheduler(c).prefill_budget(10) == 2038


def _drain(s, H, answer=lambda rid, row: 7):
    events = []
    for _ in range(10000):
        if not s.has_work():
            break
        plan = s.schedule()
        early = s.take_events()
        events += early
        if plan.n_tokens == 0:
            if early:
                continue
            break
        toks = np.array([answer(int(r), i) for i, r in enumerate(plan.logit_req)], dtype=np.int32)
        events += s.update(plan, toks)
    return events


def test_scheduler_lifecycle_and_stop_rules(H):
    c = H.SchedulerConfig()
    c.num_blocks, c.max_num_seqs, c.chunk_max, c.chunk_min = 64, 4, 16, 8
    s = H.Scheduler(c)
    s.add_request(1, np.arange(40, dtype=np.int32), 5, [99], False)
    s.add_request(2, np.arange(3, dtype=np.int32), 50, [7], False)     # stops on token 7 at once
    plan = s.schedule()
    assert plan.n_prefill >= 1 and plan.n_decode == 0 and plan.q_lens[0] == 16   # chunked by chunk_max
    ev = s.update(plan, np.full(plan.logit_rows.size, 7, dtype=np.int32))
    ev += _drain(s, H)
    by = {}
    for e in ev:
        by.setdefault(e.req_id, []).append(e)
    assert [e.token for e in by[1]] == [7] * 5 and by[1][-1].finished and by[1][-1].reason == "length"
    assert len(by[2]) == 1 and by[2][0].reason == "stop"
    assert s.num_free_blocks() + s.radix_stats()["cached_blocks"] == 64 and not s.has_work()


def test_scheduler_prefix_reuse_and_cancel(H):
    c = H.SchedulerConfig()
    c.num_blocks, c.max_num_seqs = 64, 4
    s = H.Scheduler(c)
    prompt = np.arange(50, dtype=np.int32)
    s.add_request(1, prompt, 3, [], True)
    _drain(s, H)
    s.add_request(2, np.concatenate([prompt, [5, 6, 7]]).astype(np.int32), 3, [], True)
    plan = s.schedule()
    info = s.request_info(2)
    assert info["prefix_hit"] == 48 and plan.q_lens[0] == 5 and plan.ctx_lens[0] == 53
    ok, ev = s.cancel(2)
    assert ok and ev[0].reason == "cancelled" and not s.has_work()
    assert s.radix_stats()["hit_tokens"] == 48


def test_scheduler_preempts_youngest_when_kv_runs_out(H):
    c = H.SchedulerConfig()
    c.num_blocks, c.max_num_seqs, c.enable_radix = 6, 4, False
    s = H.Scheduler(c)
    for rid in (1, 2, 3):
        s.add_request(rid, np.arange(30, dtype=np.int32), 40, [], True)
    ev = _drain(s, H)
    done = {e.req_id for e in ev if e.finished}
    assert done == {1, 2, 3} and s.preemptions() > 0
    counts = {rid: sum(1 for e in ev if e.req_id == rid and e.token >= 0) for rid in (1, 2, 3)}
    assert counts == {1: 40, 2: 40, 3: 40}
    assert s.num_free_blocks() == 6


def test_two_long_prefills_that_fill_the_pool_both_finish(H):
    """Two prompts that each fit the pool alone but not together: the younger one is preempted when
    the older one's next chunk finds no block, instead of both waiting on each other."""
    c = H.SchedulerConfig()
    c.num_blocks, c.enable_radix = 100, False
    s = H.Scheduler(c)
    for rid in (1, 2):
        s.add_request(rid, np.arange(1500, dtype=np.int32), 4, [], True)
    ev = _drain(s, H)
    assert {e.req_id for e in ev if e.finished} == {1, 2} and not s.has_work()
    assert all(e.reason == "length" for e in ev if e.finished)
    assert s.preemptions() > 0 and s.num_free_blocks() == 100


def test_request_that_can_never_fit_is_ended_not_spun_on(H):
    c = H.SchedulerConfig()
    c.num_blocks, c.enable_radix, c.chunk_max = 4, False, 32
    s = H.Scheduler(c)
    s.add_request(1, np.arange(200, dtype=np.int32), 4, [], True)   # 13 blocks needed, 4 exist
    s.add_request(2, np.arange(20, dtype=np.int32), 3, [], True)
    ev = _drain(s, H)
    by = {e.req_id: e for e in ev if e.finished}
    assert by[1].reason.startswith("prefill_error") and by[2].reason == "length"
    assert not s.has_work() and s.num_free_blocks() == 4
    # a decoding request that outgrows a pool it has to itself ends with "length"
    s.add_request(3, np.arange(40, dtype=np.int32), 500, [], True)
    ev = _drain(s, H)
    fin = [e for e in ev if e.finished]
    assert len(fin) == 1 and fin[0].req_id == 3 and fin[0].reason == "length"
    assert sum(1 for e in ev if e.token >= 0) == 4 * 16 - 40 + 1 and s.num_free_blocks() == 4


def test_forced_tokens_are_prefilled_as_one_chunk(H):
    c = H.SchedulerConfig()
    c.num_blocks, c.enable_radix = 32, False
    s = H.Scheduler(c)
    s.add_request(1, np.arange(10, dtype=np.int32), 20, [99], False)
    plan = s.schedule()
    s.update(plan, np.array([100], dtype=np.int32))
    ev = s.append_forced(1, [201, 202, 203])
    assert [e.token for e in ev] == [201, 202, 203] and not any(e.finished for e in ev)
    plan = s.schedule()
    assert plan.n_decode == 0 and plan.n_prefill == 1 and plan.q_lens[0] == 4 and plan.logit_rows.size == 1
    assert list(plan.token_ids) == [100, 201, 202, 203] and list(plan.positions) == [10, 11, 12, 13]
    ev = s.update(plan, np.array([300], dtype=np.int32))
    assert [e.token for e in ev] == [300]
    info = s.request_info(1)
    assert info["computed"] == 14 and info["generated"] == 5 and info["phase"] == 2
    plan = s.schedule()
    assert plan.n_decode == 1 and list(plan.token_ids) == [300]
    s.update(plan, np.array([7], dtype=np.int32))
    ev = s.append_forced(1, [5, 99, 6])   # a forced stop id ends the request
    assert [e.token for e in ev] == [5, 99] and ev[-1].finished and ev[-1].reason == "stop"
    assert not s.has_work() and s.num_free_blocks() == 32


def test_scheduler_speculative_accept_and_rollback(H):
    c = H.SchedulerConfig()
    c.num_blocks, c.enable_radix = 32, False
    s = H.Scheduler(c)
    s.add_request(1, np.arange(10, dtype=np.int32), 20, [], True)
    plan = s.schedule()
    s.update(plan, np.array([100], dtype=np.int32))
    s.set_drafts(1, [101, 102, 555, 104])
    plan = s.schedule()
    assert plan.n_decode == 0 and plan.n_prefill == 1 and plan.q_lens[0] == 5 and plan.logit_rows.size == 5
    assert list(plan.token_ids) == [100, 101, 102, 555, 104]
    ev = s.update(plan, np.array([101, 102, 103, 0, 0], dtype=np.int32))  # accepts 2 drafts + bonus
    assert [e.token for e in ev] == [101, 102, 103]
    info = s.request_info(1)
    assert info["computed"] == 13 and info["generated"] == 4
    assert len(info["blocks"]) == 1


def test_scheduler_reserve_ahead_holds_blocks_for_a_decode_burst(H):
    """reserve_ahead: the next decode plans allocate nothing, the first plan's table already lists the
    held blocks, budgets and the pool bound the reservation, and everything returns at the end."""
    sc = H.SchedulerConfig()
    sc.num_blocks, sc.max_num_seqs, sc.max_blocks_per_seq, sc.enable_radix = 12, 4, 16, False
    s = H.Scheduler(sc)
    rid = 5
    s.add_request(rid, np.arange(1, 21, dtype=np.int32), 40, [], True)   # 20 prompt tokens, 40 new
    assert s.reserve_ahead(rid, 8) == 0                              # still in prefill
    plan = s.schedule()
    s.update(plan, np.array([7], dtype=np.int32))
    free = s.num_free_blocks()
    assert s.reserve_ahead(rid, 30) == 30                            # 21 + 30 tokens -> 4 blocks
    assert free - s.num_free_blocks() == 2
    plan = s.schedule()
    assert plan.n_decode == 1 and plan.max_blocks == 4 and s.num_free_blocks() == free - 2
    for t in range(29):
        s.update(plan, np.array([9 + t], dtype=np.int32))
        plan = s.schedule()
        assert s.num_free_blocks() == free - 2                       # no allocation inside the burst
    assert s.reserve_ahead(rid, 100) == 10                           # bounded by the 10 tokens left of the budget
    ok, _ = s.cancel(rid)
    assert ok and s.num_free_blocks() == 12


def test_radix_eviction_log_and_adoption(H):
    """The two hooks of the KV tiers: evictions are logged with the whole token prefix their blocks
    complete, and `radix_adopt` turns a prefix back into cached blocks that the next admission hits."""
    sc = H.SchedulerConfig()
    sc.num_blocks, sc.max_num_seqs, sc.max_blocks_per_seq, sc.enable_radix = 16, 2, 16, True
    s = H.Scheduler(sc)
    s.record_evictions(True)
    a = np.arange(100, 100 + 70, dtype=np.int32)            # 4 full blocks + 6 tokens
    s.add_request(1, a, 2, [], True)
    _ = _drain(s, H)
    assert s.radix_stats()["cached_blocks"] == 4 and s.radix_cached_blocks(a[:64]) == 4
    assert s.take_evicted() == []
    # two other prompts need the pool: the cached prefix has to go
    for rid, base in ((2, 1000), (3, 2000)):
        s.add_request(rid, np.arange(base, base + 120, dtype=np.int32), 2, [], True)
        _ = _drain(s, H)
    ev = s.take_evicted()
    gone = [(np.asarray(t).tolist(), first, list(blocks)) for t, first, blocks in ev if np.asarray(t)[0] == 100]
    assert gone, ev
    covered = set()
    for toks, first, blocks in gone:
        assert len(toks) % 16 == 0 and toks == a[:len(toks)].tolist()      # the prefix up to the end of the leaf
        assert len(toks) // 16 == first + len(blocks)
        covered.update(range(first, first + len(blocks)))
    assert covered == {0, 1, 2, 3} and s.radix_cached_blocks(a[:64]) == 0
    # adoption: three blocks come back (the pool is asked for exactly three)
    free = s.num_free_blocks()
    ids = s.radix_adopt(a[:48], 3)
    assert len(ids) == 3 and len(set(ids)) == 3 and s.num_free_blocks() == free - 3
    assert s.radix_cached_blocks(a[:64]) == 3 and s.radix_adopt(a[:48], 3) == []   # already there
    s.add_request(4, a, 1, [], True)
    plan = s.schedule()
    assert plan.n_prefill == 1 and int(plan.q_lens[0]) == 70 - 48           # only the uncached tail is computed
    assert [int(b) for b in plan.prefill_block_tables.reshape(-1)[:3]] == [int(b) for b in ids]


def test_scheduler_fault_injection_isolated(H):
    c = H.SchedulerConfig()
    c.num_blocks = 32
    s = H.Scheduler(c)
    s.add_request(1, np.arange(20, dtype=np.int32), 4, [], True)
    s.add_request(2, np.arange(20, 40, dtype=np.int32), 4, [], True)
    s.inject_prefill_error(1, "injected")
    ev = _drain(s, H)
    r1 = [e for e in ev if e.req_id == 1]
    r2 = [e for e in ev if e.req_id == 2]
    assert len(r1) == 1 and r1[0].finished and r1[0].reason == "prefill_error: injected"
    assert len(r2) == 4 and r2[-1].reason == "length"
    assert s.num_free_blocks() + s.radix_stats()["cached_blocks"] == 32


def test_scheduler_heavy_hitter_pruning_keeps_positions_absolute():
    """Pruning a decoding request returns its low-score middle blocks, later tokens keep their
    absolute positions while the KV index and the context length shrink by what was dropped."""
    import numpy as np

    from oxide_tech_llm_engine_b200._build import host_ext

    H = host_ext()
    sc = H.SchedulerConfig()
    sc.num_blocks, sc.max_num_seqs, sc.enable_radix, sc.max_num_batched_tokens = 64, 2, True, 512
    sc.sla_budget = False
    sc.chunk_max = 512
    s = H.Scheduler(sc)
    free0 = s.num_free_blocks()
    s.add_request(7, np.arange(3, 3 + 200, dtype=np.int32), 40, [], True)   # 200 tokens -> 13 blocks
    plan = s.schedule()
    s.update(plan, np.asarray([5], dtype=np.int32))
    info = s.request_info(7)
    assert info["phase"] == 2 and len(info["blocks"]) == 13 and info["dropped"] == 0
    before = list(info["blocks"])
    scores = [0.0] * 13
    scores[5], scores[8] = 9.0, 7.0                                         # the heavy hitters
    keep = s.prune_request(7, scores, 1, 2, 6)                              # sink 1 + rolling 2 + 3 best
    assert keep == [0, 1, 5, 8, 11, 12]                                      # stable: the tie goes to the earliest block
    info = s.request_info(7)
    assert info["blocks"] == [before[i] for i in keep] and info["dropped"] == 7 * 16
    assert s.num_free_blocks() >= free0 - 6 - 13      # 7 blocks went back (the radix cache may still pin shared ones)
    plan = s.schedule()
    assert plan.n_decode == 1
    assert plan.positions[0] == 200                                          # absolute position
    assert plan.decode_seq_lens[0] == 201 - 112                              # keys that are left
    kv = 200 - 112
    assert plan.slot_mapping[0] == info["blocks"][kv // 16] * 16 + kv % 16
    s.update(plan, np.asarray([6], dtype=np.int32))
    s.set_drafts(7, [1, 2, 3])                                               # ignored for a pruned request
    assert s.schedule().n_prefill == 0
    ok, ev = s.cancel(7)
    assert ok
    assert s.prune_request(7, scores, 1, 2, 6) == []
