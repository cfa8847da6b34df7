"""The whole engine on the CPU backend: scheduler + block manager + radix cache + paged fp32
model + samplers, against the contiguous-cache oracle (no GPU)."""
import numpy as np
import pytest

from oxide_tech_llm_engine_b200.config import EngineConfig
from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
from oxide_tech_llm_engine_b200.engine.handle import EngineHandle
from oxide_tech_llm_engine_b200.models.config import preset
from oxide_tech_llm_engine_b200.models.reference import ReferenceModel
from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
from oxide_tech_llm_engine_b200.sampling_params import SamplingParams


def mk(name="tiny", **kw):
    mc = preset(name)
    src = SyntheticSource(mc, seed=3, std=0.08)
    base = dict(backend="cpu", max_num_seqs=4, max_num_batched_tokens=64, chunk_max=32, chunk_min=8,
                num_kv_blocks=96, ctx_size=512)
    base.update(kw)
    return LLMEngine(EngineConfig(**base), mc, weights=src), mc, src


GREEDY = SamplingParams(greedy=True, max_tokens=8, ignore_eos=True)


@pytest.mark.parametrize("name", ["tiny", "tiny-moe"])
def test_paged_engine_equals_oracle(name):
    eng, mc, src = mk(name)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(3, 1000, size=n).tolist() for n in (5, 40, 70, 17, 33)]  # 5 > max_num_seqs
    outs = eng.generate(prompts, GREEDY)
    ref = [ReferenceModel(mc, src).generate_greedy(p, 8) for p in prompts]
    assert outs == ref
    assert eng.sched.num_free_blocks() + eng.sched.radix_stats()["cached_blocks"] == 96


def test_two_clients_get_exactly_max_tokens_and_prefix_reuse():
    eng, mc, src = mk()
    events = {0: [], 1: []}
    p = list(range(10, 60))
    a = eng.add_request(p, SamplingParams(greedy=True, max_tokens=6, ignore_eos=True),
                        on_token=lambda r, e: events[0].append(e))
    b = eng.add_request(p[:20], SamplingParams(greedy=True, max_tokens=9, ignore_eos=True),
                        on_token=lambda r, e: events[1].append(e))
    while eng.has_work():
        eng.step()
    assert len(events[0]) == 6 and len(events[1]) == 9
    assert events[0][-1].finished and events[0][-1].reason == "length" and not events[0][0].finished
    # multi-turn: prompt + answer + new user turn hits the cache
    turn2 = p + eng.requests[a].output + [7, 8, 9]
    eng.generate([turn2], GREEDY)
    st = eng.sched.radix_stats()
    assert st["hit_tokens"] >= 48
    ref = ReferenceModel(mc, src).generate_greedy(turn2, 8)
    assert eng.requests[max(eng.requests)].output == ref


def test_chunked_prefill_interleaves_with_short_request():
    eng, mc, src = mk(chunk_max=8, chunk_min=4, max_num_batched_tokens=12)
    long_p = list(range(100, 190))
    eng.add_request(long_p, GREEDY)
    eng.step()
    short = eng.add_request([5, 6, 7], SamplingParams(greedy=True, max_tokens=3, ignore_eos=True))
    steps = 0
    while not eng.requests[short].finished:
        eng.step()
        steps += 1
    # the short request finished while the long prompt was still being prefilled in 8-token chunks
    assert eng.sched.request_info(0)["computed"] < len(long_p)
    while eng.has_work():
        eng.step()
    assert eng.requests[0].output == ReferenceModel(mc, src).generate_greedy(long_p, 8)


def test_radix_lru_eviction_under_pressure():
    eng, mc, src = mk(num_kv_blocks=24, max_num_seqs=2)
    rng = np.random.default_rng(5)
    for i in range(8):
        eng.generate([rng.integers(3, 1000, size=60).tolist()], SamplingParams(greedy=True, max_tokens=2, ignore_eos=True))
    st = eng.sched.radix_stats()
    assert st["cached_blocks"] <= 24 and eng.sched.num_free_blocks() >= 0
    # everything still works and is correct after evictions
    p = rng.integers(3, 1000, size=50).tolist()
    assert eng.generate([p], GREEDY)[0] == ReferenceModel(mc, src).generate_greedy(p, 8)


def test_preemption_recompute_is_transparent():
    eng, mc, src = mk(num_kv_blocks=10, enable_radix=False, max_num_seqs=3)
    rng = np.random.default_rng(6)
    prompts = [rng.integers(3, 1000, size=40).tolist() for _ in range(3)]
    sp = SamplingParams(greedy=True, max_tokens=30, ignore_eos=True)
    outs = eng.generate(prompts, sp)
    assert eng.sched.preemptions() > 0
    assert outs == [ReferenceModel(mc, src).generate_greedy(p, 30) for p in prompts]


def test_speculative_ngram_equals_plain_greedy():
    eng, mc, src = mk(speculative="ngram")
    rep = [11, 12, 13, 14, 15, 16] * 6
    sp = SamplingParams(greedy=True, max_tokens=20, ignore_eos=True)
    spec = eng.generate([rep], sp)[0]
    assert spec == ReferenceModel(mc, src).generate_greedy(rep, 20)
    assert eng.stats["steps"] > 0
    # the draft length of the request followed its acceptance rate (AdaptiveSpeculator), and the
    # counters add up: never more accepted than proposed, fewer steps than tokens when drafts hit
    r = eng.requests[max(eng.requests)]
    assert r.spec is not None and 1 <= r.spec.k <= 5
    prop, acc = eng.stats.get("spec_proposed", 0), eng.stats.get("spec_accepted", 0)
    assert prop > 0 and 0 <= acc <= prop and r.spec.proposed == prop and r.spec.accepted == acc
    if acc:
        assert eng.stats["steps"] < 20 + 3


def test_sampling_seed_determinism_and_stop_ids():
    eng, mc, src = mk()
    p = list(range(20, 40))
    sp = SamplingParams(temperature=0.9, top_k=30, top_p=0.9, min_p=0.02, seed=7, max_tokens=10, ignore_eos=True)
    a = eng.generate([p], sp)[0]
    b = eng.generate([p], sp)[0]
    c = eng.generate([p], SamplingParams(temperature=0.9, top_k=30, top_p=0.9, min_p=0.02, seed=8, max_tokens=10,
                                         ignore_eos=True))[0]
    assert a == b and len(a) == 10 and a != c
    first = ReferenceModel(mc, src).generate_greedy(p, 1)[0]
    out = eng.generate([p], SamplingParams(greedy=True, max_tokens=10, stop_token_ids=[first]))[0]
    assert out == [first] and eng.requests[max(eng.requests)].finish_reason == "stop"


def test_cancel_and_prefill_fault_free_everything():
    eng, mc, src = mk()
    free0 = eng.sched.num_free_blocks()
    rid = eng.add_request(list(range(50)), SamplingParams(greedy=True, max_tokens=100, ignore_eos=True))
    other = eng.add_request(list(range(60, 90)), GREEDY)
    eng.step()
    eng.sched.inject_prefill_error(rid, "boom")
    while eng.has_work():
        eng.step()
    assert eng.requests[rid].finish_reason == "prefill_error: boom"
    assert eng.requests[other].output == ReferenceModel(mc, src).generate_greedy(list(range(60, 90)), 8)
    rid2 = eng.add_request(list(range(50)), SamplingParams(greedy=True, max_tokens=100, ignore_eos=True))
    eng.step(); eng.step()
    assert eng.cancel(rid2) and not eng.has_work()
    assert eng.sched.num_free_blocks() + eng.sched.radix_stats()["cached_blocks"] == free0


def test_engine_handle_threads_and_failure_isolation():
    eng, mc, src = mk()
    h = EngineHandle(eng)
    try:
        p = list(range(30, 50))
        out, reason = h.generate(p, GREEDY)
        assert out == ReferenceModel(mc, src).generate_greedy(p, 8) and reason == "length"
        # an inadmissible request (empty prompt) fails alone
        st = h.submit([], GREEDY)
        ev = st.get(timeout=30)
        assert ev.finished and ev.reason.startswith("prefill_error")
        out2, _ = h.generate(p, GREEDY)
        assert out2 == out and h.active_slots() == 0
    finally:
        h.shutdown()


def test_grammar_constrained_json_is_valid():
    import json

    from oxide_tech_llm_engine_b200.tokenizer import Tokenizer

    eng, mc, src = mk()
    tok = Tokenizer.ascii_fallback(mc.vocab_size)
    eng.set_tokenizer(tok)
    sp = SamplingParams(temperature=0.8, top_k=50, seed=3, max_tokens=60, grammar='json_prefix:{"a": "', ignore_eos=True)
    rid = eng.add_request(tok.encode("give json"), sp)
    while eng.has_work():
        eng.step()
        r = eng.requests[rid]
        if r.grammar.done():
            eng.cancel(rid)
    text = tok.decode(eng.requests[rid].output)
    assert text.startswith('{"a": "')
    if eng.requests[rid].grammar.done():
        json.loads(text)


def test_grammar_jump_forward_skips_sampling_and_ends_on_accept():
    """Bytes the grammar forces are appended without a forward pass each (the fixed prefix takes
    one prefill chunk instead of one decode step per token); an accepting state ends the request
    with "stop"; the text is the same as with jump-forward off."""
    import json

    from oxide_tech_llm_engine_b200.tokenizer import Tokenizer

    outs, steps = [], []
    for jf in (True, False):
        eng, mc, src = mk(jump_forward=jf)
        tok = Tokenizer.ascii_fallback(mc.vocab_size)
        eng.set_tokenizer(tok)
        sp = SamplingParams(greedy=True, max_tokens=80, grammar='json_prefix:{"answer": "', ignore_eos=True)
        rid = eng.add_request(tok.encode("q"), sp)
        n = 0
        while eng.has_work() and n < 200:
            eng.step()
            n += 1
        r = eng.requests[rid]
        outs.append(tok.decode(r.output))
        steps.append(eng.stats["steps"])
        assert r.finished and eng.sched.num_free_blocks() + eng.sched.radix_stats()["cached_blocks"] == 96
        if jf:
            assert eng.stats.get("jump_forward_tokens", 0) >= 8
        if r.finish_reason == "stop":
            json.loads(outs[-1])
    assert outs[0].startswith('{"answer": "') and outs[0] == outs[1]
    assert steps[0] < steps[1]


def test_engine_fails_loudly_when_the_scheduler_cannot_progress():
    from oxide_tech_llm_engine_b200.errors import EngineError

    eng, mc, src = mk(num_kv_blocks=8)
    rid = eng.add_request(list(range(1, 300)), GREEDY)     # 19 blocks needed, 8 exist
    rid2 = eng.add_request(list(range(1, 20)), GREEDY)
    outs = eng.generate([], GREEDY, max_steps=100)
    assert outs == [] and not eng.has_work()
    assert eng.requests[rid].finished and eng.requests[rid].finish_reason.startswith("prefill_error")
    assert eng.requests[rid2].finish_reason == "length" and len(eng.requests[rid2].output) == 8
    # an empty plan with queued work is reported, not spun on
    class Stuck:
        def __getattr__(self, k):
            return getattr(eng_sched, k)
        def schedule(self):
            return empty_plan
        def take_events(self):
            return []
        def has_work(self):
            return True
    eng_sched = eng.sched
    empty_plan = eng.sched.schedule()
    assert empty_plan.n_tokens == 0
    eng.sched = Stuck()
    with pytest.raises(EngineError, match="no progress"):
        for _ in range(10):
            eng.step()


def test_monitor_failure_fails_requests_and_returns_blocks():
    """A peer that stops answering is found before the step: requests end with a typed reason and
    every KV block goes back to the pool."""
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
    from oxide_tech_llm_engine_b200.parallel.watchdog import RankFailure
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny")
    eng = LLMEngine(EngineConfig(model="tiny", backend="cpu", max_num_seqs=4, num_kv_blocks=64, ctx_size=256),
                    mc, weights=SyntheticSource(mc, seed=1, std=0.08))
    free0 = eng.sched.num_free_blocks()
    eng.add_request(list(range(3, 30)), SamplingParams(greedy=True, max_tokens=20, ignore_eos=True))
    eng.step()
    assert eng.sched.num_free_blocks() < free0

    class Mon:
        def check(self):
            raise RankFailure(1, "missed heartbeats for 1.00s")
    eng.attach_monitor(Mon())
    import pytest as _pt
    with _pt.raises(RankFailure):
        eng.step()
    cached = eng.sched.radix_stats()["cached_blocks"]   # full prompt blocks stay in the prefix cache
    assert eng.sched.num_free_blocks() + cached == free0 and not eng.has_work()
    assert "rank_failure" in eng.degraded
    eng.close()


def test_h2o_pruning_bounds_the_kv_of_a_long_sequence_on_cpu():
    """With heavy-hitter pruning on, a sequence never holds more than the block budget (+1 for the
    block being filled), the pool gets the rest back and decoding continues to the requested length."""
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny")
    eng = LLMEngine(EngineConfig(model="tiny", backend="cpu", max_num_seqs=2, num_kv_blocks=64, ctx_size=512,
                                 enable_radix=False, h2o_pruning=True, h2o_budget_blocks=6, h2o_sink_blocks=1,
                                 h2o_rolling_blocks=2), mc, weights=SyntheticSource(mc, seed=4, std=0.08))
    rid = eng.add_request(list(range(3, 3 + 150)), SamplingParams(greedy=True, max_tokens=40, ignore_eos=True))
    most = 0
    while eng.has_work():
        eng.step()
        info = eng.sched.request_info(rid)
        if info is not None:
            most = max(most, len(info["blocks"])) if info["dropped"] else most
            if info["dropped"]:
                assert len(info["blocks"]) <= 7
    assert eng.stats.get("h2o_pruned_blocks", 0) >= 4 and 0 < most <= 7
    assert len(eng.requests[rid].output) == 40
    assert eng.sched.num_free_blocks() == 64
    eng.close()


def test_nvfp4_moe_gguf_round_trip_on_cpu():
    import os
    import tempfile

    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.reference import ReferenceModel
    from oxide_tech_llm_engine_b200.models.weights import open_weights, write_synthetic_gguf
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny-moe")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        write_synthetic_gguf(path, mc, seed=5, weight_type="NVFP4", embed_type="Q8_0", std=0.08)
        src = open_weights(path)
        assert src.type_name("blk.0.ffn_down_exps.weight") == "NVFP4" and src.cfg.n_experts == mc.n_experts
        eng = LLMEngine(EngineConfig(model=path, backend="cpu", max_num_seqs=2, num_kv_blocks=32, ctx_size=128),
                        src.cfg, weights=src)
        p = list(range(5, 25))
        out = eng.generate([p], SamplingParams(greedy=True, max_tokens=6, ignore_eos=True))[0]
        assert out == ReferenceModel(src.cfg, src).generate_greedy(p, 6)
        eng.close()


def test_context_shift_keeps_a_sequence_going_past_its_window():
    """At the context limit the sequence keeps its first block and drops the oldest ones after it
    (whole 16-token blocks) instead of ending: it generates far beyond the window with bounded KV."""
    eng, mc, src = mk(ctx_size=64, num_kv_blocks=32, context_shift=True, shift_keep_tokens=4, shift_step_tokens=16,
                      enable_radix=False)
    sp = SamplingParams(greedy=True, max_tokens=150, ignore_eos=True)
    rid = eng.add_request(list(range(3, 33)), sp)
    peak = 0
    while eng.has_work():
        eng.step()
        info = eng.sched.request_info(rid)
        if info is not None:
            peak = max(peak, len(info["blocks"]))
            assert info["computed"] - info["dropped"] <= 64
    r = eng.requests[rid]
    assert r.finished and r.finish_reason == "length" and len(r.output) == 150
    assert peak <= 4 and eng.sched.context_shifts() >= 5
    assert eng.sched.num_free_blocks() == 32
    # without the shift the same request stops at the window
    eng2, _, _ = mk(ctx_size=64, num_kv_blocks=32, enable_radix=False)
    out2 = eng2.generate([list(range(3, 33))], sp)[0]
    assert len(out2) < 40 and out2 == r.output[:len(out2)]


def test_engine_handle_runs_steps_on_the_native_worker_thread():
    """The C++ StepWorker carries the engine steps (scheduler actor -> SPSC ring -> worker thread):
    same tokens as stepping on the handle's own thread, failures stay isolated per request."""
    eng, mc, src = mk()
    ref_eng, _, _ = mk()
    want = ref_eng.generate([[5, 6, 7, 8], [9, 10, 11]], GREEDY)
    h = EngineHandle(eng, native_worker=True)
    try:
        a = h.submit([5, 6, 7, 8], GREEDY)
        b = h.submit([9, 10, 11], GREEDY)
        outs = []
        for st in (a, b):
            toks = []
            while True:
                ev = st.get(timeout=60)
                if ev.token >= 0:
                    toks.append(ev.token)
                if ev.finished:
                    break
            outs.append(toks)
        assert outs == want
        assert h._worker is not None and h._worker.idle_stats()["commands"] >= 8
        rid = h.submit([1, 2, 3], GREEDY)
        eng.sched.inject_prefill_error(rid.req_id, "boom")
        ev = rid.get(timeout=60)
        assert ev.finished and ev.reason.startswith("prefill_error")
        assert h.generate([5, 6, 7, 8], GREEDY)[0] == want[0]
    finally:
        h.shutdown()


def test_kv_blocks_evicted_from_the_prefix_cache_come_back_from_the_host_tier(tmp_path):
    """Tier 1 -> 2 -> 3 -> 1: prompts push an older prompt's blocks out of the device prefix cache,
    the engine copies them to the host tier (and, beyond its capacity, to files); when the old
    prompt returns its blocks are copied back into fresh device blocks, the prefill shrinks to the
    uncached tail and the tokens are those of the first run."""
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny")
    rng = np.random.default_rng(8)
    old = rng.integers(3, mc.vocab_size, size=100).tolist()                      # 6 full blocks + 4 tokens
    others = [rng.integers(3, mc.vocab_size, size=120).tolist() for _ in range(4)]
    sp = SamplingParams(greedy=True, max_tokens=4, ignore_eos=True)

    def run(**kw):
        eng = LLMEngine(EngineConfig(model="tiny", backend="cpu", max_num_seqs=1, num_kv_blocks=20, ctx_size=256,
                                     enable_radix=True, **kw), mc, weights=SyntheticSource(mc, seed=4, std=0.08))
        first = eng.generate([old], sp)[0]
        for p in others:
            eng.generate([p], sp)
        before = eng.stats["prefill_tokens"]
        again = eng.generate([old], sp)[0]
        return eng, first, again, eng.stats["prefill_tokens"] - before

    plain, first, again, cost_plain = run()
    assert again == first and cost_plain == 100          # evicted and gone: the whole prompt is prefilled again
    plain.close()
    eng, first2, again2, cost = run(kv_host_blocks=4, kv_storage_blocks=64, kv_storage_dir=str(tmp_path))
    assert first2 == first and again2 == first
    assert eng.stats.get("kv_demoted_blocks", 0) >= 6 and eng.stats.get("kv_promoted_blocks", 0) == 6
    assert cost == 100 - 6 * 16                           # only the uncached tail was computed
    t = eng.kv_tier.stats
    assert t["demoted_to_storage"] > 0 and t["storage_hits"] + t["host_hits"] >= 6
    eng.close()
    # the same with int8 codes in the lower tiers (one scale per layer and tensor): same bookkeeping, a quarter
    # of the fp32 bytes, and KV that is close enough for the continuation to start the same way
    q, first3, again3, cost3 = run(kv_host_blocks=64, kv_host_quant="q8")
    assert first3 == first and cost3 == 100 - 6 * 16 and q.stats.get("kv_promoted_blocks", 0) == 6
    held = next(iter(q.kv_tier.host.values()))
    assert held.k.dtype == np.int8 and held.scales.shape == (2, mc.n_layers)
    assert again3[:2] == first[:2]
    q.close()
