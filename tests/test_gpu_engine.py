"""End-to-end engine checks on a GPU against the fp32 CPU oracle."""
import os
import tempfile

import numpy as np
import pytest
import torch

from _util import assert_consistent

pytestmark = pytest.mark.gpu


def _mk(preset_name, *, seed=3, std=0.08, weights=None, **kw):
    from oxide_tech_llm_engine_b200.config import EngineConfig
    from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource

    mc = preset(preset_name) if weights is None else weights.cfg
    src = weights or SyntheticSource(mc, seed=seed, std=std)
    base = dict(model=preset_name, max_num_seqs=8, max_num_batched_tokens=256, num_kv_blocks=256,
                ctx_size=1024, graph_buckets=(1, 2, 4, 8))
    base.update(kw)
    return LLMEngine(EngineConfig(**base), mc, weights=src), mc, src


def _oracle_tokens(mc, src, prompt, n):
    from oxide_tech_llm_engine_b200.models.reference import ReferenceModel

    return ReferenceModel(mc, src).generate_greedy(prompt, n)


def _agreement(a, b):
    n = min(len(a), len(b))
    same = 0
    for x, y in zip(a[:n], b[:n]):
        if x != y:
            break
        same += 1
    return same / max(n, 1)


@pytest.mark.parametrize("name", ["tiny", "tiny-moe"])
def test_engine_matches_oracle(name):
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    eng, mc, src = _mk(name)
    rng = np.random.default_rng(1)
    prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (4, 33, 100, 17)]
    outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=12, ignore_eos=True))
    eng.check_device_status()
    # bf16 activations against an fp32 oracle: near ties may flip, so score each token against
    # the oracle's logits given the engine's own history
    assert_consistent(mc, src, prompts, outs)
    eng.close()


def test_first_step_logits_close():
    from oxide_tech_llm_engine_b200.models.reference import ReferenceModel
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    eng, mc, src = _mk("tiny")
    prompt = np.random.default_rng(2).integers(3, mc.vocab_size, size=50).tolist()
    eng.add_request(prompt, SamplingParams(greedy=True, max_tokens=2, ignore_eos=True))
    eng.step()
    got = eng.model.logits[0].float().cpu()
    ref = ReferenceModel(mc, src).forward(prompt)[0]
    cos = torch.nn.functional.cosine_similarity(got, ref, dim=0).item()
    assert cos > 0.995, cos
    assert int(got.argmax()) == int(ref.argmax())
    eng.close()


def test_chunked_prefill_graph_and_prefix_cache_are_consistent():
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    sp = SamplingParams(greedy=True, max_tokens=10, ignore_eos=True)
    rng = np.random.default_rng(4)
    shared = rng.integers(3, 1000, size=64).tolist()
    prompts = [shared + rng.integers(3, 1000, size=n).tolist() for n in (9, 21, 40)]
    eng, mc, src = _mk("tiny")
    base = eng.generate(prompts, sp)
    # same prompts again: served from the radix cache
    again = eng.generate(prompts, sp)
    st = eng.sched.radix_stats()
    assert st["hit_tokens"] >= 3 * 64, st
    assert again == base
    eng.close()
    # small chunks, no graphs
    eng2, _, _ = _mk("tiny", chunk_max=32, chunk_min=16, max_num_batched_tokens=48, cuda_graph=False,
                     enable_radix=False)
    small = eng2.generate(prompts, sp)
    eng2.close()
    agree = [_agreement(a, b) for a, b in zip(base, small)]
    assert np.mean(agree) >= 0.9, (agree, base, small)


@pytest.mark.parametrize("qtype", ["Q8_0", "Q4_K", "Q4_0"])
def test_gguf_quantized_serving(qtype):
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import open_weights, write_synthetic_gguf
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny", d_model=256, ffn_dim=512, head_dim=64)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        write_synthetic_gguf(path, mc, seed=5, weight_type=qtype, embed_type="Q8_0", std=0.08)
        src = open_weights(path)
        eng, mc2, _ = _mk("tiny", weights=src)
        assert eng.model.weight_mode == "quant"
        rng = np.random.default_rng(6)
        prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (6, 40)]
        outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=10, ignore_eos=True))
        eng.check_device_status()
        assert_consistent(mc2, src, prompts, outs)
        eng.close()


def test_nvfp4_moe_checkpoint_is_served_through_the_fused_expert_path():
    """A Mixtral-style GGUF whose matrices are NVFP4 blocks but whose sizes do not fit the 128 x 256-value
    tiles of the fp4 tensor-core path (the tiny preset): the expert weights are expanded to bf16 at load
    and run through the router / grouped GEMM / combine. (Sizes that fit are served packed, next test.)"""
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import open_weights, write_synthetic_gguf
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny-moe")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        write_synthetic_gguf(path, mc, seed=5, weight_type="NVFP4", embed_type="Q8_0", std=0.08)
        src = open_weights(path)
        assert src.type_name("blk.0.ffn_gate_exps.weight") == "NVFP4"
        eng, mc2, _ = _mk("tiny-moe", weights=src)
        assert eng.model.weight_mode == "bf16" and mc2.is_moe
        rng = np.random.default_rng(9)
        prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (6, 40)]
        outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=10, ignore_eos=True))
        eng.check_device_status()
        assert_consistent(mc2, src, prompts, outs)
        eng.close()


def test_nvfp4_moe_checkpoint_is_served_packed_on_the_fp4_tensor_core_path():
    """A Mixtral-style GGUF with NVFP4 expert matrices whose sizes fit the fp4 tiles: the experts stay
    packed (no bf16 copy exists), both expert GEMMs run on the block-scaled fp4 path, and the tokens
    stay close to the fp32 oracle of the same (dequantised) weights; activations are quantised to
    fp4 as well, so the tolerance is wider than for bf16."""
    from oxide_tech_llm_engine_b200 import ops
    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import open_weights, write_synthetic_gguf
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    mc = preset("tiny-moe", d_model=256, ffn_dim=512, head_dim=64)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        write_synthetic_gguf(path, mc, seed=5, weight_type="NVFP4", embed_type="Q8_0", std=0.08)
        src = open_weights(path)
        eng, mc2, _ = _mk("tiny-moe", weights=src)
        assert eng.model.weight_mode == "nvfp4"
        L0 = eng.model.layers[0]
        assert isinstance(L0["w_gu"], ops.Nvfp4Weight) and L0["w_gu"].q.dtype == torch.uint8
        assert not any(isinstance(v, torch.Tensor) and v.dtype == torch.bfloat16 and v.dim() == 3 for v in L0.values())
        # the packed matrices decode to exactly what the file's blocks decode to
        want = torch.from_numpy(src.f32("blk.0.ffn_down_exps.weight")).to("cuda")
        assert torch.equal(L0["w_down"].dequant(), want)
        rng = np.random.default_rng(9)
        prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (6, 40)]
        outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=10, ignore_eos=True))
        eng.check_device_status()
        assert all(len(o) == 10 for o in outs)
        assert_consistent(mc2, src, prompts, outs, tol=1.0, min_exact=0.4)
        eng.close()


def test_fp8_block_scaled_serving():
    """Block-scaled fp8 projections: tokens stay consistent with the fp32 oracle's logits."""
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    from oxide_tech_llm_engine_b200.models.config import preset
    from oxide_tech_llm_engine_b200.models.weights import SyntheticSource

    mc = preset("tiny", d_model=256, ffn_dim=512, head_dim=64)
    src = SyntheticSource(mc, seed=7, std=0.08)
    eng, mc, src = _mk("tiny", weights=src, weight_mode="fp8")
    assert eng.model.weight_mode == "fp8" and eng.model.layers[0]["w_qkv"][0].dtype == torch.float8_e4m3fn
    rng = np.random.default_rng(8)
    prompts = [rng.integers(3, mc.vocab_size, size=n).tolist() for n in (5, 70, 150)]
    outs = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=10, ignore_eos=True))
    eng.check_device_status()
    assert_consistent(mc, src, prompts, outs, tol=0.6, min_exact=0.5)
    eng.close()


def test_sampling_and_cancel_and_speculative():
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    eng, mc, src = _mk("tiny", speculative="ngram")
    rng = np.random.default_rng(7)
    p = rng.integers(3, 1000, size=20).tolist()
    a = eng.generate([p], SamplingParams(temperature=0.9, top_k=20, top_p=0.9, seed=11, max_tokens=8,
                                         ignore_eos=True))
    b = eng.generate([p], SamplingParams(temperature=0.9, top_k=20, top_p=0.9, seed=11, max_tokens=8,
                                         ignore_eos=True))
    assert a == b and len(a[0]) == 8
    rid = eng.add_request(p, SamplingParams(greedy=True, max_tokens=50, ignore_eos=True))
    eng.step()
    assert eng.cancel(rid)
    assert not eng.has_work()
    free0 = eng.sched.num_free_blocks()
    # repetitive prompt: the n-gram drafter gets tokens accepted, results equal plain greedy
    rep = (rng.integers(3, 1000, size=8).tolist()) * 6
    spec = eng.generate([rep], SamplingParams(greedy=True, max_tokens=16, ignore_eos=True))
    eng.close()
    eng2, _, _ = _mk("tiny")
    plain = eng2.generate([rep], SamplingParams(greedy=True, max_tokens=16, ignore_eos=True))
    eng2.close()
    assert _agreement(spec[0], plain[0]) >= 0.75, (spec, plain)
    assert free0 > 0


def test_steady_state_decode_allocates_no_device_memory():
    """After warm-up, decode steps (CUDA-graph replays, staging upload, device sampler, D2H of the
    ids) run out of buffers made at construction: the caching allocator hands out nothing."""
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams
    from oxide_tech_llm_engine_b200.utils.alloc_guard import AllocGuard

    eng, mc, src = _mk("tiny")
    rng = np.random.default_rng(11)
    for n in (5, 19, 40):
        eng.add_request(rng.integers(3, mc.vocab_size, size=n).tolist(),
                        SamplingParams(greedy=True, max_tokens=64, ignore_eos=True))
    for _ in range(8):          # prefill + graph capture + a few replays
        eng.step()
    torch.cuda.synchronize()
    replays0 = eng.stats["graph_replays"]
    with AllocGuard(device=eng.device) as g:
        for _ in range(16):
            eng.step()
        torch.cuda.synchronize()
    assert eng.stats["graph_replays"] - replays0 == 16
    assert g.delta.blocks == 0 and g.delta.segments == 0, g.delta
    eng.close()


def test_h2o_pruning_on_device_scores():
    """Heavy-hitter pruning with block scores from the device (last layer's query against the
    sequence's keys): the KV of a long sequence stays within the budget, the tokens before the
    first pruning equal the unpruned run, decoding reaches the requested length, all blocks return."""
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    sp = SamplingParams(greedy=True, max_tokens=48, ignore_eos=True)
    prompt = np.random.default_rng(12).integers(3, 1000, size=90).tolist()
    base, mc, src = _mk("tiny", enable_radix=False)
    ref = base.generate([prompt], sp)[0]
    base.close()
    eng, _, _ = _mk("tiny", enable_radix=False, h2o_pruning=True, h2o_budget_blocks=6, h2o_sink_blocks=1,
                    h2o_rolling_blocks=2)
    free0 = eng.sched.num_free_blocks()
    rid = eng.add_request(prompt, sp)
    first_pruned_at = None
    while eng.has_work():
        eng.step()
        info = eng.sched.request_info(rid)
        if info is not None and info["dropped"]:
            assert len(info["blocks"]) <= 7
            if first_pruned_at is None:
                first_pruned_at = len(eng.requests[rid].output)
    eng.check_device_status()
    out = eng.requests[rid].output
    assert first_pruned_at is not None and eng.stats["h2o_pruned_blocks"] >= 1
    assert len(out) == 48 and out[:first_pruned_at] == ref[:first_pruned_at]
    assert eng.sched.num_free_blocks() == free0
    eng.close()


def test_a_device_wait_that_ran_out_degrades_the_engine_and_returns_every_block():
    """The status word that a kernel sets when a bounded wait expires is read with the sampled ids
    of the step: requests end with a typed reason, blocks go back to the pool, the hand-off
    counters are re-armed, and the engine serves again afterwards."""
    from oxide_tech_llm_engine_b200 import ops
    from oxide_tech_llm_engine_b200.errors import CollectiveTimeout
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    eng, mc, src = _mk("tiny", enable_radix=False)
    free0 = eng.sched.num_free_blocks()
    sp = SamplingParams(greedy=True, max_tokens=8, ignore_eos=True)
    want = eng.generate([[5, 6, 7, 8, 9]], sp)[0]
    rids = [eng.add_request(list(range(3, 3 + n)), sp) for n in (20, 7)]
    eng.step()
    ops.status_word(eng.device).fill_(4)      # what a kernel writes when its peer never arrived
    with pytest.raises(CollectiveTimeout):
        eng.step()
    assert all(eng.requests[r].finished and eng.requests[r].finish_reason == "collective_timeout" for r in rids)
    assert eng.sched.num_free_blocks() == free0 and not eng.has_work()
    assert eng.stats["degraded"] and eng.stats["device_faults"] == 1
    assert int(ops.status_word(eng.device).item()) == 0
    assert int(eng.model.tickets.abs().max().item()) == 0
    again = eng.generate([[5, 6, 7, 8, 9]], sp)[0]
    assert again == want
    eng.close()


def test_decode_burst_matches_step_by_step_decoding():
    """In-graph step advance + mapped-host mailbox: bursts of graph replays without a host round trip
    produce exactly the tokens of one-step-at-a-time decoding, including a request that meets a stop
    token in the middle of a burst, budgets that end inside a burst and blocks that fill up."""
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    rng = np.random.default_rng(5)
    prompts = [rng.integers(3, 200, size=n).tolist() for n in (9, 30, 47)]
    plain, mc, _ = _mk("tiny")
    want = plain.generate(prompts, SamplingParams(greedy=True, max_tokens=45, ignore_eos=True))
    # a stop token that the second request is known to emit mid-way
    stop_tok = want[1][20]
    first_hit = want[1].index(stop_tok)
    want_stop = plain.generate([prompts[1]], SamplingParams(greedy=True, max_tokens=45, stop_token_ids=[stop_tok]))[0]
    assert len(want_stop) == first_hit + 1
    plain.close()

    eng, _, _ = _mk("tiny", decode_burst=8, burst_max_batch=4, enable_radix=False)
    free0 = eng.sched.num_free_blocks()
    got = eng.generate(prompts, SamplingParams(greedy=True, max_tokens=45, ignore_eos=True))
    assert got == want
    assert eng.stats.get("burst_steps", 0) >= 30, eng.stats
    got_stop = eng.generate([prompts[1]], SamplingParams(greedy=True, max_tokens=45, stop_token_ids=[stop_tok]))[0]
    assert got_stop == want_stop
    # every block is back in the pool afterwards (reservations of ended requests included)
    assert eng.sched.num_running() == 0
    eng.check_device_status()
    assert eng.sched.num_free_blocks() == free0
    single = eng.generate([prompts[0]], SamplingParams(greedy=True, max_tokens=7, ignore_eos=True))[0]
    assert single == want[0][:7] and eng.sched.num_free_blocks() == free0
    eng.close()
