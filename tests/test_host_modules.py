"""CSKV files, KV tiers, quantised KV blocks, context shift, beam search, LoRA, slots, catalog,
hardware profiles, tracing (CPU)."""
import json
import os

import numpy as np
import pytest

from oxide_tech_llm_engine_b200.config import EngineConfig
from oxide_tech_llm_engine_b200.engine import cskv, decoding, kv_tiers, lora, slots
from oxide_tech_llm_engine_b200.engine.engine import LLMEngine
from oxide_tech_llm_engine_b200.errors import EngineError, OutOfMemory, SlotsExhausted, UnsupportedFormat
from oxide_tech_llm_engine_b200.models import catalog
from oxide_tech_llm_engine_b200.models.config import preset
from oxide_tech_llm_engine_b200.models.reference import ReferenceModel
from oxide_tech_llm_engine_b200.models.weights import SyntheticSource
from oxide_tech_llm_engine_b200.sampling_params import SamplingParams
from oxide_tech_llm_engine_b200.utils import hardware, tracing


def test_cskv_headers_all_versions():
    h = cskv.CskvHeader(cskv.V_DENSE_F16, 4, 100, 2, 64)
    b = h.to_bytes()
    assert b[:4] == b"CSKV" and len(b) == 25
    h2, off = cskv.CskvHeader.parse(b + b"\0" * 8)
    assert off == 25 and (h2.num_layers, h2.seq_len, h2.num_kv_heads, h2.head_dim) == (4, 100, 2, 64)
    assert h2.dtype == np.float16 and len(cskv.CskvHeader(1, 2, 5, 1, 8).to_bytes()) == 24
    lay = h.layout()
    assert len(lay) == 8 and lay[1]["offset"] - lay[0]["offset"] == 100 * 2 * 64 * 2
    hy = cskv.CskvHeader(cskv.V_HYBRID, 3, 10, 2, 64, gdn_conv_state_len=7, gdn_recurrent_len=9, layer_kinds=[0, 1, 0])
    hy2, _ = cskv.CskvHeader.parse(hy.to_bytes())
    assert hy2.kind == "hybrid" and hy2.layer_kinds == [0, 1, 0] and hy2.gdn_recurrent_len == 9
    ml, _ = cskv.CskvHeader.parse(cskv.CskvHeader(cskv.V_MLA_F16, 2, 4, qk_dim=192).to_bytes())
    assert ml.kind == "mla" and ml.qk_dim == 192
    with pytest.raises(UnsupportedFormat):
        cskv.CskvHeader.parse(b"CSKV" + (99).to_bytes(4, "little") + b"\0" * 16)
    with pytest.raises(UnsupportedFormat):
        cskv.CskvHeader.parse(b"XXXX" + b"\0" * 20)


def test_cskv_save_and_resume_through_the_prefix_cache(tmp_path):
    mc = preset("tiny")
    src = SyntheticSource(mc, seed=3, std=0.08)
    cfg = EngineConfig(backend="cpu", max_num_seqs=2, max_num_batched_tokens=64, num_kv_blocks=64, ctx_size=512)
    eng = LLMEngine(cfg, mc, weights=src)
    prompt = list(range(10, 60))
    rid = eng.add_request(prompt, SamplingParams(greedy=True, max_tokens=30, ignore_eos=True))
    for _ in range(6):
        eng.step()
    path = str(tmp_path / "state.cskv")
    h = cskv.save_sequence(eng, rid, path)
    assert h.version == cskv.V_DENSE_F16 and h.num_layers == mc.n_layers and os.path.exists(path + ".manifest.json")
    man = json.load(open(path + ".manifest.json"))
    assert man["tokens"] == h.seq_len and man["token_ids"][:50] == prompt
    # a fresh engine restores the state and serves the same prompt from the cache
    eng2 = LLMEngine(cfg, mc, weights=src)
    n = cskv.load_prefix(eng2, path)
    assert n == h.seq_len // 16 * 16 and n >= 48
    out = eng2.generate([prompt], SamplingParams(greedy=True, max_tokens=8, ignore_eos=True))[0]
    assert eng2.sched.radix_stats()["hit_tokens"] >= 48
    assert out == ReferenceModel(mc, src).generate_greedy(prompt, 8)   # f16 KV round trip keeps the argmax


def test_hierarchical_tiers_and_payload(tmp_path):
    toks = np.arange(64, dtype=np.int32)
    hs = kv_tiers.prefix_hashes(toks)
    assert len(hs) == 4 and len(set(hs)) == 4
    other = toks.copy()
    other[20] = 7
    ho = kv_tiers.prefix_hashes(other)
    assert ho[0] == hs[0] and ho[1] != hs[1] and ho[2] != hs[2]     # chained: a change poisons the suffix
    rng = np.random.default_rng(0)
    def mk(i):
        return kv_tiers.KvBlockPayload(hs[i], toks[i * 16:(i + 1) * 16].copy(),
                                       rng.standard_normal((2, 2, 16, 8)).astype(np.float16),
                                       rng.standard_normal((2, 2, 16, 8)).astype(np.float16))
    c = kv_tiers.HierarchicalKvCache(host_blocks=2, storage_blocks=1, storage_dir=str(tmp_path))
    ps = [mk(i) for i in range(4)]
    for p in ps:
        c.demote(p)
    assert len(c.host) == 2 and len(c.storage) == 1 and c.stats["dropped"] == 1
    assert c.lookup(hs[3]) is not None and c.stats["host_hits"] == 1
    got = c.lookup(hs[1])                                            # from the file tier, promoted
    assert got is not None and np.array_equal(got.k, ps[1].k) and c.stats["storage_hits"] == 1
    assert c.lookup(hs[0]) is None and c.stats["misses"] == 1
    blob = ps[2].seal().to_bytes()
    bad = bytearray(blob)
    bad[-1] ^= 0xFF
    with pytest.raises(EngineError):
        kv_tiers.KvBlockPayload.from_bytes(bytes(bad))
    assert kv_tiers.KvBlockPayload.from_bytes(blob).verify()
    # a file of the storage tier that vanished or was damaged is a miss, not an error
    c2 = kv_tiers.HierarchicalKvCache(host_blocks=1, storage_blocks=4, storage_dir=str(tmp_path / "t3"))
    for p in (mk(0), mk(1), mk(2)):
        c2.demote(p)
    paths = list(c2.storage.values())
    assert len(paths) == 2
    os.unlink(paths[0])
    with open(paths[1], "r+b") as f:
        f.seek(-1, 2)
        f.write(b"\x00" if open(paths[1], "rb").read()[-1:] != b"\x00" else b"\x01")
    assert c2.lookup(hs[0]) is None and c2.lookup(hs[1]) is None
    assert c2.stats["storage_errors"] == 2 and c2.stats["storage_hits"] == 0
    # int8 payloads with per-layer scales survive the file round trip
    q = kv_tiers.KvBlockPayload(hs[3], toks[48:64].copy(), rng.integers(-127, 127, (2, 2, 16, 8)).astype(np.int8),
                                rng.integers(-127, 127, (2, 2, 16, 8)).astype(np.int8), 0,
                                np.asarray([[0.5, 0.25], [1.5, 2.0]], np.float32)).seal()
    back = kv_tiers.KvBlockPayload.from_bytes(q.to_bytes())
    assert back.k.dtype == np.int8 and np.array_equal(back.k, q.k) and np.array_equal(back.scales, q.scales)


def test_quantized_kv_blocks_context_shift_registry(tmp_path):
    x = np.random.default_rng(1).standard_normal((4, 16, 8)).astype(np.float32)
    for mode, tol in (("f32", 0), ("f16", 2e-3), ("q8", 0.02), ("q4", 0.3)):
        q = kv_tiers.QuantizedKvBlock.quantize(x, mode)
        assert np.abs(q.dequantize() - x).max() <= tol * np.abs(x).max() + 1e-9
    assert kv_tiers.QuantizedKvBlock.quantize(x, "q4").nbytes() == x.size // 2
    cs = kv_tiers.ContextShiftManager(max_ctx=100, keep_prefix=4, shift_step=10)
    assert cs.plan(50) is None and cs.plan(100) == (4, 10) and cs.plan(130, 1) == (4, 31)
    assert cs.apply(list(range(100))) == list(range(4)) + list(range(14, 100))
    reg = kv_tiers.PromptCacheRegistry()
    reg.register([1, 2, 3], "a")
    reg.register([1, 2, 3, 4, 5], "b")
    assert reg.lookup([1, 2, 3]) == ("a", 3) and reg.lookup([1, 2, 3, 4, 5, 6]) == ("b", 5) and reg.lookup([9])[0] is None
    d = kv_tiers.KvCacheDumpContainer()
    d.add(0, "key", kv_tiers.QuantizedKvBlock.quantize(x, "q8"))
    p = str(tmp_path / "dump.json")
    d.dump(p)
    (layer, kind, q), = kv_tiers.KvCacheDumpContainer.load(p)
    assert layer == 0 and kind == "key" and np.abs(q.dequantize() - x).max() < 0.03 * np.abs(x).max()


def test_beam_search_and_best_of_n():
    assert abs(decoding.length_penalty(1) - 1.0) < 1e-9
    lp = np.log(np.array([[0.6, 0.3, 0.1], [0.1, 0.2, 0.7]]))
    beams = decoding.beam_step([decoding.Beam([5], -0.1), decoding.Beam([6], -0.2)], lp, beam_width=2, eos_id=2)
    assert [b.tokens for b in beams] == [[6, 2], [5, 0]] and beams[0].finished
    nxt = decoding.beam_step(beams, lp[:1], beam_width=2, eos_id=2)
    assert any(b.finished and b.tokens == [6, 2] for b in nxt)
    order = decoding.rank_candidates([([1, 2, 3, 4], -4.0), ([1], -2.0), ([1, 2], -1.0)])
    assert order[0] == 2


def test_lora_merge_equals_activation_path():
    mc = preset("tiny")
    src = SyntheticSource(mc, seed=2, std=0.05)
    rng = np.random.default_rng(3)
    name = "blk.0.attn_q.weight"
    ad = lora.LoraAdapter("a", rank=4, alpha=8.0, a={name: rng.standard_normal((4, mc.d_model)).astype(np.float32)},
                          b={name: rng.standard_normal((mc.q_dim, 4)).astype(np.float32)})
    merged = lora.MergedSource(src, ad)
    x = rng.standard_normal((3, mc.d_model)).astype(np.float32)
    want = x @ src.f32(name).T + ad.apply_activation(name, x)
    assert np.allclose(x @ merged.f32(name).T, want, atol=1e-4)
    assert merged.f32("blk.1.attn_q.weight") is not None and merged.type_name(name) == "F32"
    reg = lora.LoraRegistry()
    reg.register(ad)
    assert reg.names() == ["a"] and reg.get("a").scale == 2.0
    # a merged source changes what the model generates
    p = [5, 6, 7, 8]
    assert ReferenceModel(mc, lora.MergedSource(src, lora.LoraAdapter(
        "big", 4, 400.0, ad.a, ad.b))).generate_greedy(p, 4) != ReferenceModel(mc, src).generate_greedy(p, 4)


def test_lora_safetensors_ingest(tmp_path):
    from oxide_tech_llm_engine_b200.formats.safetensors import write_safetensors

    rng = np.random.default_rng(4)
    t = {"base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight": rng.standard_normal((2, 16)).astype(np.float32),
         "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight": rng.standard_normal((8, 2)).astype(np.float32)}
    p = str(tmp_path / "adapter.safetensors")
    write_safetensors(p, t, "F32", {"lora_alpha": "4"})
    ad = lora.load_adapter_safetensors(p, "x")
    assert ad.rank == 2 and ad.alpha == 4.0 and ad.delta("blk.0.attn_q.weight").shape == (8, 16)


def test_slots_lifecycle_arenas():
    m = slots.SlotManager(2, chunk_size=8)
    a = m.lease(1, 20)
    with m.leased(2, 3) as b:
        assert m.total_active_slots() == 2
        with pytest.raises(SlotsExhausted):
            m.lease(3, 1)
        assert m.next_chunk(b) == 3 and b.state == slots.SlotState.DECODE
    assert m.total_active_slots() == 1
    assert [m.next_chunk(a) for _ in range(3)] == [8, 8, 4] and a.state == slots.SlotState.DECODE
    m.on_token(a, True)
    assert a.state == slots.SlotState.FINISHED
    lc = slots.RequestLifecycle()
    lc.to(slots.RequestPhase.ALLOCATED).to(slots.RequestPhase.PREFILLING).to(slots.RequestPhase.DECODING).to(slots.RequestPhase.TERMINAL)
    with pytest.raises(EngineError):
        lc.to(slots.RequestPhase.DECODING)
    ar = slots.DeviceMemoryArena.calibrate(1000, 100, 200, utilisation=0.9)
    assert ar.n_slots == 4 and ar.bind(7) == 0 and ar.bind(8) == 200
    ar.unbind(7)
    assert ar.bind(9) == 0
    hp = slots.HostPinnedArena(1024, pin=False)
    x = hp.alloc(100)
    y = hp.alloc(100)
    assert x.numel() == 100 and y.data_ptr() - x.data_ptr() == 128
    with pytest.raises(OutOfMemory):
        hp.alloc(4096)


def test_catalog_profiles_tracing(monkeypatch, tmp_path):
    assert catalog.lookup("Meta-Llama-3-8B-Instruct-Q4_K_M.gguf").key == "llama3-8b"
    assert catalog.lookup("/x/DeepSeek-R1-0528-Qwen3-8B-Q4_K_M.gguf").key == "deepseek-r1-qwen3-8b"
    assert catalog.lookup("mixtral-8x7b").config.n_experts == 8 and catalog.lookup("nope-model") is None
    assert len(catalog.catalog()) >= 12
    assert hardware.architecture(10, 0) == "blackwell" and hardware.architecture(9, 0) == "hopper"
    p = hardware.lookup_profile("NVIDIA B200")
    assert p.sm_count == 148 and p.tensor_core_gen == 5 and p.nvlink_gbs_per_dir == 900.0
    sd = hardware.SharedDevice(1000)
    sd.reserve(600, "weights")
    with pytest.raises(OutOfMemory):
        sd.reserve(500, "kv")
    sd.release(600)
    assert sd.free_bytes() == 1000

    class FakeNvml:  # energy sampler against a fake NVML: reads only
        e = 0
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetTotalEnergyConsumption(self, h):
            FakeNvml.e += 5000
            return FakeNvml.e
    es = hardware.EnergySampler(0, nvml=FakeNvml())
    es.start()
    r = es.stop(tokens=100)
    assert abs(r["joules"] - 5.0) < 1e-9 and abs(r["tokens_per_joule"] - 20.0) < 1e-9
    monkeypatch.setenv("OXB_DEBUG_LAYER", "1")
    import torch
    assert tracing.debug_tensor("x", torch.arange(10.0)) == [0.0, 1.0, 2.0, 3.0]
    tr = tracing.StepTrace(str(tmp_path / "t.jsonl"))
    tr.record(1, 4, 0, 1.5)
    tr.close()
    assert json.loads(open(tmp_path / "t.jsonl").read())["decode"] == 4
