"""Tokenizer, chat templates, CLI parsing, mesh / split planning, RoPE tables, roofline, CSKV (CPU)."""
import numpy as np
import pytest

from oxide_tech_llm_engine_b200 import chat_template as ct
from oxide_tech_llm_engine_b200.cli import engine_config_from_args, normalize_argv, parse_args
from oxide_tech_llm_engine_b200.errors import BenchmarkIntegrityViolation, ConfigError
from oxide_tech_llm_engine_b200.models.config import preset
from oxide_tech_llm_engine_b200.models.rope import inv_freq_table
from oxide_tech_llm_engine_b200.parallel import mesh
from oxide_tech_llm_engine_b200.tokenizer import Tokenizer
from oxide_tech_llm_engine_b200.utils.roofline import RooflineReceipt


def test_tokenizer_greedy_longest_match_and_specials():
    vocab = ["<unk>", "<s>", "</s>", "▁hello", "▁he", "llo", "▁world", "▁", "h", "<|im_end|>", "<0x21>", "w"]
    t = Tokenizer(vocab, bos_id=1, eos_id=2)
    ids = t.encode("hello world!<|im_end|>")
    assert ids == [1, 3, 6, 10, 9]
    assert t.decode(ids) == "hello world!"
    assert t.is_stop_token(2) and t.is_stop_token(9) and not t.is_stop_token(3)
    assert set(t.stop_ids()) == {2, 9}


def test_ascii_fallback_round_trip():
    t = Tokenizer.ascii_fallback(1024)
    s = "Héllo, wörld! 123"
    assert t.decode(t.encode(s)) == s
    assert t.vocab_size == 1024 and len(t.vocab_bytes()) == 1024


def test_chat_templates():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "U"}]
    assert ct.render_chat(msgs, ct.ChatFormat.CHATML) == \
        "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nU<|im_end|>\n<|im_start|>assistant\n"
    assert ct.render_chat(msgs, ct.ChatFormat.LLAMA3).startswith("<|begin_of_text|><|start_header_id|>system")
    assert "[INST] S\n\nU [/INST]" in ct.render_chat(msgs, ct.ChatFormat.MISTRAL)
    assert ct.render_chat(msgs, ct.ChatFormat.GEMMA).endswith("<start_of_turn>model\n")
    assert "### Response:" in ct.render_chat(msgs, ct.ChatFormat.ALPACA)
    assert ct.render_chat(msgs, ct.ChatFormat.RAW) == "S\nU"
    assert ct.detect("llama", "Meta-Llama-3-8B") == ct.ChatFormat.LLAMA3
    assert ct.detect("qwen2", "") == ct.ChatFormat.CHATML and ct.detect("gemma2", "") == ct.ChatFormat.GEMMA
    assert ct.detect("", "DeepSeek-R1") == ct.ChatFormat.DEEPSEEK and ct.parse_format("mistral") == ct.ChatFormat.MISTRAL
    assert "<|eot_id|>" in ct.stop_strings(ct.ChatFormat.LLAMA3)


def test_cli_flags_and_normalisation():
    assert normalize_argv(["-ngl", "33", "-md", "d.gguf", "--cb"]) == ["--n-gpu-layers", "33", "--draft-model", "d.gguf",
                                                                       "--continuous-batching"]
    a = parse_args(["-m", "x.gguf", "-ngl", "20", "-c", "4096", "--temp", "0.2", "--top-k", "10", "--greedy",
                    "--max-slots", "8", "-b", "cpu", "-p", "hi", "-n", "5", "--speculative", "ngram"])
    assert a.model == "x.gguf" and a.n_gpu_layers == 20 and a.ctx_size == 4096 and a.greedy and a.max_tokens == 5
    cfg = engine_config_from_args(a)
    assert cfg.backend == "cpu" and cfg.max_num_seqs == 8 and cfg.speculative == "ngram" and cfg.ctx_size == 4096
    # the KV tier flags reach the engine (defaults of the reference: 8192 host blocks, 32768 storage blocks)
    assert cfg.kv_host_blocks == 8192 and cfg.kv_storage_blocks == 32768 and cfg.kv_storage_dir is None
    t = engine_config_from_args(parse_args(["-m", "x.gguf", "-b", "cpu", "--kv-host-blocks", "16", "--kv-storage-dir", "/tmp/kv",
                                            "--kv-host-quant", "q8", "--decode-burst", "4"]))
    assert (t.kv_host_blocks, t.kv_storage_dir, t.kv_host_quant, t.decode_burst) == (16, "/tmp/kv", "q8", 4)
    s = parse_args(["server", "--port", "9000", "-m", "tiny", "-b", "cpu"])
    assert s.command == "server" and s.port == 9000
    d = parse_args([])
    assert d.temp == 0.7 and d.top_p == 0.95 and d.min_p == 0.05 and d.repeat_penalty == 1.1 and d.top_k == 40 \
        and d.seed == 42 and d.max_tokens == 512 and d.max_slots == 64 and d.draft_tokens == 5
    with pytest.raises(ConfigError):
        parse_args(["-b", "rocm"])
    with pytest.raises(ConfigError):
        parse_args(["-b", "nonsense"])


def test_mesh_coordinates_and_splits():
    m = mesh.ParallelMeshConfig(tp=2, cp=2, ep=1, dp=2, pp=2)
    assert m.world_size == 16
    seen = set()
    for r in range(16):
        c = mesh.MeshCoordinate.from_global_rank(r, m)
        assert c.to_global_rank(m) == r
        seen.add((c.tp, c.cp, c.ep, c.dp, c.pp))
    assert len(seen) == 16
    assert mesh.MeshCoordinate.from_global_rank(1, m).tp == 1 and mesh.MeshCoordinate.from_global_rank(2, m).cp == 1
    assert mesh.split_sizes(80, 3) == [27, 27, 26] and sum(mesh.split_sizes(28672, 8, multiple=32)) == 28672
    assert mesh.layer_partition_for_rank(80, 3, 2) == (54, 80)
    assert mesh.split_sizes(100, 2, weights=[3, 1]) == [75, 25]
    st = mesh.RingAttentionStep.plan(32768, 8, 0)
    assert st.chunk_seq_len == 4096 and st.send_peer == 7 and st.recv_peer == 1


def test_rope_tables():
    base, ms = inv_freq_table(preset("tiny"))
    assert ms == 1.0 and base[0] == 1.0 and np.all(np.diff(base) < 0)
    lin, _ = inv_freq_table(preset("tiny", rope_scaling="linear", rope_factor=4.0))
    assert np.allclose(lin, base / 4)
    l3, _ = inv_freq_table(preset("tiny", rope_scaling="llama3", rope_factor=8.0, rope_orig_ctx=8192))
    assert np.isclose(l3[0], base[0]) and np.all(l3 <= base + 1e-12) and l3[-1] < base[-1]
    yarn, yms = inv_freq_table(preset("tiny", rope_scaling="yarn", rope_factor=4.0, rope_orig_ctx=2048))
    assert yms > 1.0 and np.isclose(yarn[0], base[0]) and yarn[-1] < base[-1]


def test_roofline_receipt_rejects_impossible_numbers():
    mc = preset("llama3-8b")
    peaks = {"hbm_gbs": 6531.3, "bf16_tflops": 1627.6, "bf16_tflops_sustained": 1387.6}
    r = RooflineReceipt.from_run(mc, tokens_per_s=200.0, batch=1, peaks=peaks)
    assert 0.4 < r.mbu < 0.6 and r.mfu < 0.01
    with pytest.raises(BenchmarkIntegrityViolation):
        RooflineReceipt.from_run(mc, tokens_per_s=1138.45 * 4, batch=1, peaks=peaks)


def test_energy_sampler_against_fake_nvml():
    from oxide_tech_llm_engine_b200.utils.energy import EnergySampler

    class FakeNvml:
        def __init__(self, counter=True):
            self.counter, self.mj, self.mw = counter, 5_000_000, 700_000
        def nvmlInit(self): pass
        def nvmlDeviceGetHandleByIndex(self, i): return i
        def nvmlDeviceGetTotalEnergyConsumption(self, h):
            if not self.counter:
                raise RuntimeError("not supported")
            return self.mj
        def nvmlDeviceGetPowerUsage(self, h): return self.mw
    now = [10.0]
    nv = FakeNvml(counter=True)
    s = EnergySampler(0, nvml=nv, clock=lambda: now[0]).start()
    nv.mj += 1_400_000
    now[0] += 2.0
    r = s.stop(tokens=2800)
    assert r.source == "counter" and abs(r.joules - 1400.0) < 1e-6 and abs(r.watts - 700.0) < 1e-6
    assert abs(r.tokens_per_joule - 2.0) < 1e-9 and r.to_dict()["tokens"] == 2800
    nv2 = FakeNvml(counter=False)
    s2 = EnergySampler(0, nvml=nv2, clock=lambda: now[0], period_s=3600)
    assert s2.source == "integrated"
    s2.start()
    s2.sample_once(0.5)
    nv2.mw = 900_000
    s2.sample_once(0.5)
    now[0] += 1.0
    r2 = s2.stop(tokens=10)
    assert abs(r2.joules - 800.0) < 1e-6 and abs(r2.watts - 800.0) < 1e-6

    class Broken:
        def nvmlInit(self): raise RuntimeError("no driver")
    r3 = EnergySampler(0, nvml=Broken()).start().stop(5)
    assert r3.source == "unavailable" and r3.joules == 0 and r3.tokens_per_joule == 0


def test_alloc_guard_with_fake_counters():
    import pytest as _pt

    from oxide_tech_llm_engine_b200.utils.alloc_guard import AllocGuard

    class Src:
        def __init__(self): self.s = {"allocation.all.allocated": 10, "segment.all.allocated": 2,
                                      "allocated_bytes.all.peak": 100}
        def memory_stats(self): return dict(self.s)
    src = Src()
    with AllocGuard(stats_source=src) as g:
        pass
    assert g.delta.blocks == 0 and g.delta.segments == 0
    with _pt.raises(AssertionError):
        with AllocGuard(stats_source=src):
            src.s["allocation.all.allocated"] += 3
    with AllocGuard(stats_source=src, max_blocks=5) as g2:
        src.s["allocation.all.allocated"] += 3
    assert g2.delta.blocks == 3


def test_facade_builder_transaction_and_ascii_mask():
    import numpy as np
    import pytest as _pt

    import oxide_tech_llm_engine_b200 as oxb
    from oxide_tech_llm_engine_b200._build import host_ext
    from oxide_tech_llm_engine_b200.engine.transactional import KvTransaction
    from oxide_tech_llm_engine_b200.errors import OutOfMemory, TransactionAborted
    from oxide_tech_llm_engine_b200.grammar import ascii_first_byte_mask
    from oxide_tech_llm_engine_b200.sampling_params import SamplingParams

    eng = (oxb.Engine.builder().model("tiny").backend("cpu").context_size(256).max_slots(2)
           .option(num_kv_blocks=32).build())
    out = eng.generate([[5, 6, 7, 8]], SamplingParams(greedy=True, max_tokens=4, ignore_eos=True))
    assert len(out[0]) == 4
    eng.close()
    with _pt.raises(ValueError):
        oxb.Engine.builder().backend("rocm")
    cfg = (oxb.Engine.builder().model("tiny").kv_tiers(64, "/tmp/kv", 128, quant="q8").decode_burst(8, 4)
           .speculative("ngram", 4).config())
    assert (cfg.kv_host_blocks, cfg.kv_storage_dir, cfg.kv_storage_blocks, cfg.kv_host_quant) == (64, "/tmp/kv", 128, "q8")
    assert (cfg.decode_burst, cfg.burst_max_batch, cfg.speculative, cfg.draft_tokens) == (8, 4, "ngram", 4)

    H = host_ext()
    pool = H.BlockPool(4)
    t = H.SequenceBlockTable(pool)
    with KvTransaction(t, 20) as tx:
        tx.commit()
    assert t.num_tokens() == 20 and pool.num_free() == 2
    with _pt.raises(RuntimeError):
        with KvTransaction(t, 20):
            assert pool.num_free() == 1
            raise RuntimeError("step failed")
    assert t.num_tokens() == 20 and pool.num_free() == 2      # rolled back
    with _pt.raises(OutOfMemory):
        with KvTransaction(t, 200):
            pass
    with _pt.raises(TransactionAborted):
        with KvTransaction(t, 5) as tx:
            tx.abort("verify rejected")
    assert t.num_tokens() == 20

    m = ascii_first_byte_mask(b'{["', [b"{a", b"x", b"", b"[1", b'"k'])
    assert m.tolist() == [True, False, False, True, True]


def test_fuse_quant_rows_stacks_packed_matrices():
    import numpy as np
    import torch

    from oxide_tech_llm_engine_b200.formats import quants
    from oxide_tech_llm_engine_b200.models.llama import QuantLinear, fuse_quant_rows

    rng = np.random.default_rng(3)
    K = 256
    mats = [(rng.standard_normal((n, K)) * 0.05).astype(np.float32) for n in (8, 4, 4)]
    lins = [QuantLinear("Q4_K", quants.quantize_2d("Q4_K", m), m.shape[0], K, torch.device("cpu")) for m in mats]
    fused = fuse_quant_rows(lins)
    assert fused is not None and fused.n == 16 and fused.k == K and fused.type_name == "Q4_K"
    raw = fused.w.numpy().reshape(16, -1)
    got = quants.dequantize_2d("Q4_K", raw, 16, K)
    want = np.concatenate([quants.dequantize_2d("Q4_K", quants.quantize_2d("Q4_K", m), m.shape[0], K) for m in mats])
    np.testing.assert_array_equal(got, want)
    other = QuantLinear("Q8_0", quants.quantize_2d("Q8_0", mats[0]), 8, K, torch.device("cpu"))
    assert fuse_quant_rows([lins[0], other]) is None          # different block types are not stacked


def test_decode_gemm_configs_respect_the_kernel_limits():
    """`ops.pick_decode_cfg` for the shapes of the serving configurations (70B at TP 1..8, 8B, Mixtral
    attention): one wave of work items, no more splits than the in-kernel fix-up can land, tiles that
    divide N where the SwiGLU epilogue needs it. A violation would only show as a launch error on a GPU."""
    from oxide_tech_llm_engine_b200 import ops

    sms = 148
    shapes = []
    for tp in (1, 2, 4, 8):
        shapes += [(256, 2 * 28672 // tp, 8192, True), (256, 8192, 28672 // tp, False),
                   (256, (64 + 16) * 128 // tp, 8192, False), (256, 8192, 8192 // tp, False)]
    shapes += [(192, 2 * 14336, 4096, True), (136, 4096, 14336, False), (256, 6144, 4096, False), (129, 128256, 4096, False)]
    for m, n, k, swiglu in shapes:
        bn, mt, sp = ops.pick_decode_cfg(m, n, k, swiglu=swiglu, sms=sms)
        assert bn in (64, 128, 256) and mt == 2 and sp >= 1, (m, n, k, bn, mt, sp)
        tiles = -(-n // bn)
        kb = -(-k // 64)
        if sp > 1:
            assert tiles * sp <= sms, (m, n, k, bn, sp)
            assert sp <= ops.max_fixup_splits(bn, mt, swiglu), (m, n, k, bn, sp)
            assert -(-kb // -(-kb // sp)) == sp            # the launcher's rounding keeps this split count
        if swiglu:
            assert n % bn == 0
    assert ops.pick_decode_cfg(100, 4096, 4096)[1] == 1    # up to 128 rows: one 128-row tile per weight tile
