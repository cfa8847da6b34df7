"""Checkpoint formats and block codecs (CPU)."""
import os
import struct

import numpy as np
import pytest

from oxide_tech_llm_engine_b200.errors import UnsupportedFormat
from oxide_tech_llm_engine_b200.formats import quants
from oxide_tech_llm_engine_b200.formats.gguf import GgufFile, GgufWriter
from oxide_tech_llm_engine_b200.formats.safetensors import SafeTensorsFile, write_safetensors
from oxide_tech_llm_engine_b200.models.config import config_from_gguf, preset
from oxide_tech_llm_engine_b200.models.weights import SyntheticSource, open_weights, write_synthetic_gguf

# round-trip error bounds in the style of the reference's golden manifest (quant L_inf 5e-2 rel, cos 1e-3)
BOUNDS = {"Q8_0": (0.01, 0.9999), "Q6_K": (0.03, 0.999), "Q5_K": (0.05, 0.998), "Q5_1": (0.05, 0.998),
          "Q5_0": (0.06, 0.998), "Q4_K": (0.08, 0.995), "Q4_1": (0.08, 0.995), "Q4_0": (0.12, 0.994),
          "IQ4_NL": (0.15, 0.994), "NVFP4": (0.2, 0.99), "Q3_K": (0.25, 0.98), "Q2_K": (0.4, 0.93),
          "TQ2_0": (0.8, 0.6)}


@pytest.mark.parametrize("name", list(BOUNDS))
def test_quant_round_trip(name):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((16, 512)) * 0.05).astype(np.float32)
    raw = quants.quantize_2d(name, w)
    assert raw.shape == (16, quants.row_bytes(name, 512))
    d = quants.dequantize_2d(name, raw, 16, 512)
    err = np.abs(d - w).max() / np.abs(w).max()
    cos = float((d * w).sum() / np.linalg.norm(d) / np.linalg.norm(w))
    assert err < BOUNDS[name][0] and cos > BOUNDS[name][1], (name, err, cos)


def test_block_sizes_match_ggml():
    sizes = {"Q4_0": 18, "Q4_1": 20, "Q5_0": 22, "Q5_1": 24, "Q8_0": 34, "Q8_1": 36, "Q2_K": 84, "Q3_K": 110,
             "Q4_K": 144, "Q5_K": 176, "Q6_K": 210, "TQ2_0": 66, "PTQ1_0": 28, "IQ4_NL": 18}
    for k, v in sizes.items():
        assert quants.TYPES[k].nbytes == v


def test_known_q4_0_and_q8_0_blocks():
    # hand-packed blocks: d = 0.5, nibbles 0..15 -> (q - 8) * d for elements j and j + 16
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blk[2:18] = np.arange(16) | (np.arange(15, -1, -1) << 4)
    out = quants.dequantize("Q4_0", blk, 32)
    assert np.allclose(out[:16], (np.arange(16) - 8) * 0.5)
    assert np.allclose(out[16:], (np.arange(15, -1, -1) - 8) * 0.5)
    b8 = np.zeros(34, np.uint8)
    b8[0:2] = np.frombuffer(np.float16(0.25).tobytes(), np.uint8)
    b8[2:] = np.arange(-16, 16).astype(np.int8).view(np.uint8)
    assert np.allclose(quants.dequantize("Q8_0", b8, 32), np.arange(-16, 16) * 0.25)


def test_e4m3_codec():
    vals = np.array([0.0, 0.5, 1.0, -1.5, 448.0, 1000.0, 2 ** -9, -0.02], np.float32)
    back = quants.e4m3_to_f32(quants.f32_to_e4m3(vals))
    assert back[4] == 448.0 and back[5] == 448.0 and back[0] == 0.0
    assert np.allclose(back[[1, 2, 3]], [0.5, 1.0, -1.5])
    assert abs(back[7] + 0.02) < 0.002


def test_gguf_write_parse(tmp_path):
    p = str(tmp_path / "x.gguf")
    w = GgufWriter(p, {"general.architecture": "llama", "llama.block_count": 3, "f": 1.5, "s": "hi",
                       "arr": np.arange(5, dtype=np.int32), "strs": ["a", "bc"], "neg": -7, "big": 2 ** 40, "b": True})
    a = np.random.default_rng(1).standard_normal((4, 64)).astype(np.float32)
    w.add_tensor("t.f32", a, "F32")
    w.add_tensor("t.q8", a, "Q8_0")
    w.add_tensor("t.bf16", a, "BF16")
    w.write()
    g = GgufFile.open(p)
    assert g.version == 3 and g.metadata["llama.block_count"] == 3 and g.metadata["s"] == "hi"
    assert abs(g.metadata["f"] - 1.5) < 1e-6 and g.metadata["neg"] == -7 and g.metadata["big"] == 2 ** 40
    assert list(g.metadata["arr"]) == [0, 1, 2, 3, 4] and g.metadata["strs"] == ["a", "bc"] and g.metadata["b"] is True
    assert g.tensors["t.q8"].shape == (64, 4) and g.tensors["t.q8"].torch_shape == (4, 64)
    assert g.data_offset % 32 == 0
    assert np.array_equal(g.dequantize("t.f32"), a)
    assert np.abs(g.dequantize("t.q8") - a).max() < 0.03
    assert np.abs(g.dequantize("t.bf16") - a).max() < 0.02
    g.close()


def test_gguf_rejects_bad_input():
    with pytest.raises(UnsupportedFormat):
        GgufFile.parse(b"NOPE" + b"\0" * 32)
    with pytest.raises(UnsupportedFormat):
        GgufFile.parse(b"GGUF" + struct.pack("<I", 9) + b"\0" * 32)
    # unknown tensor type code
    buf = b"GGUF" + struct.pack("<IQQ", 3, 1, 0) + struct.pack("<Q", 1) + b"t" + struct.pack("<I", 1) + \
        struct.pack("<Q", 32) + struct.pack("<IQ", 99, 0)
    with pytest.raises(UnsupportedFormat, match="Unsupported GGUF quant type code"):
        GgufFile.parse(buf + b"\0" * 64)


def test_gguf_v1_header():
    # version 1 uses 32-bit counts and string lengths
    key = b"general.alignment"
    buf = b"GGUF" + struct.pack("<III", 1, 0, 1) + struct.pack("<I", len(key)) + key + struct.pack("<II", 4, 64)
    g = GgufFile.parse(buf + b"\0" * 128)
    assert g.version == 1 and g.metadata["general.alignment"] == 64 and g.data_offset % 64 == 0


def test_config_from_gguf_round_trip(tmp_path):
    mc = preset("tiny", rope_scaling="llama3", rope_factor=8.0, sliding_window=128, logit_softcap=30.0)
    p = str(tmp_path / "m.gguf")
    write_synthetic_gguf(p, mc, seed=1, weight_type="Q4_0")
    src = open_weights(p)
    c = src.cfg
    for f in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn_dim", "vocab_size", "rope_scaling",
              "sliding_window"):
        assert getattr(c, f) == getattr(mc, f), f
    assert c.logit_softcap == 30.0 and not c.tie_embeddings
    assert src.type_name("blk.0.attn_q.weight") == "Q4_0" and src.type_name("token_embd.weight") == "Q8_0"
    moe = preset("tiny-moe")
    p2 = str(tmp_path / "moe.gguf")
    write_synthetic_gguf(p2, moe, seed=1, weight_type="Q8_0")
    c2 = open_weights(p2).cfg
    assert c2.n_experts == 8 and c2.n_experts_used == 2 and c2.ffn_dim == moe.ffn_dim


def test_safetensors_round_trip(tmp_path):
    p = str(tmp_path / "m.safetensors")
    rng = np.random.default_rng(2)
    t = {"a": rng.standard_normal((3, 8)).astype(np.float32), "b": rng.standard_normal(5).astype(np.float32)}
    for dt, tol in (("F32", 0), ("F16", 2e-3), ("BF16", 2e-2)):
        write_safetensors(p, t, dt, {"format": "pt"})
        f = SafeTensorsFile(p)
        assert f.metadata == {"format": "pt"} and f.info("a")["shape"] == [3, 8]
        assert np.abs(f.f32("a") - t["a"]).max() <= tol + 1e-9


def test_safetensors_hf_layout_matches_gguf_names(tmp_path):
    import json

    from oxide_tech_llm_engine_b200.models.reference import ReferenceModel
    from oxide_tech_llm_engine_b200.models.weights import SafeTensorsSource

    mc = preset("tiny")
    src = SyntheticSource(mc, seed=4, std=0.08)
    inv = {"token_embd.weight": "model.embed_tokens.weight", "output.weight": "lm_head.weight",
           "output_norm.weight": "model.norm.weight"}
    lay = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
           "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
           "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}
    tensors = {}
    for n in src.names():
        if n in inv:
            tensors[inv[n]] = src.f32(n)
        else:
            _, i, rest = n.split(".", 2)
            tensors[f"model.layers.{i}.{lay[rest[:-7]]}.weight"] = src.f32(n)
    d = tmp_path / "hf"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors, "F32")
    json.dump({"num_hidden_layers": mc.n_layers, "hidden_size": mc.d_model, "num_attention_heads": mc.n_heads,
               "num_key_value_heads": mc.n_kv_heads, "head_dim": mc.head_dim, "intermediate_size": mc.ffn_dim,
               "vocab_size": mc.vocab_size, "rms_norm_eps": mc.rms_eps, "rope_theta": mc.rope_theta},
              open(d / "config.json", "w"))
    st = SafeTensorsSource(str(d))
    assert st.cfg.head_dim == mc.head_dim and st.cfg.ffn_dim == mc.ffn_dim
    prompt = [5, 9, 77, 300]
    assert ReferenceModel(st.cfg, st).generate_greedy(prompt, 6) == ReferenceModel(mc, src).generate_greedy(prompt, 6)
