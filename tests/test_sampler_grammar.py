"""Host sampler pipeline and DFA grammars (CPU)."""
import numpy as np
import pytest

from oxide_tech_llm_engine_b200.grammar import REJECT, GrammarState, json_object_dfa, json_prefix_dfa
from oxide_tech_llm_engine_b200.sampler import HostSampler, XorShift64, first_char_mask
from oxide_tech_llm_engine_b200.sampling_params import SamplingParams


def logits(n=100, seed=0):
    return np.random.default_rng(seed).standard_normal(n).astype(np.float32) * 3


def test_top_k_one_and_greedy_pick_argmax():
    l = logits()
    assert HostSampler(SamplingParams(top_k=1)).sample(l, []) == int(l.argmax())
    assert HostSampler(SamplingParams(temperature=0.0)).sample(l, []) == int(l.argmax())


def test_seed_determinism_and_distribution():
    l = np.array([2.0, 1.0, 0.0, -9.0], np.float32)
    p = SamplingParams(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, seed=5)
    a = [HostSampler(p).sample(l, []) for _ in range(3)]
    assert len(set(a)) == 1
    s = HostSampler(p)
    draws = np.array([s.sample(l, []) for _ in range(4000)])
    want = np.exp(l) / np.exp(l).sum()
    freq = np.array([(draws == i).mean() for i in range(4)])
    assert np.abs(freq - want).max() < 0.03


def test_min_p_and_top_p_and_xtc():
    l = np.log(np.array([0.5, 0.3, 0.15, 0.05], np.float32))
    s = HostSampler(SamplingParams(temperature=1.0, top_k=0, top_p=1.0, min_p=0.5, seed=1))
    assert set(s.sample(l, []) for _ in range(200)) <= {0, 1}
    s = HostSampler(SamplingParams(temperature=1.0, top_k=0, top_p=0.6, min_p=0.0, seed=1))
    assert set(s.sample(l, []) for _ in range(200)) <= {0, 1}
    s = HostSampler(SamplingParams(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, xtc_probability=1.0,
                                   xtc_threshold=0.1, seed=1))
    assert 0 not in set(s.sample(l, []) for _ in range(200))


def test_penalties_bias_bans():
    l = np.zeros(10, np.float32)
    l[3] = 5.0
    l[4] = 4.0
    assert HostSampler(SamplingParams(top_k=1, repeat_penalty=2.0)).sample(l, [3]) == 4
    assert HostSampler(SamplingParams(top_k=1, presence_penalty=2.0)).sample(l, [3]) == 4
    assert HostSampler(SamplingParams(top_k=1, frequency_penalty=0.6)).sample(l, [3, 3]) == 4
    assert HostSampler(SamplingParams(top_k=1, banned_tokens=[3])).sample(l, []) == 4
    assert HostSampler(SamplingParams(top_k=1, logit_bias={7: 10.0})).sample(l, []) == 7
    assert HostSampler(SamplingParams(top_k=1, newline_penalty=3.0), newline_token_id=3).sample(l, []) == 4
    # penalties only look at the last repeat_last_n tokens
    assert HostSampler(SamplingParams(top_k=1, repeat_penalty=2.0, repeat_last_n=2)).sample(l, [3, 8, 9]) == 3


def test_dry_penalises_repeated_continuation():
    l = np.zeros(20, np.float32)
    l[5] = 1.0
    hist = [1, 2, 3, 5, 9, 1, 2, 3]  # "1 2 3" was followed by 5 before
    assert HostSampler(SamplingParams(top_k=1, dry_multiplier=0.0)).sample(l, hist) == 5
    assert HostSampler(SamplingParams(top_k=1, dry_multiplier=2.0, dry_allowed_length=2)).sample(l, hist) != 5


def test_mirostat_tfs_typical_run():
    l = logits(500, 3)
    for p in (SamplingParams(mirostat=1), SamplingParams(mirostat=2)):
        s = HostSampler(p)
        mu0 = s.mu
        assert s.sample(l, []) == int(l.argmax()) and s.mu != mu0
    for p in (SamplingParams(tfs_z=0.5, seed=2), SamplingParams(typical_p=0.5, seed=2)):
        t = HostSampler(p).sample(l, [])
        assert 0 <= t < 500


def test_xorshift_and_first_char_mask():
    r = XorShift64(42)
    v = [r.next_f32() for _ in range(1000)]
    assert 0.0 <= min(v) and max(v) < 1.0 and 0.4 < np.mean(v) < 0.6
    m = first_char_mask([b"{x", b"a", b"", b"{"], {ord("{")})
    assert m[0] & 0b1111 == 0b1001
    l = np.array([0.0, 9.0, 0.0, 1.0], np.float32)
    assert HostSampler(SamplingParams(top_k=1)).sample(l, [], allow_mask=m) == 3


def test_json_dfa_accepts_and_rejects():
    d = json_object_dfa()
    ok = [b'{}', b' { "a" : 1 }', b'{"k":"v","n":-3.5,"t":true,"f":false,"z":null}', b'{"e":"q\\"x"}']
    bad = [b'[1]', b'{a:1}', b'{"a":}', b'{"a":1,}', b'{"a":tru}']
    for s in ok:
        assert d.is_accepting(d.walk(d.start, s)), s
    for s in bad:
        assert not d.is_accepting(d.walk(d.start, s)) if d.walk(d.start, s) != REJECT else True


def test_jump_forward_and_token_mask():
    d = json_prefix_dfa(b'{"name": "')
    forced, state = d.find_jump_forward_bytes(d.start)
    assert forced == b'{"name": "'
    vocab = [b'{"', b'name', b'": "', b'x', b'"}', b'[', b'']
    g = GrammarState(d, vocab)
    m = g.allow_mask(len(vocab))
    assert m[0] & 1 and not (m[0] >> 5) & 1 and not (m[0] >> 3) & 1
    for t in (0, 1, 2, 3, 4):
        g.advance(t)
    assert g.done()
    det = json_object_dfa().deterministic_transition(0)
    assert det is None  # whitespace or '{' are both legal at the start
