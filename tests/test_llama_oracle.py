"""Pins the CPU restatement of the Llama / Qwen decoder (oracle/llama_oracle.cpp) on the
known-answer values of the reference's own unit tests (ferrum_core/src/llm.rs:788-1160,
llm_score.rs:100-138). No GPU."""
import math

import numpy as np
import pytest

from ferrum_cpu_b200 import synth
from tests import oracle as O


def det(n, seed):
    """The deterministic test generator of llm.rs:772-782: xorshift (13, 7, 17), top 24 bits -> [-1, 1)."""
    x = (seed | 1) & 0xFFFFFFFFFFFFFFFF
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        x ^= (x << 13) & 0xFFFFFFFFFFFFFFFF
        x ^= x >> 7
        x ^= (x << 17) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(x >> 40) / np.float32(1 << 23) - np.float32(1.0))
    return out


# ---- RMSNorm (llm.rs:790-812) ------------------------------------------------------------
def test_rmsnorm_matches_formula():
    w = np.array([2.0, 0.5, 1.0, 1.5], dtype=np.float32)
    x = np.array([1.0, -2.0, 3.0, 0.5], dtype=np.float32)
    out = O.rmsnorm(x, w, 1e-6)
    ms = np.float32((x * x).sum(dtype=np.float32) / np.float32(4.0))
    inv = np.float32(1.0) / np.sqrt(np.float32(ms + np.float32(1e-6)))
    assert np.abs(out - x * inv * w).max() < 1e-6


def test_rmsnorm_unit_weight_gives_unit_rms():
    out = O.rmsnorm(det(8, 5), np.ones(8, dtype=np.float32), 1e-6)
    assert abs(math.sqrt(float((out * out).sum()) / 8.0) - 1.0) < 1e-3


# ---- RoPE (llm.rs:816-933) ---------------------------------------------------------------
@pytest.mark.parametrize("neox", [False, True])
def test_rope_at_position_zero_is_identity(neox):
    x = det(16, 9)
    assert np.abs(O.apply_rope(x, 2, 8, 8, 0, neox=neox) - x).max() < 1e-6


@pytest.mark.parametrize("neox", [False, True])
def test_rope_preserves_norm(neox):
    x = det(8, 3)
    y = O.apply_rope(x, 1, 8, 8, 5, neox=neox)
    assert abs(float((x * x).sum()) - float((y * y).sum())) < 1e-4


def test_rope_norm_and_neox_differ():
    x = det(8, 7)
    assert np.abs(O.apply_rope(x, 1, 8, 8, 3) - O.apply_rope(x, 1, 8, 8, 3, neox=True)).max() > 1e-3


@pytest.mark.parametrize("neox", [False, True])
def test_rope_with_unit_factors_is_bit_identical_to_unscaled(neox):
    for pos in (0, 1, 5, 17, 300):
        x = det(16, 3)
        a = O.apply_rope(x, 2, 8, 8, pos, neox=neox)
        b = O.apply_rope(x, 2, 8, 8, pos, neox=neox, freq_factors=[1.0] * 4, linear_factor=1.0)
        assert a.tobytes() == b.tobytes()


def test_rope_freq_factors_hand_computed():
    # llm.rs:894-918: head_dim = rope_dim = 4, base 10000, factors [1, 4]: t0 = pos, t1 = pos * 0.01 / 4
    want = {2: [-0.41614684, 0.9092974, 0.9999875, 0.004999979], 7: [0.75390225, 0.6569866, 0.9998469, 0.017499107]}
    for pos, w in want.items():
        x = O.apply_rope([1.0, 0.0, 1.0, 0.0], 1, 4, 4, pos, freq_factors=[1.0, 4.0])
        assert np.abs(x - np.array(w, dtype=np.float32)).max() < 1e-6
        y = O.apply_rope([1.0, 1.0, 0.0, 0.0], 1, 4, 4, pos, neox=True, freq_factors=[1.0, 4.0])
        assert np.abs(y - np.array([w[0], w[2], w[1], w[3]], dtype=np.float32)).max() < 1e-6


@pytest.mark.parametrize("neox", [False, True])
def test_linear_factor_two_halves_the_effective_position(neox):
    for pos in (2, 6, 10, 64):
        x = det(8, 9)
        a = O.apply_rope(x, 1, 8, 8, pos, neox=neox, linear_factor=2.0)
        b = O.apply_rope(x, 1, 8, 8, pos // 2, neox=neox)
        assert a.tobytes() == b.tobytes()


def test_partial_rotary_leaves_the_tail_of_each_head():
    x = det(16, 11)
    y = O.apply_rope(x, 2, 8, 4, 9)
    assert np.array_equal(y[4:8], x[4:8]) and np.array_equal(y[12:16], x[12:16])
    assert np.abs(y[:4] - x[:4]).max() > 1e-3


# ---- SwiGLU (llm.rs:1032-1051) -----------------------------------------------------------
def test_silu_gate_matches_manual():
    g, u = det(6, 1), det(6, 2)
    want = (g / (np.float32(1.0) + np.exp(-g))) * u
    assert np.abs(O.silu_mul(g, u) - want).max() < 1e-6


# ---- windows and log-softmax (llm_score.rs:104-138) --------------------------------------
def test_windows_cover_every_target_once_with_half_a_window_of_history():
    for n, w in [(2, 2), (5, 8), (9, 8), (40, 8), (41, 7), (100, 16)]:
        nxt = 1
        for start, first, end in O.llama_plan_windows(n, w, 1):
            assert first == nxt
            assert end > first and end - start <= w + 1
            assert start == 0 or first - start >= w // 2
            nxt = end
        assert nxt == n
    assert O.llama_plan_windows(5, 8, 1) == [(0, 1, 5)]


def test_windows_start_at_the_first_scored_target():
    assert O.llama_plan_windows(5, 8, 3) == [(0, 3, 5)]
    assert O.llama_plan_windows(5, 8, 0) == O.llama_plan_windows(5, 8, 1)
    assert O.llama_plan_windows(5, 8, 5) == []
    assert O.llama_plan_windows(30, 8, 20) == [(16, 20, 25), (21, 25, 30)]


def test_log_prob_is_a_normalised_log_softmax():
    logits = [1.0, 2.0, 3.0, -1.0]
    assert abs(sum(math.exp(O.llama_log_prob(logits, t)) for t in range(4)) - 1.0) < 1e-12
    assert abs(O.llama_log_prob([0.0, 0.0], 1) + math.log(2.0)) < 1e-12


# ---- model (llm.rs:974-1160, 1275-1420) --------------------------------------------------
def tiny(**kw):
    return synth.llama_named("llama-tiny", perturb=True, **kw)


@pytest.mark.parametrize("kw", [dict(), dict(rope_type=1), dict(freq_factors=[1.0, 4.0] * 4, rope_linear_factor=2.0),
                                dict(qkv_bias=True, tied=False), dict(rope_dim=8)])
def test_cached_decode_matches_full_forward(kw):
    sm = tiny(**kw)
    m = O.OracleLlama(sm)
    assert m.ok
    tokens = [3, 7, 1, 9, 4, 0, 500, 7]
    full = m.forward_tokens(tokens)
    for t, tok in enumerate(tokens):
        got = m.forward_one(tok)
        assert np.abs(got - full[t]).max() < 1e-3
    assert m.pos() == len(tokens)
    m.clear()
    assert m.pos() == 0


def test_scaling_changes_the_logits():
    tokens = [3, 7, 1, 9, 4, 0]
    plain = O.OracleLlama(tiny()).forward_tokens(tokens)
    scaled = O.OracleLlama(tiny(freq_factors=[1.0, 4.0] * 4, rope_linear_factor=2.0)).forward_tokens(tokens)
    assert not np.array_equal(plain, scaled)
    assert np.array_equal(plain[0], scaled[0])         # position 0 is never rotated


def test_create_refuses_what_the_reference_refuses():
    # llm.rs:1012-1027 (5 heads cannot share 2 KV heads), :1342-1371 (odd / oversized rope_dim), :936-951 (factors)
    shape = list(synth.LLAMA_SHAPES["llama-tiny"])
    bad_gqa = list(shape)
    bad_gqa[3], bad_gqa[4], bad_gqa[5] = 6, 4, 16
    assert not O.OracleLlama(synth.SynthLlama(*bad_gqa)).ok
    assert not O.OracleLlama(tiny(rope_dim=5)).ok
    assert not O.OracleLlama(tiny(rope_dim=32)).ok
    assert not O.OracleLlama(tiny(freq_factors=[1.0, 0.0] * 4)).ok
    assert not O.OracleLlama(tiny(freq_factors=[1.0, float("nan")] * 4)).ok
    assert not O.OracleLlama(tiny(rope_linear_factor=0.0)).ok
    assert not O.OracleLlama(tiny(rope_linear_factor=-2.0)).ok


def test_score_from_matches_one_forward_per_window():
    sm = tiny()
    m = O.OracleLlama(sm)
    ids = synth.token_ids(3, 40, sm.dims["vocab"])
    total, n, greedy, lp, gr = m.score_from(ids, 1, 16)
    assert n == 39
    assert abs(total - float(lp.sum())) < 1e-9
    # a text that fits one window is one forward pass: each target is the log-softmax of its row
    total1, n1, _, lp1, _ = m.score_from(ids[:12], 1, 16)
    logits = m.forward_tokens(ids[:12])
    want = [O.llama_log_prob(logits[t - 1], int(ids[t])) for t in range(1, 12)]
    assert n1 == 11 and np.abs(lp1 - np.array(want)).max() < 1e-12
    # the conditioning prefix is not scored
    total3, n3, _, lp3, _ = m.score_from(ids[:12], 5, 16)
    assert n3 == 7 and abs(total3 - float(lp1[4:].sum())) < 1e-9
    assert m.score_from(ids, 1, 1) is None and m.score_from(ids, 1, sm.dims["ctx"] + 1) is None


def test_generate_is_deterministic_respects_stops_and_the_context():
    sm = tiny()
    m = O.OracleLlama(sm)
    prompt = [1, 2, 3]
    a = m.generate(prompt, 12, O.Rng(7), temperature=0.8, top_k=40, top_p=0.95)
    b = m.generate(prompt, 12, O.Rng(7), temperature=0.8, top_k=40, top_p=0.95)
    assert np.array_equal(a, b) and a.size == 12
    # top_k = 1 is greedy whatever the seed (llm.rs:1304-1322)
    g1 = m.generate(prompt, 8, O.Rng(1), temperature=1.0, top_k=1)
    g2 = m.generate(prompt, 8, O.Rng(99), temperature=1.0, top_k=1)
    g0 = m.generate(prompt, 8, O.Rng(5), temperature=0.0)
    assert np.array_equal(g1, g2) and np.array_equal(g1, g0)
    # a stop id ends the generation and is kept
    s = m.generate(prompt, 8, O.Rng(5), temperature=0.0, stops=[int(g0[2])])
    assert s.size <= 3 and s[-1] == g0[2]
    # the context window bounds prompt and generation (llm.rs:1380-1408)
    ctx = sm.dims["ctx"]
    assert m.generate(list(range(ctx)), 4, O.Rng(1)) is None
    long = m.generate(list(range(ctx - 3)), 50, O.Rng(1), temperature=0.0)
    assert long.size == 3
    assert m.generate([], 4, O.Rng(1)) is None
