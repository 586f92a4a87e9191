"""Parity of the Llama / Qwen CUDA path (through the C ABI) with the CPU oracle, on seeded
synthetic Q8_0 models. Tolerance: 1e-3 max-abs on log-probs and logits; greedy tokens equal
wherever the oracle's top-two margin is above the tolerance."""
import ctypes as C

import numpy as np
import pytest

from ferrum_cpu_b200 import _lib, synth
from ferrum_cpu_b200.engine import FerrumCudaError, sampling
from ferrum_cpu_b200.llama import CudaLlama
from tests import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-3
FP32_TOL = 2e-4

VARIANTS = {
    "norm": dict(),
    "neox": dict(rope_type=1),
    "scaled": dict(freq_factors=[1.0, 4.0, 1.5, 2.0, 1.0, 8.0, 1.0, 3.0], rope_linear_factor=2.0),
    "qwen": dict(qkv_bias=True, tied=False, rope_type=1, rope_base=1000000.0),
    "partial": dict(rope_dim=8),
}


def build(name="llama-tiny", math_mode=0, **kw):
    sm = synth.llama_named(name, perturb=True, math_mode=math_mode, **kw)
    return sm, O.OracleLlama(sm, threads=4), CudaLlama.from_synth(sm)


@pytest.fixture(scope="module", params=sorted(VARIANTS))
def tiny(request):
    return build(**VARIANTS[request.param])


@pytest.fixture(scope="module")
def mini():
    return build("llama-mini", seed=5)


def test_forward_tokens_matches_oracle(tiny):
    sm, om, gm = tiny
    ids = synth.token_ids(1, 33, sm.dims["vocab"])
    want, got = om.forward_tokens(ids), gm.forward_tokens(ids)
    assert np.abs(got - want).max() < FP32_TOL


def test_cached_decode_matches_oracle_and_the_full_forward(tiny):
    sm, om, gm = tiny
    ids = synth.token_ids(2, 20, sm.dims["vocab"])
    full = gm.forward_tokens(ids)
    cache = gm.new_cache()
    om.clear()
    for t, tok in enumerate(ids):
        got, want = gm.forward_one(tok, cache), om.forward_one(tok)
        assert np.abs(got - want).max() < FP32_TOL, t
        assert np.abs(got - full[t]).max() < FP32_TOL, t      # llm.rs:1123-1141
    assert cache.pos() == ids.size
    cache.clear()
    assert cache.pos() == 0
    assert np.abs(gm.forward_one(ids[0], cache) - full[0]).max() < FP32_TOL


def test_score_from_matches_oracle(tiny):
    sm, om, gm = tiny
    ids = synth.token_ids(3, 100, sm.dims["vocab"])
    for start, window in [(1, 64), (1, 16), (30, 24), (0, 7), (100, 16)]:
        total, n, greedy, lp, gr = om.score_from(ids, start, window)
        sc, glp, ggr = gm.score_from(ids, start, window, per_token=True)
        assert sc.n_tokens == n
        assert np.abs(glp - lp).max() < FP32_TOL
        assert abs(sc.logprob - total) < FP32_TOL * max(n, 1)
        assert np.array_equal(ggr, gr) and sc.greedy == greedy
    sc = gm.score_rolling(ids[:9], 16)
    assert sc.n_tokens == 8


def test_score_sequences_matches_score_from(mini):
    sm, om, gm = mini
    ids = synth.token_ids(4, 5 * 48, sm.dims["vocab"]).reshape(5, 48)
    scores, lp = gm.score_sequences(ids, batch_windows=2, per_token=True)
    for i in range(5):
        one, olp, _ = gm.score_from(ids[i], 1, 64, per_token=True)
        assert scores[i].n_tokens == 47 and abs(scores[i].logprob - one.logprob) < 1e-6
        assert np.abs(lp[i] - olp).max() < 1e-6
    total, n, greedy, wlp, _ = om.score_from(ids[0], 1, 64)
    assert np.abs(lp[0] - wlp).max() < FP32_TOL


def test_mini_model_forward_and_decode(mini):
    # head_dim 32 (the tiled window kernel), 4 query heads per key/value head, d_ff 704
    sm, om, gm = mini
    ids = synth.token_ids(6, 70, sm.dims["vocab"])
    want, got = om.forward_tokens(ids), gm.forward_tokens(ids)
    assert np.abs(got - want).max() < FP32_TOL
    cache = gm.new_cache()
    for t, tok in enumerate(ids[:24]):
        assert np.abs(gm.forward_one(tok, cache) - want[t]).max() < FP32_TOL


def test_batched_prime_equals_token_by_token(tiny, mini):
    for sm, om, gm in (tiny, mini):
        ids = synth.token_ids(13, 40, sm.dims["vocab"])
        a, b = gm.new_cache(), gm.new_cache()
        step = None
        for t in ids[:32]:
            step = gm.forward_one(t, a)
        batched = gm.prime(ids[:32], b)
        assert b.pos() == a.pos() == 32
        assert np.abs(batched - step).max() < 1e-4
        om.clear()
        want = None
        for t in ids[:32]:
            want = om.forward_one(t)
        assert np.abs(batched - want).max() < FP32_TOL
        for t in ids[32:]:                                   # the filled caches carry the decode on
            assert np.abs(gm.forward_one(t, a) - gm.forward_one(t, b)).max() < 1e-4
        short = gm.prime(ids[:5], b)                          # below the threshold: the step path
        om.clear()
        for t in ids[:5]:
            want = om.forward_one(t)
        assert b.pos() == 5 and np.abs(short - want).max() < FP32_TOL


def test_narrow_deep_model_decode_matches_forward_and_oracle():
    # 16 blocks, vocabulary 32000, d 512 / F 2048: the ring GEMV's tile shapes for wide rows, a long chain of steps
    sm = synth.llama_named("llama-narrow", seed=3)
    gm = CudaLlama.from_synth(sm)
    ids = synth.token_ids(14, 24, sm.dims["vocab"])
    full = gm.forward_tokens(ids)
    cache = gm.new_cache()
    for t, tok in enumerate(ids):
        assert np.abs(gm.forward_one(tok, cache) - full[t]).max() < FP32_TOL, t
    om = O.OracleLlama(sm, threads=8)
    want = om.forward_tokens(ids[:6])
    assert np.abs(full[:6] - want).max() < FP32_TOL
    out1, _ = gm.generate(ids[:12], 16, sampling(temperature=0.0))
    out2, _ = gm.generate(ids[:12], 16, sampling(temperature=0.0))
    assert np.array_equal(out1, out2)                         # bitwise repeatable
    gm.close()


def test_tensor_core_window_forward_stays_within_tolerance():
    sm, om, gm = build("llama-mini", math_mode=_lib.FC_MATH_BF16X3, seed=5)
    ids = synth.token_ids(6, 200, sm.dims["vocab"])
    want, got = om.forward_tokens(ids), gm.forward_tokens(ids)
    assert np.abs(got - want).max() < TOL
    total, n, greedy, lp, gr = om.score_from(ids, 1, 128)
    sc, glp, ggr = gm.score_from(ids, 1, 128, per_token=True)
    assert sc.n_tokens == n and np.abs(glp - lp).max() < TOL


def test_tensor_core_attention_with_grouped_heads():
    # head_dim 64 in the bf16x3 mode: rotated q | k | v planes -> tcgen05 attention -> wo GEMM from planes
    sm, om, gm = build("llama-hd64", math_mode=_lib.FC_MATH_BF16X3, seed=9, rope_type=1, qkv_bias=True)
    V = sm.dims["vocab"]
    ids = synth.token_ids(21, 300, V)
    want, got = om.forward_tokens(ids), gm.forward_tokens(ids)
    assert np.abs(got - want).max() < TOL
    seqs = synth.token_ids(22, 3 * 100, V).reshape(3, 100)          # windows that are no multiple of the 128-row tile
    scores, lp = gm.score_sequences(seqs, batch_windows=3, per_token=True)
    for i in range(3):
        total, n, greedy, wlp, _ = om.score_from(seqs[i], 1, 128)
        assert scores[i].n_tokens == n and np.abs(lp[i] - wlp).max() < TOL
    # the fp32 mode of the same model (SIMT attention) agrees with the tensor-core mode
    sm.config.math_mode = _lib.FC_MATH_FP32
    g32 = CudaLlama.from_synth(sm)
    assert np.abs(g32.forward_tokens(ids) - got).max() < TOL
    g32.close()


@pytest.mark.parametrize("mode,tol", [(_lib.FC_MATH_FP32, FP32_TOL), (_lib.FC_MATH_BF16X3, TOL)])
def test_widths_that_are_no_powers_of_two(mode, tol):
    sm, om, gm = build("qwen-odd", math_mode=mode, seed=4, rope_type=1, qkv_bias=True, tied=False, rope_base=1000000.0)
    V = sm.dims["vocab"]
    ids = synth.token_ids(31, 150, V)
    want = om.forward_tokens(ids)
    assert np.abs(gm.forward_tokens(ids) - want).max() < tol
    cache = gm.new_cache()
    for t, tok in enumerate(ids[:20]):                       # the ring GEMV with 28 and 76 chunks per row
        assert np.abs(gm.forward_one(tok, cache) - want[t]).max() < FP32_TOL, t
    primed = gm.prime(ids[:40], cache)
    assert np.abs(primed - want[39]).max() < FP32_TOL
    total, n, greedy, lp, gr = om.score_from(ids, 1, 64)
    sc, glp, _ = gm.score_from(ids, 1, 64, per_token=True)
    assert sc.n_tokens == n and np.abs(glp - lp).max() < tol


def margins(om, prompt, tokens):
    """Top-two logit gap of the oracle at every generated position."""
    om.clear()
    logits = None
    for t in prompt:
        logits = om.forward_one(t)
    out = []
    for t in tokens:
        top = np.sort(logits)[-2:]
        out.append(float(top[1] - top[0]))
        logits = om.forward_one(t)
    return out


def test_greedy_generation_matches_oracle(tiny):
    sm, om, gm = tiny
    prompt = synth.token_ids(7, 6, sm.dims["vocab"])
    want = om.generate(prompt, 24, O.Rng(1), temperature=0.0)
    got, _ = gm.generate(prompt, 24, sampling(temperature=0.0))
    gap = margins(om, prompt, want)
    for i, (a, b) in enumerate(zip(got, want)):
        if a != b:
            assert gap[i] < TOL, f"token {i}: {a} != {b} with margin {gap[i]:.3e}"
            break
    assert got.size == want.size == 24
    # the cache holds the prompt and every kept token (llm.rs:750-751 feeds the last one too)
    assert gm.last_cache_pos == prompt.size + 24


def test_sampled_generation_matches_oracle(tiny):
    sm, om, gm = tiny
    prompt = synth.token_ids(8, 5, sm.dims["vocab"])
    for kw in (dict(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1), dict(temperature=1.0, top_k=1),
               dict(temperature=0.0, repetition_penalty=1.3)):
        rng = O.Rng(11)
        want = om.generate(prompt, 16, rng, **kw)
        got, state = gm.generate(prompt, 16, sampling(**kw), rng_state=O.Rng(11).state.value)
        assert np.array_equal(got, want), kw
        assert state == rng.state.value                      # the generator advanced exactly as the reference's


def test_stops_context_bound_and_cancel(tiny):
    sm, om, gm = tiny
    ctx = sm.dims["ctx"]
    prompt = synth.token_ids(9, 4, sm.dims["vocab"])
    free, _ = gm.generate(prompt, 10, sampling(temperature=0.0))
    stopped, _ = gm.generate(prompt, 10, sampling(temperature=0.0), stops=[int(free[3])])
    first = list(free).index(int(free[3]))
    assert np.array_equal(stopped, free[:first + 1])
    assert gm.last_cache_pos == prompt.size + first       # the stop id is kept but not fed
    long_prompt = synth.token_ids(10, ctx - 3, sm.dims["vocab"])
    out, _ = gm.generate(long_prompt, 50, sampling(temperature=0.0))
    assert out.size == 3                                     # llm.rs:730: max_new.min(ctx - prompt.len())
    with pytest.raises(FerrumCudaError) as e:
        gm.generate(synth.token_ids(10, ctx, sm.dims["vocab"]), 4, sampling())
    assert e.value.code == _lib.FC_E_DIM
    with pytest.raises(FerrumCudaError) as e:
        gm.generate([], 4, sampling())
    assert e.value.code == _lib.FC_E_DIM
    flag = C.c_int32(1)
    out, _ = gm.generate(prompt, 5, sampling(temperature=0.0), cancel=flag)
    assert out.size == 0                                     # cancelled while reading the prompt: nothing


def test_errors_are_statuses_not_traps(tiny):
    sm, om, gm = tiny
    V, ctx = sm.dims["vocab"], sm.dims["ctx"]
    with pytest.raises(FerrumCudaError) as e:
        gm.forward_tokens([1, V, 2])
    assert e.value.code == _lib.FC_E_DIM
    cache = gm.new_cache()
    with pytest.raises(FerrumCudaError) as e:
        gm.forward_one(V, cache)
    assert e.value.code == _lib.FC_E_DIM and cache.pos() == 0
    for t in synth.token_ids(12, ctx, V):
        gm.forward_one(t, cache, want_logits=False)
    assert cache.pos() == ctx
    with pytest.raises(FerrumCudaError) as e:
        gm.forward_one(1, cache)
    assert e.value.code == _lib.FC_E_DIM and cache.pos() == ctx
    for bad in (1, ctx + 1):
        with pytest.raises(FerrumCudaError) as e:
            gm.score_from([1, 2, 3], 1, bad)
        assert e.value.code == _lib.FC_E_DIM
    with pytest.raises(FerrumCudaError):
        gm.score_rolling([1], 8)


def test_1b_shape_matches_the_golden_fixture():
    """Llama-3.2-1B shape, synthetic weights: per-token log-probs and greedy tokens against
    tests/golden/llama_1b.npz (made by tests/golden/make_golden_llama.py from the oracle)."""
    import os
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llama_1b.npz"))
    sm = synth.llama_named("llama-1b", seed=0)
    ids = gold["ids"]
    for mode, tol in ((_lib.FC_MATH_FP32, FP32_TOL), (_lib.FC_MATH_BF16X3, TOL)):
        sm.config.math_mode = mode
        gm = CudaLlama.from_synth(sm)
        sc, lp, gr = gm.score_from(ids, 1, 2048, per_token=True)
        assert sc.n_tokens == ids.size - 1
        assert np.abs(lp - gold["logprob"]).max() < tol
        assert abs(sc.logprob - float(gold["total"])) < tol * sc.n_tokens
        assert np.array_equal(gr, gold["is_greedy"])
        if mode == _lib.FC_MATH_FP32:
            toks, _ = gm.generate(gold["prompt"], gold["tokens"].size, sampling(temperature=0.0))
            assert gold["margin"].min() > TOL and np.array_equal(toks, gold["tokens"])
            # size-independent property at the full shape: the cached path reproduces the window forward
            full = gm.forward_tokens(ids[:12])
            cache = gm.new_cache()
            for t, tok in enumerate(ids[:12]):
                assert np.abs(gm.forward_one(tok, cache) - full[t]).max() < FP32_TOL
        gm.close()
