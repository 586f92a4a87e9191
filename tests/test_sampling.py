"""Device sampler (sample.cu) against the oracle's restatement of slm/sampling.rs:124-210."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import ferrum_cpu_b200 as fcb  # noqa: E402
from ferrum_cpu_b200 import synth  # noqa: E402
from tests import oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def _pair(logits, seed, recent=(), **kw):
    """(oracle token, device token) for the same generator state; both advance it the same way."""
    rng = O.Rng(seed)
    start = rng.state.value
    want = O.sample_with_params(logits, rng, recent=recent, **kw)
    got, state = fcb.sample_logits(logits, start, fcb.sampling(**kw), recent=recent)
    assert state == rng.state.value, "the device must advance the generator exactly as the reference"
    return want, got


def test_known_answers_of_the_reference_hold_on_the_device():
    # sampling.rs:397-423, :219-231, :297-335
    logits = [0.1, 2.0, 1.9, -1.0]
    for t in (0.0, -1.0):
        for s in range(5):
            assert _pair(logits, s, temperature=t) == (1, 1)
    assert _pair(logits, 0, recent=[1], temperature=0.0, repetition_penalty=2.0) == (2, 2)
    assert _pair([1.0, 5.0, 5.0], 1, temperature=0.0) == (1, 1)
    assert _pair([0.5, -1.2, 2.3], 1, recent=[99], temperature=0.0, repetition_penalty=1.5)[1] == 2
    for s in range(50):
        assert _pair([5.0, 4.0, -2.0, -3.0, -5.0], s, top_k=2)[1] in (0, 1)
        assert _pair([10.0, 1.0, 0.5, 0.0], s, top_p=0.5)[1] == 0
    ones = sum(_pair([4.0, 3.0, -2.0], s, recent=[0], repetition_penalty=100.0)[1] == 1 for s in range(200))
    assert ones > 160


def _cdf64(logits, recent, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0):
    """The filtered distribution of sample_with_params in float64 (no rounding to speak of)."""
    w = np.asarray(logits, dtype=np.float64).copy()
    if abs(repetition_penalty - 1.0) > 1.2e-7 and repetition_penalty > 0:
        for t in recent:
            w[t] = w[t] / repetition_penalty if w[t] > 0 else w[t] * repetition_penalty
    t = max(temperature, 0.01)
    p = np.exp((w - w.max()) / t)
    p /= p.sum()
    if 0 < top_k < p.size:
        p[p < np.sort(p)[::-1][top_k - 1]] = 0.0
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cum = np.cumsum(p[order])
        n_keep = int(np.searchsorted(cum, top_p, side="left")) + 1
        keep = np.zeros(p.size, dtype=bool)
        keep[order[:n_keep]] = True
        p[~keep] = 0.0
    p /= p.sum()
    return p, np.cumsum(p)


@pytest.mark.parametrize("kw", [dict(), dict(temperature=0.7), dict(top_k=40), dict(top_p=0.9), dict(temperature=0.8, top_k=50, top_p=0.95),
                                dict(temperature=1.2, repetition_penalty=1.3)])
def test_draws_follow_the_reference_distribution_on_vocabulary_sized_rows(kw):
    """V = 50257 log-probabilities. The reference adds 50257 f32 terms one after the other, so its
    own rounding (about 1e-5 of the unit mass) is as large as a token's probability and no
    parallel sum can reproduce its index bit for bit. What both must satisfy: the drawn token
    carries mass, and the draw r lies inside the token's slice of the exact cumulative
    distribution widened by 2e-4; the generator state agrees on every draw."""
    V = 50257
    raw = synth.Rng(5).normal(V, 2.5)
    logp = (raw - np.log(np.exp(raw.astype(np.float64)).sum())).astype(np.float32)
    recent = synth.token_ids(9, 300, V)
    p, cdf = _cdf64(logp, recent, **kw)
    same = 0
    for seed in range(1, 41):
        r = O.Rng(seed).next_f32()
        want, got = _pair(logp, seed, recent=recent, **kw)
        for tok in (want, got):
            assert p[tok] > 0.0, "a token that top-k / top-p removed was drawn"
            lo = cdf[tok] - p[tok]
            assert lo - 2e-4 <= r <= cdf[tok] + 2e-4, (tok, r, lo, cdf[tok])
        same += want == got
    assert same >= 20      # most draws agree index for index


def test_greedy_with_penalty_matches_exactly_on_vocabulary_sized_rows():
    V = 50257
    logp = synth.Rng(6).normal(V, 2.5)
    recent = synth.token_ids(9, 300, V)
    for rp in (1.0, 1.2, 3.0):
        want, got = _pair(logp, 1, recent=recent, temperature=0.0, repetition_penalty=rp)
        assert want == got
    # the most likely tokens sit in `recent`: the penalty decides
    top = np.argsort(-logp)[:3]
    want, got = _pair(logp, 1, recent=list(top[:2]) * 2, temperature=0.0, repetition_penalty=50.0)
    assert want == got


def test_generate_sampled_follows_the_reference_loop():
    """token_stream.rs:66-189 with a sampler: prime, draw from ln(max(p, 1e-12)) with the window as
    `recent`, feed, repeat; re-prime on ctx/2 when the window outgrows the context."""
    sm = synth.SynthModel(2, 64, 2, 128, 24, 96, seed=3, perturb=True)
    om = O.OracleModel(sm)
    gm = fcb.CudaSlm(sm.config, sm.weights)
    prompt = synth.token_ids(4, 6, 96)
    kw = dict(temperature=0.9, top_k=20, top_p=0.9, repetition_penalty=1.2)
    rng = O.Rng(77)
    start = rng.state.value
    # the reference loop on the oracle
    window = list(prompt)
    dist = om.prime(window)
    want = []
    for _ in range(30):                                   # 6 + 30 > 24: crosses a re-prime
        logits = np.log(np.maximum(dist, np.float32(1e-12))).astype(np.float32)
        nxt = O.sample_with_params(logits, rng, recent=window, **kw)
        want.append(nxt)
        window.append(nxt)
        if len(window) > 24:
            window = window[-12:]
            dist = om.prime(window)
        else:
            dist = om.feed(nxt)
    got, state = gm.generate_sampled(prompt, 30, fcb.sampling(**kw), start)
    assert state == rng.state.value
    # identical until (if ever) a draw lands on a rounding boundary; from there the windows differ
    same = 0
    while same < 30 and got[same] == want[same]:
        same += 1
    assert same >= 25, f"sequences split after {same} tokens: {got[:same + 1]} vs {want[:same + 1]}"
    # temperature 0 is the greedy path with the penalty applied
    g0, _ = gm.generate_sampled(prompt, 10, fcb.sampling(temperature=0.0), 1)
    g1, _ = gm.generate_tokens(prompt, 10)
    assert np.array_equal(g0, g1)
    gm.close()
    om.close()
