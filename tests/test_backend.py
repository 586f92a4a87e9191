"""Cross-request batched scoring (fc_score_requests) and the Backend mirror: every request gets
the score it gets alone, whatever it shares a forward pass with."""
import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import _lib, synth
from ferrum_cpu_b200.backend import CudaBackend, GenRequest
from tests import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny():
    sm = synth.named("tiny", seed=0, perturb=True)
    return sm, O.OracleModel(sm, threads=4), fcb.CudaSlm(sm.config, sm.weights)


def test_requests_batched_together_score_as_they_do_alone(tiny):
    sm, om, gm = tiny
    V, T = sm.dims[5], sm.dims[4]
    rng = np.random.default_rng(3)
    reqs = []
    for i, n in enumerate([2, 5, 40, T, T + 1, 3 * T + 7, 17, 1, 0, 300]):
        ids = synth.token_ids(50 + i, n, V) if n else np.zeros(0, np.int32)
        reqs.append((ids, int(rng.integers(0, max(n, 1) + 1))))
    got = gm.score_requests(reqs, batch_windows=4)
    for (ids, start), s in zip(reqs, got):
        one = gm.token_logprobs(ids, start) if ids.size else fcb.Score(0.0, 0, True)
        assert s.n_tokens == one.n_tokens and s.greedy == one.greedy
        assert abs(s.logprob - one.logprob) < 1e-6 * max(1, s.n_tokens)
    # and as the oracle scores them
    ids, start = reqs[5]
    total, n, greedy, _, _ = om.token_logprobs(ids, start)
    assert got[5].n_tokens == n and abs(got[5].logprob - total) < 2e-4 * n
    with pytest.raises(fcb.FerrumCudaError) as e:
        gm.score_requests([(np.array([1, V], np.int32), 1)])
    assert e.value.code == _lib.FC_E_DIM


def test_backend_answers_queued_requests_in_one_flush(tiny):
    sm, om, gm = tiny
    V = sm.dims[5]
    be = CudaBackend(gm, batch_windows=8)
    ctx, cont = synth.token_ids(1, 12, V), synth.token_ids(2, 5, V)
    text = synth.token_ids(3, 200, V)
    t1, t2, t3 = be.submit_score(ctx, cont), be.submit_score_rolling(text), be.submit_score(ctx[:1], cont)
    replies = be.flush()
    assert set(replies) == {t1, t2, t3} and be.flush() == {}
    alone = gm.token_logprobs(np.concatenate([ctx, cont]), len(ctx))
    assert replies[t1]["n_tokens"] == 5 and abs(replies[t1]["logprob"] - alone.logprob) < 1e-6
    assert replies[t1]["greedy"] == alone.greedy and "greedy" not in replies[t2]
    assert replies[t2]["n_tokens"] == 199
    assert be.score(ctx, cont) == replies[t1]
    assert be.score_rolling(text) == replies[t2]
    with pytest.raises(fcb.FerrumCudaError):
        be.submit_score([], cont)


def test_backend_generate(tiny):
    sm, om, gm = tiny
    V = sm.dims[5]
    be = CudaBackend(gm)
    prompt = [int(t) for t in synth.token_ids(4, 8, V)]
    greedy = be.generate(GenRequest(prompt, max_tokens=12, temperature=0.0))
    want, _ = om.generate_greedy(np.array(prompt, np.int32), 12)
    assert greedy["n_tokens"] == 12 and greedy["tokens"][:4] == [int(t) for t in want[:4]]
    a = be.generate(GenRequest(prompt, max_tokens=10, temperature=0.9, top_k=50, top_p=0.95, seed=7))
    b = be.generate(GenRequest(prompt, max_tokens=10, temperature=0.9, top_k=50, top_p=0.95, seed=7))
    assert a == b and a["n_tokens"] == 10
    gone = np.ones(1, dtype=np.int32)
    assert be.generate(GenRequest(prompt, cancel=gone)) is None      # the client already left
