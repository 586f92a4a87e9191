"""Several model handles behind one C call (fc_score_sequences_multi / fc_decode_batch_multi) and the
per-layer statistics trace (fc_model_set_layer_stats)."""
import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import engine, synth
from tests import oracle as O

pytestmark = pytest.mark.gpu


def _models(sm, n):
    """n handles on the visible GPUs (round robin: on a one-GPU box they share the device, which exercises
    the same host-thread plumbing)."""
    ndev = fcb.device_count()
    return [fcb.CudaSlm(sm.config, sm.weights, device=i % ndev) for i in range(n)]


def test_multi_model_scoring_equals_one_model():
    sm = synth.named("tiny", seed=0, perturb=True)
    V, T = sm.dims[5], sm.dims[4]
    ids = synth.token_ids(9, 7 * T, V).reshape(7, T)          # 7 sequences over 3 handles: blocks of 2, 2, 3
    one = fcb.CudaSlm(sm.config, sm.weights)
    want_scores, want_lp = one.score_sequences(ids, batch_windows=4)
    models = _models(sm, 3)
    fcb.take_launch_count()
    scores, lp = engine.score_sequences_multi(models, ids, batch_windows=4)
    assert fcb.take_launch_count() > 0                          # the workers' launches are credited to the caller
    assert np.array_equal(lp, want_lp)
    for a, b in zip(scores, want_scores):
        assert a.logprob == b.logprob and a.n_tokens == b.n_tokens and a.greedy == b.greedy
    # an error inside one worker comes back as that model's status and message
    bad = ids.copy()
    bad[5, 3] = V
    with pytest.raises(fcb.FerrumCudaError) as e:
        engine.score_sequences_multi(models, bad)
    assert e.value.code == fcb._lib.FC_E_DIM and "model 2 of 3" in str(e.value)
    for m in models + [one]:
        m.close()


def test_multi_model_decode_equals_one_model():
    sm = synth.named("tiny", seed=0, perturb=True)
    V = sm.dims[5]
    prompts = np.stack([synth.token_ids(60 + i, 12, V) for i in range(9)])
    one = fcb.CudaSlm(sm.config, sm.weights)
    want = one.decode_batch(prompts, 16)
    models = _models(sm, 2)
    got = engine.decode_batch_multi(models, prompts, 16)
    # streams are independent: how they are batched (9 in one lock-step batch, or 4 + 5) cannot change a token
    for a, b in zip(got, want):
        assert np.array_equal(a, b)
    for m in models + [one]:
        m.close()


@pytest.mark.parametrize("mode", [fcb.FC_MATH_FP32, fcb.FC_MATH_BF16X3])
def test_layer_stats_records(mode):
    """One record per layer output; the embedding record against exact host arithmetic
    (verbose::stats, verbose.rs:85-100), and the NaN / Inf counts of a healthy model are zero."""
    sm = synth.SynthModel(2, 128, 2, 256, 32, 200, seed=3, perturb=True, math_mode=mode)   # head_dim 64: both paths
    gm = fcb.CudaSlm(sm.config, sm.weights)
    gm.set_layer_stats(True)
    ids = synth.token_ids(4, 32, 200)
    gm.token_logprobs(ids, 1)
    st = gm.layer_stats()
    assert len(st) == sm.dims[0] + 2
    for rec in st:
        assert rec["nan_count"] == 0 and rec["inf_count"] == 0 and rec["n_elements"] == 32 * 128
        assert rec["min"] <= rec["mean"] <= rec["max"]
    # the embedding record is exact arithmetic on both sides: tok[id] + pos[t]
    tok = synth.q8_0_dequantize(sm.token_embd, 200 * 128).reshape(200, 128)
    emb = tok[ids] + sm.position_embd.reshape(32, 128)
    assert st[0]["min"] == emb.min() and st[0]["max"] == emb.max() and abs(st[0]["mean"] - emb.mean(dtype=np.float64)) < 1e-6
    # the final LayerNorm of a row has (gain-weighted) zero mean and unit scale: a sanity range, not a parity claim
    assert abs(st[-1]["mean"]) < 0.5 and st[-1]["max"] < 10 and st[-1]["min"] > -10
    gm.set_layer_stats(False)
    gm.token_logprobs(ids, 1)
    assert gm.layer_stats() == []
    gm.close()
