"""The imported decoder with every Linear packed as the reference's importer packs it (Gguf::load_llama(kind),
gguf/llama.rs:13-27,164-171: per-input-row int8 / int4 QWeights run by ops::qlinear) against the CPU oracle in the same
mode: full forward, cached decode, scoring, greedy generation, and the model loaded from a GGUF file."""
import numpy as np
import pytest

from ferrum_cpu_b200 import gguf_file, synth
from ferrum_cpu_b200.engine import sampling
from ferrum_cpu_b200.llama import CudaLlama
from tests import oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-4     # on logits of magnitude ~1: the kernel's fused multiply-adds against the oracle's separately rounded sums

CASES = [("norm", dict(), 0), ("norm4", dict(), 1), ("qwen", dict(qkv_bias=True, tied=False, rope_type=1, rope_base=1000000.0), 0),
         ("qwen4", dict(qkv_bias=True, tied=False, rope_type=1, rope_base=1000000.0), 1)]


@pytest.fixture(scope="module", params=CASES, ids=[c[0] for c in CASES])
def packed(request):
    _, kw, kind = request.param
    sm = synth.llama_named("llama-tiny", perturb=True, **kw)
    return sm, O.OracleLlama(sm, threads=4, prec=kind), CudaLlama.from_synth(sm, prec=kind), kind


def test_packing_changes_the_model(packed):
    """The packed model is a different function from the Q8_0 one (a per-row grid on top of the block grid): the test
    below would pass trivially if the packed path silently ran the Q8_0 matrices."""
    sm, om, gm, kind = packed
    ids = synth.token_ids(1, 12, sm.dims["vocab"])
    plain = O.OracleLlama(sm, threads=2).forward_tokens(ids)
    assert np.abs(om.forward_tokens(ids) - plain).max() > 10 * TOL


def test_forward_tokens_matches_oracle(packed):
    sm, om, gm, kind = packed
    ids = synth.token_ids(1, 33, sm.dims["vocab"])
    want, got = om.forward_tokens(ids), gm.forward_tokens(ids)
    assert np.abs(got - want).max() < TOL * max(1.0, float(np.abs(want).max()))


def test_cached_decode_matches_oracle_and_the_full_forward(packed):
    sm, om, gm, kind = packed
    ids = synth.token_ids(2, 20, sm.dims["vocab"])
    full = gm.forward_tokens(ids)
    cache = gm.new_cache()
    om.clear()
    for t, tok in enumerate(ids):
        got, want = gm.forward_one(tok, cache), om.forward_one(tok)
        scale = max(1.0, float(np.abs(want).max()))
        assert np.abs(got - want).max() < TOL * scale, t
        assert np.abs(got - full[t]).max() < TOL * scale, t
    assert cache.pos() == ids.size


def test_score_from_matches_oracle(packed):
    sm, om, gm, kind = packed
    ids = synth.token_ids(3, 50, sm.dims["vocab"])
    for start, window in ((1, 16), (7, 32), (1, 64)):
        total, n, greedy, lp, gr = om.score_from(ids, start, window)
        sc, glp, ggr = gm.score_from(ids, start, window, per_token=True)
        assert sc.n_tokens == n
        assert np.abs(glp - lp).max() < 1e-3                   # the stated bound on log-probs
        assert abs(sc.logprob - total) < 1e-3 * max(n, 1)


def test_greedy_generation_matches_oracle(packed):
    sm, om, gm, kind = packed
    prompt = synth.token_ids(4, 9, sm.dims["vocab"])
    want = om.generate(prompt, 16, O.Rng(1), temperature=0.0)
    got, _ = gm.generate(prompt, 16, sampling(temperature=0.0))
    n = min(len(got), len(want))
    # tokens agree until a step where the oracle's own top two are closer than the tolerance
    for i in range(n):
        if got[i] != want[i]:
            om.clear()
            logits = None
            for t in list(prompt) + list(want[:i]):
                logits = om.forward_one(int(t))
            top = np.sort(logits)[-2:]
            assert top[1] - top[0] < 10 * TOL, f"token {i}: got {got[i]}, want {want[i]}, margin {top[1] - top[0]:.3e}"
            break


def test_model_from_file_equals_model_from_arrays(tmp_path):
    sm = synth.llama_named("llama-tiny", perturb=True, seed=7)
    path = gguf_file.write_llama_gguf(tmp_path / "tiny.gguf", sm)
    ids = synth.token_ids(5, 24, sm.dims["vocab"])
    for kind in (0, 1):
        a, b = CudaLlama.from_synth(sm, prec=kind), CudaLlama.from_gguf(path, prec=kind)
        assert np.array_equal(a.forward_tokens(ids), b.forward_tokens(ids))
        a.close()
        b.close()
