"""The imported decoder with every matrix kept in the file's own block format and decoded inside the kernels
(fc_llama_load_gguf_native), against the CPU oracle running the reference's precision-preserving import
(load_llama_prec(None), gguf/llama.rs:171-176): the same file's tensors decoded to f32 by the numpy restatement of
gguf/dequant.rs and handed to the oracle as f32 Linears and an f32 embedding table."""
import ctypes as C

import numpy as np
import pytest

from ferrum_cpu_b200 import _lib, gguf_file, synth
from ferrum_cpu_b200.engine import sampling
from ferrum_cpu_b200.llama import CudaLlama
from tests import oracle as O
from tests.test_ggml_formats import GD, random_any

pytestmark = pytest.mark.gpu
TOL = 2e-4

STEMS = [("attn_q", "wq_q8"), ("attn_k", "wk_q8"), ("attn_v", "wv_q8"), ("attn_output", "wo_q8"), ("ffn_gate", "gate_q8"),
         ("ffn_up", "up_q8"), ("ffn_down", "down_q8")]


@pytest.fixture(scope="module")
def native(tmp_path_factory):
    """Rows of 256 and 512 values, matrices in a mix of formats; returns (dims, oracle on the decoded f32 tensors,
    model with the blocks resident as stored)."""
    sm = synth.SynthLlama(384, 256, 2, 4, 2, 64, 512, 64, perturb=True, seed=3)
    c = sm.dims
    d, F, qd, kvd = c["d_model"], c["d_ff"], c["n_head"] * c["head_dim"], c["n_kv_head"] * c["head_dim"]
    shapes = {"attn_q": (qd, d), "attn_k": (kvd, d), "attn_v": (kvd, d), "attn_output": (d, qd), "ffn_gate": (F, d),
              "ffn_up": (F, d), "ffn_down": (d, F)}
    kinds = [GD.Q4_K, GD.Q6_K, GD.Q4_0, GD.Q5_K, GD.Q5_0, GD.Q8_0, GD.Q4_1, GD.F16, GD.Q2_K, GD.Q3_K, GD.Q5_1]
    raw, decoded, seed = {}, {}, 30

    def put(name, n, k):
        nonlocal seed
        t = kinds[seed % len(kinds)]
        blocks = random_any(t, n * k, seed)
        raw[name] = (t, blocks)
        decoded[name] = GD.dequantize(t, blocks, n * k).reshape(n, k)
        seed += 1

    for i in range(c["n_layer"]):
        for stem, _ in STEMS:
            put(f"blk.{i}.{stem}.weight", *shapes[stem])
    put("token_embd.weight", c["vocab"], d)
    # the writer wants Q8_0 arrays of the right size for the tensors it is not given raw: all of them are raw here
    path = gguf_file.write_llama_gguf(tmp_path_factory.mktemp("native") / "native.gguf", sm, raw=raw)
    om = O.OracleLlama(sm, threads=4)
    for i in range(c["n_layer"]):
        for which, (stem, _) in enumerate(STEMS):
            om.set_f32(i, which, decoded[f"blk.{i}.{stem}.weight"])
    om.set_f32(0, 8, decoded["token_embd.weight"])
    om.set_f32(0, 7, decoded["token_embd.weight"])            # tied head: the embedding transposed
    gm = CudaLlama.from_gguf(path, prec="native")
    return c, om, gm


def test_forward_tokens_matches_the_f32_import(native):
    c, om, gm = native
    ids = synth.token_ids(1, 33, c["vocab"])
    want, got = om.forward_tokens(ids), gm.forward_tokens(ids)
    assert np.abs(got - want).max() < TOL * max(1.0, float(np.abs(want).max()))


def test_cached_decode_matches_the_f32_import(native):
    c, om, gm = native
    ids = synth.token_ids(2, 20, c["vocab"])
    full = gm.forward_tokens(ids)
    cache = gm.new_cache()
    om.clear()
    for t, tok in enumerate(ids):
        got, want = gm.forward_one(tok, cache), om.forward_one(tok)
        scale = max(1.0, float(np.abs(want).max()))
        assert np.abs(got - want).max() < TOL * scale, t
        assert np.abs(got - full[t]).max() < TOL * scale, t
    assert cache.pos() == ids.size


def test_scoring_and_generation(native):
    c, om, gm = native
    ids = synth.token_ids(3, 50, c["vocab"])
    total, n, greedy, lp, gr = om.score_from(ids, 1, 32)
    sc, glp, ggr = gm.score_from(ids, 1, 32, per_token=True)
    # random blocks give logits in the hundreds: the bound is relative to them (1e-3 absolute holds at the usual scale)
    assert sc.n_tokens == n and np.abs(glp - lp).max() < 1e-3 + 2e-5 * float(np.abs(lp).max())
    prompt = synth.token_ids(4, 9, c["vocab"])
    want = om.generate(prompt, 12, O.Rng(1), temperature=0.0)
    got, _ = gm.generate(prompt, 12, sampling(temperature=0.0))
    for i in range(min(len(got), len(want))):
        if got[i] != want[i]:
            om.clear()
            logits = None
            for t in list(prompt) + list(want[:i]):
                logits = om.forward_one(int(t))
            top = np.sort(logits)[-2:]
            assert top[1] - top[0] < 10 * TOL, f"token {i}: got {got[i]}, want {want[i]}, margin {top[1] - top[0]:.3e}"
            break


def test_rows_that_do_not_hold_whole_blocks_are_refused(tmp_path):
    sm = synth.llama_named("llama-tiny", perturb=True)        # rows of 64 values: no K-quant super-block fits
    c = sm.dims
    blocks = random_any(GD.Q4_K, c["vocab"] * c["d_model"], 5)
    path = gguf_file.write_llama_gguf(tmp_path / "bad.gguf", sm, raw={"token_embd.weight": (GD.Q4_K, blocks)})
    with pytest.raises(_lib.FerrumCudaError):
        CudaLlama.from_gguf(path, prec="native")
