"""fc_gguf_probe / fc_model_load_gguf: the direct GGUF path (no f32 expansion of the matrices).
Container and names as gguf/header.rs:9-66 and loader/gpt2.rs:201-262."""
import os
import struct
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import ferrum_cpu_b200 as fcb  # noqa: E402
from ferrum_cpu_b200 import gguf_file, synth  # noqa: E402
from ferrum_cpu_b200._lib import FC_E_DIM, FC_E_FORMAT  # noqa: E402
from ferrum_cpu_b200.engine import gguf_probe  # noqa: E402


@pytest.fixture(scope="module")
def model_and_file(tmp_path_factory):
    sm = synth.SynthModel(2, 64, 2, 128, 32, 96, seed=7, perturb=True)
    path = tmp_path_factory.mktemp("gguf") / "m.gguf"
    gguf_file.write_gpt2_gguf(str(path), sm)
    return sm, str(path)


def test_probe_reads_the_dimensions(model_and_file):
    sm, path = model_and_file
    cfg = gguf_probe(path)
    assert (cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.ctx, cfg.vocab) == sm.dims
    assert cfg.tied == 1
    # a non-default alignment moves the data section (header.rs:60-64)
    p64 = path + ".a64"
    gguf_file.write_gpt2_gguf(p64, sm, alignment=64)
    assert gguf_probe(p64).vocab == 96
    # version 2 is accepted, an untied head is seen
    p2 = path + ".v2"
    gguf_file.write_gpt2_gguf(p2, sm, version=2, untied_head=sm.token_embd)
    assert gguf_probe(p2).tied == 0
    # a row permutation sets the vocabulary size
    assert gguf_probe(path, row_perm=np.arange(90)).vocab == 90


def _expect(code, fn):
    with pytest.raises(fcb.FerrumCudaError) as e:
        fn()
    assert e.value.code == code, str(e.value)
    return str(e.value)


def test_probe_rejects_what_the_reference_rejects(model_and_file, tmp_path):
    sm, path = model_and_file
    raw = bytearray(open(path, "rb").read())
    bad = tmp_path / "bad.gguf"

    def variant(mutate):
        b = bytearray(raw)
        mutate(b)
        bad.write_bytes(bytes(b))
        return str(bad)

    assert "magic" in _expect(FC_E_FORMAT, lambda: gguf_probe(variant(lambda b: b.__setitem__(0, 0x00))))
    assert "version" in _expect(FC_E_FORMAT, lambda: gguf_probe(variant(lambda b: b.__setitem__(slice(4, 8), struct.pack("<I", 7)))))
    _expect(FC_E_FORMAT, lambda: gguf_probe(variant(lambda b: b.__delitem__(slice(200, len(b))))))       # truncated directory
    _expect(FC_E_FORMAT, lambda: gguf_probe(variant(lambda b: b.__delitem__(slice(len(b) - 64, len(b))))))  # tensor past the end
    _expect(FC_E_FORMAT, lambda: gguf_probe(str(tmp_path / "missing.gguf")))
    # layer_norm_epsilon other than 1e-5 (gpt2.rs:209-215)
    p = str(tmp_path / "eps.gguf")
    gguf_file.write_gpt2_gguf(p, sm, eps=1e-6)
    assert "epsilon" in _expect(FC_E_FORMAT, lambda: gguf_probe(p))
    # a permutation entry outside the file's rows
    _expect(FC_E_DIM, lambda: gguf_probe(path, row_perm=np.array([0, 1, 500])))
    # a matrix stored as F32 instead of Q8_0
    sm2 = synth.SynthModel(1, 32, 1, 64, 8, 40, seed=1)
    p = str(tmp_path / "f32mat.gguf")
    gguf_file.write_gpt2_gguf(p, sm2)
    b = bytearray(open(p, "rb").read())
    name = b"blk.0.ffn_up.weight"
    at = b.index(name) + len(name) + 4 + 16      # name, n_dims, two u64 dims -> the type field
    assert struct.unpack_from("<I", b, at)[0] == 8
    struct.pack_into("<I", b, at, 0)
    open(p, "wb").write(bytes(b))
    assert "ffn_up" in _expect(FC_E_FORMAT, lambda: gguf_probe(p))
    # crafted directory entries: an offset near 2^64 (must not wrap the bounds check), an offset off
    # the file's alignment, and a tensor name that appears twice
    gguf_file.write_gpt2_gguf(p, sm2)
    good = bytearray(open(p, "rb").read())
    name = b"blk.0.ffn_up.weight"
    at = good.index(name) + len(name) + 4 + 16 + 4      # name, n_dims, two u64 dims, type -> the offset field
    real = struct.unpack_from("<Q", good, at)[0]
    for off, word in ((0xFFFFFFFFFFFFFFE0, "past the end"), (real + 16, "alignment")):
        b = bytearray(good)
        struct.pack_into("<Q", b, at, off)
        open(p, "wb").write(bytes(b))
        assert word in _expect(FC_E_FORMAT, lambda: gguf_probe(p))
    b = bytearray(good)
    old, dup = b"blk.0.ffn_down.bias", b"blk.0.attn_qkv.bias"
    assert len(old) == len(dup)
    k = b.index(old)
    b[k:k + len(old)] = dup
    open(p, "wb").write(bytes(b))
    assert "twice" in _expect(FC_E_FORMAT, lambda: gguf_probe(p))


@pytest.mark.gpu
def test_model_from_gguf_equals_model_from_arrays(model_and_file, tmp_path):
    sm, path = model_and_file
    a = fcb.CudaSlm(sm.config, sm.weights)
    b = fcb.CudaSlm.from_gguf(path)
    ids = synth.token_ids(5, 30, 96)
    sa, lpa, _ = a.token_logprobs(ids, per_token=True)
    sb, lpb, _ = b.token_logprobs(ids, per_token=True)
    assert np.array_equal(lpa, lpb) and sa.logprob == sb.logprob
    ta, _ = a.generate_tokens(ids[:9], 12)
    tb, _ = b.generate_tokens(ids[:9], 12)
    assert np.array_equal(ta, tb)
    # the file stores the token rows in another order; the loader's row_perm undoes it
    order = np.random.default_rng(3).permutation(96)        # file row r holds model row order[r]
    p2 = str(tmp_path / "perm.gguf")
    gguf_file.write_gpt2_gguf(p2, sm, row_order=order)
    perm = np.argsort(order)                                 # perm[model id] = file row
    c = fcb.CudaSlm.from_gguf(p2, row_perm=perm)
    sc, lpc, _ = c.token_logprobs(ids, per_token=True)
    assert np.array_equal(lpa, lpc)
    for m in (a, b, c):
        m.close()
