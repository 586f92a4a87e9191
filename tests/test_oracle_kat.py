"""Pins the CPU oracle (and the library's host codecs) to the known-answer values held by
the reference's own unit tests. Each test names the reference test it restates. CPU only."""
import ctypes as C
import math

import numpy as np
import pytest

import ferrum_cpu_b200 as fcb
from ferrum_cpu_b200 import _lib, synth
from tests import oracle as O


def both_f16_decoders():
    return [("oracle", lambda h: O.lib().fo_f16_to_f32(h)), ("library", lambda h: _lib.lib().fc_f16_to_f32(h))]


def both_f16_encoders():
    return [("oracle", lambda v: O.lib().fo_f32_to_f16(v)), ("library", lambda v: _lib.lib().fc_f32_to_f16(v))]


# gguf/dequant.rs:527-538 f16_special_values
@pytest.mark.parametrize("name,dec", both_f16_decoders())
def test_f16_special_values(name, dec):
    assert dec(0x0000) == 0.0
    assert dec(0x8000) == 0.0 and math.copysign(1.0, dec(0x8000)) == -1.0
    assert dec(0x3C00) == 1.0
    assert dec(0x7C00) == math.inf and dec(0xFC00) == -math.inf
    assert math.isnan(dec(0x7E00))
    assert dec(0x0001) == 2.0 ** -24


@pytest.mark.parametrize("name,dec", both_f16_decoders())
def test_f16_decode_every_half_matches_ieee(name, dec):
    halves = np.arange(65536, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([dec(int(h)) for h in halves], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.all(np.isnan(got[~finite]))


# gguf_write/blocks.rs:12-61: RNE, overflow, subnormals, canonical NaN
@pytest.mark.parametrize("name,enc", both_f16_encoders())
def test_f32_to_f16_matches_ieee_rne(name, enc):
    rs = np.random.RandomState(1)
    bits = rs.randint(0, 2 ** 32, size=20000, dtype=np.uint64).astype(np.uint32)
    # concentrate half of the samples on the half range, subnormals and ties included
    mag = np.exp(rs.uniform(np.log(2.0 ** -27), np.log(70000.0), size=20000)).astype(np.float32)
    mag *= rs.choice([-1.0, 1.0], size=20000).astype(np.float32)
    ties = (np.arange(2048, dtype=np.float32) + 0.5) * np.float32(2.0 ** -24)   # subnormal ties
    ties2 = np.float32(1.0) + (np.arange(1024, dtype=np.float32) * 2 + 1) * np.float32(2.0 ** -11)
    vals = np.concatenate([bits.view(np.float32), mag, ties, ties2,
                           np.array([65504.0, 65519.9, 65520.0, 65536.0, 1e9, -1e9, 0.0, -0.0, 2.0 ** -25, 2.0 ** -24 * 1.5],
                                    dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    for v, w in zip(vals, want):
        got = enc(float(v))
        if math.isnan(float(v)):
            assert got & 0x7FFF == 0x7E00
        else:
            assert got == int(w), (float(v), hex(got), hex(int(w)))


def both_q8():
    return [("oracle", O.q8_0_encode, O.q8_0_decode), ("library", synth.q8_0_quantize, synth.q8_0_dequantize)]


def split(raw):
    raw = raw.reshape(-1, 34)
    d16 = raw[:, 0].astype(np.uint16) | (raw[:, 1].astype(np.uint16) << 8)
    return d16, raw[:, 2:].view(np.int8)


# quant.rs:332-343 q8_0_block_matches_llama_cpp_reference
@pytest.mark.parametrize("name,enc,dec", both_q8())
def test_q8_0_block_formula(name, enc, dec):
    x = ((np.arange(32, dtype=np.float32) - np.float32(15.5)) * np.float32(0.37)).astype(np.float32)
    d16, q = split(enc(x))
    amax = np.float32(np.abs(x).max())
    d = np.float32(amax / np.float32(127.0))
    assert d16[0] == O.lib().fo_f32_to_f16(float(d))
    inv = np.float32(1.0) / d
    want = np.array([math.floor(abs(float(v * inv)) + 0.5) * (1 if v >= 0 else -1) for v in x])
    assert np.array_equal(q[0].astype(np.float64), want)
    dz, qz = split(enc(np.zeros(32, dtype=np.float32)))
    assert dz[0] == 0 and not qz.any()


# quant.rs:357-365 rounds half away from zero, amax -> 127
@pytest.mark.parametrize("name,enc,dec", both_q8())
def test_q8_0_ties_away_and_amax(name, enc, dec):
    x = np.zeros(32, dtype=np.float32)
    x[:8] = [127.0, 0.5, 1.5, -0.5, -2.5, 2.4999, -126.5, 0.49]
    d16, q = split(enc(x))
    assert O.lib().fo_f16_to_f32(int(d16[0])) == 1.0
    assert q[0, :8].tolist() == [127, 1, 2, -1, -3, 2, -127, 0]
    assert not q[0, 8:].any()


# quant.rs:368-388 negative extreme / single outlier
@pytest.mark.parametrize("name,enc,dec", both_q8())
def test_q8_0_negative_extreme_and_outlier(name, enc, dec):
    neg = np.full(32, -0.01, dtype=np.float32)
    neg[7] = -3.0
    d16, q = split(enc(neg))
    assert q[0, 7] == -127 and (q[0] <= 0).all()
    d = O.lib().fo_f16_to_f32(int(d16[0]))
    assert abs(d - 3.0 / 127.0) < 3.0 / 127.0 * 1e-3
    pos = np.zeros(32, dtype=np.float32)
    pos[31] = 5.0
    _, q = split(enc(pos))
    assert q[0, 31] == 127 and not q[0, :31].any()


# quant.rs:391-401 zero block / sub-f16 block never NaN
@pytest.mark.parametrize("name,enc,dec", both_q8())
def test_q8_0_zero_and_underflow(name, enc, dec):
    tiny = np.full(32, 1e-30, dtype=np.float32)
    back = dec(enc(tiny), 32)
    assert np.isfinite(back).all() and (back == 0).all()


# quant.rs:404-422 + gguf_write/blocks.rs:279-300: 34-byte layout, blocks independent,
# decode == q * f16(d) exactly, snap is a fixed point (quant.rs:346-354)
@pytest.mark.parametrize("name,enc,dec", both_q8())
def test_q8_0_layout_decode_and_fixed_point(name, enc, dec):
    x = np.array([((i * 37 % 101) - 50.0) / 7.0 for i in range(128)], dtype=np.float32)
    x[32:64] = 0.0
    x[64:96] = -np.abs(x[64:96])
    x[100] = 900.0
    raw = enc(x)
    assert raw.size == 4 * 34
    assert raw[34] == 0 and raw[35] == 0
    d16, q = split(raw)
    back = dec(raw, 128)
    for b in range(4):
        d = np.float32(O.lib().fo_f16_to_f32(int(d16[b])))
        assert np.array_equal(back[b * 32:(b + 1) * 32], q[b].astype(np.float32) * d)
    assert np.array_equal(enc(back), raw), "re-encoding snapped values is idempotent"


def test_library_and_oracle_codecs_agree_bitwise():
    x = O.fill_normal(7, 32 * 4096, 0.02)
    assert np.array_equal(O.q8_0_encode(x), synth.q8_0_quantize(x))
    raw = O.q8_0_encode(x)
    assert np.array_equal(O.q8_0_decode(raw, x.size).view(np.uint32), synth.q8_0_dequantize(raw, x.size).view(np.uint32))


# rng.rs: determinism, remapped zero seed, unit interval, unit variance
def test_rng_streams_agree_and_are_standard_normal():
    a = O.fill_normal(0, 20000, 1.0)
    b = synth.Rng(0).normal(20000, 1.0)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert abs(float(a.mean())) < 0.05 and abs(float(a.std()) - 1.0) < 0.05
    assert O.lib().fo_rng_seed(0) == 0x9E3779B97F4A7C15 == _lib.lib().fc_rng_seed(0)
    st = C.c_uint64(1)
    x = 1
    x ^= (x << 13) & (2 ** 64 - 1); x ^= x >> 7; x ^= (x << 17) & (2 ** 64 - 1)
    assert O.lib().fo_rng_next_u64(C.byref(st)) == (x * 0x2545F4914F6CDD1D) % 2 ** 64
    assert np.array_equal(O.fill_ids(3, 1000, 4096), synth.token_ids(3, 1000, 4096))
    assert O.fill_ids(3, 1000, 4096).max() < 4096


# activation.rs:183-195 gelu_known_values, :169-180 saturation
def test_gelu_known_values():
    g = O.lib().fo_gelu
    for x, want in [(1.0, 0.8411919), (-1.0, -0.1588081), (0.5, 0.345714)]:
        assert abs(g(x) - want) < 2e-6
    assert g(0.0) == 0.0
    for x in [10.0, 12.5, 30.0, 1e4, 1e10, 1e20, 3e38]:
        assert g(x) == np.float32(x) and abs(g(-x)) == 0.0


# tests/tests/test_layer.rs:8-26 and ops.rs:591-596
def test_linear_and_matmul_known_answers():
    y = O.linear([[0.5, 1.5]], [[1, 2, 3], [4, 5, 6]], [0.1, 0.2, 0.3])
    assert np.allclose(y, [[6.6, 8.7, 10.8]], atol=1e-5)
    c = O.linear([[1, 2], [3, 4]], [[5, 6], [7, 8]], None)
    assert c.ravel().tolist() == [19.0, 22.0, 43.0, 50.0]


# ops.rs:538-579, 729-778: tiled / threaded engine == plain triple loop, bit for bit
@pytest.mark.parametrize("m,k,n", [(1, 7, 5), (3, 300, 17), (5, 257, 263), (9, 33, 520), (4, 256, 256), (13, 515, 40), (70, 64, 96)])
def test_engine_is_bit_identical_to_triple_loop(m, k, n):
    rs = np.random.RandomState(m * 1000 + k)
    x, w, b = rs.randn(m, k).astype(np.float32), rs.randn(k, n).astype(np.float32), rs.randn(n).astype(np.float32)
    want = O.linear(x, w, b, naive=True)
    for threads in (1, 2, 3, 4, 8):
        got = O.linear(x, w, b, threads=threads)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), threads


# layer/norm.rs:99-124
def test_layernorm_known_behaviour():
    y = O.layernorm([[1, 2, 3, 4], [10, -10, 20, -20]], [1] * 4, [0] * 4)
    for row in y:
        assert abs(row.mean()) < 1e-4 and abs(row.var() - 1.0) < 1e-3
    y = O.layernorm([[5.0] * 4], [2.0] * 4, [1.0] * 4)
    assert np.allclose(y, 1.0, atol=1e-3)


# sampling.rs:392-398
def test_argmax_first_ties():
    assert O.argmax_first([1.0]) == 0
    assert O.argmax_first([0.1, 2.0, 2.0, 1.0]) == 1
    assert O.argmax_first([3.0, 3.0, 3.0]) == 0
    assert O.argmax_first([-1.0, -0.5, -0.5]) == 1
    assert O.argmax_first([-np.inf, -np.inf]) == 0


def test_softmax_rows_sum_to_one():
    p = O.softmax_rows(np.random.RandomState(0).randn(5, 999) * 3)
    assert np.allclose(p.sum(axis=1), 1.0, atol=1e-5) and (p >= 0).all()


# ---- sampler (slm/sampling.rs tests, :215-470) ---------------------------------------------
def test_pick_by_mass_known_answers():
    # sampling.rs:452-468
    assert O.pick_by_mass([0.5, 0.4, 0.0, 0.0], 0.95) == 1
    assert O.pick_by_mass([0.0, 0.0, 0.0], 0.5) == 0
    assert O.pick_by_mass([0.2, 0.3, 0.5], 0.0) == 0
    assert O.pick_by_mass([0.2, 0.3, 0.5], 0.2) == 0
    assert O.pick_by_mass([0.2, 0.3, 0.5], 0.21) == 1
    assert O.pick_by_mass([0.2, 0.3, 0.5], 1.0) == 2
    assert O.pick_by_mass([0.0, 1.0], 0.0) == 1


def test_sampler_known_answers():
    # zero / negative temperature is argmax and draws nothing (sampling.rs:397-423)
    logits = [0.1, 2.0, 1.9, -1.0]
    for t in (0.0, -1.0):
        for s in range(20):
            assert O.sample_with_params(logits, O.Rng(s), temperature=t) == 1
    assert O.sample_with_params(logits, O.Rng(0), temperature=0.0, repetition_penalty=2.0, recent=[1]) == 2
    r, r2 = O.Rng(3), O.Rng(3)
    before = r.next_u64()
    O.sample_with_params(logits, r2, temperature=0.0)
    assert r2.next_u64() == before
    assert O.sample_with_params([1.0, 5.0, 5.0], O.Rng(1), temperature=0.0) == 1
    # out-of-vocabulary recent tokens are ignored (sampling.rs:219-231)
    lg = [0.5, -1.2, 2.3]
    assert O.sample_with_params(lg, O.Rng(1), temperature=0.0, repetition_penalty=1.5, recent=[99]) == \
        O.sample_with_params(lg, O.Rng(1), temperature=0.0, repetition_penalty=1.5)
    # top_p = 1 equals disabled (sampling.rs:249-264)
    lg = [0.5, -1.2, 2.3, 0.0, 1.1]
    a, b = O.Rng(5), O.Rng(5)
    for _ in range(100):
        assert O.sample_with_params(lg, a) == O.sample_with_params(lg, b, top_p=1.0)
    # top_k restricts the support (sampling.rs:297-317); top_p keeps the minimal set (:319-335)
    rng = O.Rng(7)
    for _ in range(500):
        assert O.sample_with_params([5.0, 4.0, -2.0, -3.0, -5.0], rng, top_k=2) in (0, 1)
    rng = O.Rng(3)
    for _ in range(500):
        assert O.sample_with_params([10.0, 1.0, 0.5, 0.0], rng, top_p=0.5) == 0
    # a heavy repetition penalty redirects the mass (sampling.rs:337-362)
    rng = O.Rng(11)
    ones = sum(O.sample_with_params([4.0, 3.0, -2.0], rng, repetition_penalty=100.0, recent=[0]) == 1 for _ in range(1000))
    assert ones > 800


def test_temperature_only_sampler_matches_the_legacy_formula():
    # sampling.rs:266-295: temperature softmax + one next_f32 draw + first index reaching r
    logits = np.array([0.5, -1.2, 2.3, 0.0, 1.1, -0.4], dtype=np.float32)
    temp = np.float32(0.8)
    r1, r2 = O.Rng(42), O.Rng(42)
    for _ in range(200):
        p = np.exp((logits - logits.max()) / temp).astype(np.float32)
        s = np.float32(0)
        for v in p:
            s = np.float32(s + v)
        p = (p / s).astype(np.float32)
        r = r1.next_f32()
        c, want = np.float32(0), len(p) - 1
        for i, v in enumerate(p):
            c = np.float32(c + v)
            if r <= c:
                want = i
                break
        assert O.sample_with_params(logits, r2, temperature=float(temp)) == want
