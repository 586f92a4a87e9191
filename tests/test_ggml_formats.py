"""GGML block formats at the import boundary. Q4_0 and Q5_0 blocks re-blocked exactly to Q8_0 (fc_ggml_to_q8_0): the
oracle's decoders on the reference's known-answer block, the codec against the oracle bit for bit, and a llama GGUF file
that stores its projections in those formats against the model built from the re-blocked arrays. Every other format
the reference's importer reads (Q4_1, Q5_1, Q8_1, Q2_K .. Q6_K, f16, f32): the numpy restatement of the reference's
decoders (oracle/gguf_dequant.py) on the reference's own known-answer blocks (gguf/dequant.rs:337-547), the library's
decoders against it bit for bit on random blocks, and the decode-and-re-encode import route."""
import ctypes as C
import struct

import numpy as np
import pytest

import importlib.util
import os

from ferrum_cpu_b200 import _lib, gguf_file, llama, synth
from tests import oracle as O

_spec = importlib.util.spec_from_file_location(
    "gguf_dequant", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "oracle", "gguf_dequant.py"))
GD = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(GD)

Q4_0, Q5_0, Q8_0 = 2, 6, 8


def random_blocks(ggml_type, n, seed):
    """n values of valid blocks: f16 scales around 0.02 / 8, every nibble / high-bit pattern."""
    rng = np.random.default_rng(seed)
    bb = {Q4_0: 18, Q5_0: 22}[ggml_type]
    out = rng.integers(0, 256, size=(n // 32, bb), dtype=np.uint8)
    scales = (rng.standard_normal(n // 32) * 0.0025).astype(np.float16)
    out[:, :2] = scales.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def to_q8_0(ggml_type, raw, n):
    out = np.empty(n // 32 * 34, dtype=np.uint8)
    rc = _lib.lib().fc_ggml_to_q8_0(ggml_type, raw.ctypes.data_as(C.c_void_p), n, out.ctypes.data_as(C.c_void_p))
    assert rc == _lib.FC_OK
    return out


def test_q5_0_known_answer_block():
    # gguf/dequant.rs:371-393: qh bit j is the fifth bit of element j, bit j + 16 of element j + 16
    raw = np.frombuffer(np.float16(2.0).tobytes() + struct.pack("<I", (1 << 0) | (1 << 17)) + bytes([0x21] * 16), dtype=np.uint8)
    out = O.dequant_ggml(Q5_0, raw, 32)
    assert out[0] == 2.0 * (17 - 16) and out[1] == 2.0 * (1 - 16) and out[17] == 2.0 * (18 - 16) and out[16] == 2.0 * (2 - 16)
    L = _lib.lib()
    assert (L.fc_ggml_block_bytes(Q4_0), L.fc_ggml_block_bytes(Q5_0), L.fc_ggml_block_bytes(Q8_0)) == (18, 22, 34)
    assert L.fc_ggml_block_bytes(3) == 0 and L.fc_ggml_block_bytes(12) == 0                  # Q4_1, Q4_K: not integer-level formats


def test_q4_0_layout():
    # gguf/dequant.rs:73-80: low nibble -> element j, high nibble -> element j + 16, centred at 8
    raw = np.frombuffer(np.float16(0.5).tobytes() + bytes((j | ((15 - j) << 4)) for j in range(16)), dtype=np.uint8)
    out = O.dequant_ggml(Q4_0, raw, 32)
    assert np.array_equal(out[:16], 0.5 * (np.arange(16) - 8)) and np.array_equal(out[16:], 0.5 * (15 - np.arange(16) - 8))


@pytest.mark.parametrize("ggml_type", [Q4_0, Q5_0])
def test_reblocking_is_exact(ggml_type):
    n = 32 * 257
    raw = random_blocks(ggml_type, n, 3)
    got = synth.q8_0_dequantize(to_q8_0(ggml_type, raw, n), n)
    want = O.dequant_ggml(ggml_type, raw, n)
    assert got.tobytes() == want.tobytes()
    assert O.q8_0_decode(to_q8_0(ggml_type, raw, n), n).tobytes() == want.tobytes()
    bad = np.empty(34, np.uint8)
    assert _lib.lib().fc_ggml_to_q8_0(3, raw.ctypes.data_as(C.c_void_p), 32, bad.ctypes.data_as(C.c_void_p)) == _lib.FC_E_FORMAT
    assert _lib.lib().fc_ggml_to_q8_0(ggml_type, raw.ctypes.data_as(C.c_void_p), 48, bad.ctypes.data_as(C.c_void_p)) == _lib.FC_E_FORMAT


def mixed_format_model(tmp_path):
    """A tiny Llama whose projections alternate between Q4_0 and Q5_0 in the file; sm holds the re-blocked Q8_0."""
    sm = synth.llama_named("llama-tiny", perturb=True, seed=2)
    c = sm.dims
    d, F, qd, kvd = c["d_model"], c["d_ff"], c["n_head"] * c["head_dim"], c["n_kv_head"] * c["head_dim"]
    shapes = dict(wq_q8=("attn_q", qd, d), wk_q8=("attn_k", kvd, d), wv_q8=("attn_v", kvd, d), wo_q8=("attn_output", d, qd),
                  gate_q8=("ffn_gate", F, d), up_q8=("ffn_up", F, d), down_q8=("ffn_down", d, F))
    raw, seed = {}, 10
    for i, lw in enumerate(sm.layers):
        for key, (stem, n, k) in shapes.items():
            typ = Q4_0 if seed % 2 else Q5_0
            blocks = random_blocks(typ, n * k, seed)
            lw[key][:] = to_q8_0(typ, blocks, n * k)             # the arrays the model-from-arrays reads
            raw[f"blk.{i}.{stem}.weight"] = (typ, blocks)
            seed += 1
    tok = random_blocks(Q4_0, c["vocab"] * d, 99)
    sm.token_embd[:] = to_q8_0(Q4_0, tok, c["vocab"] * d)
    raw["token_embd.weight"] = (Q4_0, tok)
    return sm, gguf_file.write_llama_gguf(tmp_path / "mixed.gguf", sm, raw=raw)


def test_probe_accepts_q4_0_and_q5_0_files(tmp_path):
    sm, path = mixed_format_model(tmp_path)
    cfg = llama.gguf_probe(path)
    assert cfg.vocab == sm.dims["vocab"] and cfg.n_layer == sm.dims["n_layer"]


@pytest.mark.gpu
def test_model_from_q4_q5_file_equals_model_from_reblocked_arrays(tmp_path):
    sm, path = mixed_format_model(tmp_path)
    a, b = llama.CudaLlama.from_synth(sm), llama.CudaLlama.from_gguf(path)
    ids = synth.token_ids(5, 40, sm.dims["vocab"])
    la, lb = a.forward_tokens(ids), b.forward_tokens(ids)
    assert np.array_equal(la, lb)
    want = O.OracleLlama(sm, threads=2).forward_tokens(ids)      # and both are the reference's values on those weights
    assert np.abs(la - want).max() < 2e-4 * max(1.0, float(np.abs(want).max()))
    a.close()
    b.close()


# ---- every block format of the reference's importer ------------------------------------------------------------
def half(v):
    return np.float16(v).tobytes()


def lib_dequant(t, raw, n):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    rc = _lib.lib().fc_ggml_dequantize(t, raw.ctypes.data_as(C.c_void_p), raw.size, n, out.ctypes.data_as(C.c_void_p))
    return rc, out


def both(t, raw, n):
    """The oracle's values, after checking that the library's are the same bits."""
    raw = np.frombuffer(bytes(raw), dtype=np.uint8)
    want = GD.dequantize(t, raw, n)
    rc, got = lib_dequant(t, raw, n)
    assert rc == _lib.FC_OK and got.tobytes() == want.tobytes()
    return want


K_SCALES_D2_M0 = bytes([2, 2, 2, 2, 0, 0, 0, 0, 2, 2, 2, 2])   # every sub-block: scale 2, minimum 0 (dequant.rs:482-490)


def test_known_answer_blocks_of_the_reference():
    # dequant.rs:337-350 Q8_1: d = 0.5, levels -16 .. 15, the block sum is ignored
    out = both(GD.Q8_1, half(0.5) + half(0.0) + bytes((i - 16) & 0xFF for i in range(32)), 32)
    assert np.array_equal(out, 0.5 * (np.arange(32) - 16))
    # dequant.rs:352-369 Q4_1: d * nibble + m
    los, his = [j % 15 for j in range(16)], [(j + 3) % 15 for j in range(16)]
    out = both(GD.Q4_1, half(0.25) + half(1.0) + bytes((his[j] << 4) | los[j] for j in range(16)), 32)
    assert np.array_equal(out[:16], 0.25 * np.array(los) + 1.0) and np.array_equal(out[16:], 0.25 * np.array(his) + 1.0)
    # dequant.rs:371-393 Q5_0 / Q5_1: bit j of qh is the fifth bit of element j, bit j + 16 of element j + 16
    qh = struct.pack("<I", (1 << 0) | (1 << 17))
    q50 = both(GD.Q5_0, half(2.0) + qh + bytes([0x21] * 16), 32)
    assert (q50[0], q50[1], q50[17], q50[16]) == (2.0 * 1, 2.0 * -15, 2.0 * 2, 2.0 * -14)
    q51 = both(GD.Q5_1, half(2.0) + half(0.5) + qh + bytes([0x21] * 16), 32)
    assert (q51[0], q51[17]) == (2.0 * 17 + 0.5, 2.0 * 18 + 0.5)
    # dequant.rs:410-430 Q2_K: every 2-bit value 1, scales i | (15 - i) << 4, d 1, dmin 0.5 -> group g: g - 0.5 (15 - g)
    out = both(GD.Q2_K, bytes(i | ((15 - i) << 4) for i in range(16)) + bytes([0x55] * 64) + half(1.0) + half(0.5), 256)
    assert np.array_equal(out.reshape(16, 16), np.repeat((np.arange(16) - 0.5 * (15 - np.arange(16)))[:, None], 16, 1))
    # dequant.rs:432-463 Q3_K: low bits 1, all scales 34 (-> 2), d 1: high bit set -> 2, clear -> (1 - 4) * 2 = -6
    body = bytes([0x55] * 64) + bytes([0x22] * 8) + bytes([0xAA] * 4) + half(1.0)
    assert np.all(both(GD.Q3_K, bytes([0xFF] * 32) + body, 256) == 2.0)
    assert np.all(both(GD.Q3_K, bytes([0x00] * 32) + body, 256) == -6.0)
    # dequant.rs:465-480 Q6_K: nibbles 8, 2-bit fields 2 -> 40 - 32 = 8; scales 2, d 0.5 -> 8.0
    assert np.all(both(GD.Q6_K, bytes([0x88] * 128) + bytes([0xAA] * 64) + bytes([2] * 16) + half(0.5), 256) == 8.0)
    # dequant.rs:484-490 the packed 6-bit pairs
    assert all(GD.scale_min_k4(j, K_SCALES_D2_M0) == (2, 0) for j in range(8))
    # dequant.rs:492-503 Q4_K: d * sc = 1, minimum 0, nibbles 3 -> 3.0
    assert np.all(both(GD.Q4_K, half(0.5) + half(0.0) + K_SCALES_D2_M0 + bytes([0x33] * 128), 256) == 3.0)
    # dequant.rs:506-524 Q5_K: without and with every high bit -> 3.0 and 19.0
    for qhb, want in ((0x00, 3.0), (0xFF, 19.0)):
        assert np.all(both(GD.Q5_K, half(0.5) + half(0.0) + K_SCALES_D2_M0 + bytes([qhb] * 32) + bytes([0x33] * 128), 256) == want)


def test_sizes_and_short_data():
    L = _lib.lib()
    # gguf/format.rs:107-130, dequant.rs:395-408, :388-390
    sizes = {GD.Q5_0: (64, 44), GD.Q5_1: (64, 48), GD.Q4_K: (256, 144), GD.Q5_K: (256, 176), GD.Q6_K: (256, 210),
             GD.Q2_K: (256, 84), GD.Q3_K: (256, 110), GD.Q8_1: (32, 36), GD.Q4_1: (32, 20), GD.F16: (3, 6), GD.F32: (3, 12)}
    for t, (n, nbytes) in sizes.items():
        assert L.fc_ggml_type_bytes(t, n) == nbytes == GD.type_nbytes(t, n)
    for t, n in ((GD.Q5_0, 30), (GD.Q4_K, 200), (GD.Q2_K, 200), (15, 256), (4, 32)):
        assert L.fc_ggml_type_bytes(t, n) == 0 and GD.type_nbytes(t, n) is None
    # dequant.rs:540-547: one block holds 256 values; asking for more than the data holds is refused
    for t, bb in ((GD.Q2_K, 84), (GD.Q3_K, 110), (GD.Q4_K, 144)):
        assert lib_dequant(t, np.zeros(bb, np.uint8), 256)[0] == _lib.FC_OK
        assert lib_dequant(t, np.zeros(bb, np.uint8), 257)[0] == _lib.FC_E_FORMAT
        assert lib_dequant(t, np.zeros(bb, np.uint8), 512)[0] == _lib.FC_E_FORMAT
        with pytest.raises(ValueError):
            GD.dequantize(t, np.zeros(bb, np.uint8), 512)


def random_any(t, n, seed):
    """n values of random blocks of type t with finite f16 scales / minima."""
    rng = np.random.default_rng(seed)
    vals, bb = GD.BLOCK[t]
    if t == GD.F32:
        return rng.standard_normal(n).astype(np.float32).view(np.uint8)
    if t == GD.F16:
        return rng.standard_normal(n).astype(np.float16).view(np.uint8)
    raw = rng.integers(0, 256, size=(n // vals, bb), dtype=np.uint8)
    halves = {GD.Q4_0: [0], GD.Q5_0: [0], GD.Q8_0: [0], GD.Q4_1: [0, 2], GD.Q5_1: [0, 2], GD.Q8_1: [0, 2], GD.Q4_K: [0, 2],
              GD.Q5_K: [0, 2], GD.Q6_K: [208], GD.Q2_K: [80, 82], GD.Q3_K: [108]}[t]
    for at in halves:
        raw[:, at:at + 2] = (rng.standard_normal(n // vals) * 0.01).astype(np.float16).view(np.uint8).reshape(-1, 2)
    return raw.reshape(-1)


@pytest.mark.parametrize("t", sorted(GD.BLOCK))
def test_library_decoders_equal_the_oracle_bit_for_bit(t):
    n = GD.BLOCK[t][0] * 5 if GD.BLOCK[t][0] > 1 else 96
    raw = random_any(t, n, 40 + t)
    rc, got = lib_dequant(t, raw, n)
    assert rc == _lib.FC_OK
    assert got.tobytes() == GD.dequantize(t, raw, n).tobytes()


@pytest.mark.parametrize("t", sorted(GD.BLOCK))
def test_import_route_to_q8_0(t):
    """Exact where the format is an f16 scale times an integer; otherwise the decoded values through the Q8_0 block
    encoder (quant.rs:271-280), whose error is at most half a level of each block's own scale plus the rounding of
    that scale to f16 (2^-11 of up to 127 levels)."""
    n = 512
    raw = random_any(t, n, 70 + t)
    out = np.empty(n // 32 * 34, dtype=np.uint8)
    rc = _lib.lib().fc_ggml_requantize_q8_0(t, raw.ctypes.data_as(C.c_void_p), raw.size, n, out.ctypes.data_as(C.c_void_p))
    assert rc == _lib.FC_OK
    vals = GD.dequantize(t, raw, n)
    back = synth.q8_0_dequantize(out, n)
    if t in (GD.Q4_0, GD.Q5_0, GD.Q8_0):
        assert back.tobytes() == vals.tobytes()
    else:
        assert out.tobytes() == synth.q8_0_quantize(vals).tobytes()
        amax = np.abs(vals.reshape(-1, 32)).max(axis=1, keepdims=True)
        assert np.all(np.abs(back.reshape(-1, 32) - vals.reshape(-1, 32)) <= amax / 127.0 * (0.5 + 127.0 / 2048.0) * 1.002 + 1e-12)
    short = _lib.lib().fc_ggml_requantize_q8_0(t, raw.ctypes.data_as(C.c_void_p), raw.size - 1, n, out.ctypes.data_as(C.c_void_p))
    assert short == _lib.FC_E_FORMAT


def k_quant_model(tmp_path):
    """A tiny Llama whose matrices sit in the file as Q4_K, Q6_K, Q5_K, Q4_1 and f16; sm holds what the import route
    makes of them."""
    # rows of 256 and 512 values: whole super-blocks along every row, as ggml requires of K-quant tensors
    sm = synth.SynthLlama(384, 256, 2, 4, 2, 64, 512, 64, perturb=True, seed=3)
    c = sm.dims
    d, F, qd, kvd = c["d_model"], c["d_ff"], c["n_head"] * c["head_dim"], c["n_kv_head"] * c["head_dim"]
    shapes = dict(wq_q8=("attn_q", qd, d), wk_q8=("attn_k", kvd, d), wv_q8=("attn_v", kvd, d), wo_q8=("attn_output", d, qd),
                  gate_q8=("ffn_gate", F, d), up_q8=("ffn_up", F, d), down_q8=("ffn_down", d, F))
    kinds = [GD.Q4_K, GD.Q6_K, GD.Q5_K, GD.Q4_1, GD.F16, GD.Q2_K, GD.Q3_K, GD.Q5_1]
    raw, seed = {}, 20

    def put(name, dst, n_vals):
        nonlocal seed
        t = kinds[seed % len(kinds)]
        if n_vals % GD.BLOCK[t][0]:
            t = GD.Q4_1
        blocks = random_any(t, n_vals, seed)
        out = np.empty(n_vals // 32 * 34, dtype=np.uint8)
        rc = _lib.lib().fc_ggml_requantize_q8_0(t, blocks.ctypes.data_as(C.c_void_p), blocks.size, n_vals, out.ctypes.data_as(C.c_void_p))
        assert rc == _lib.FC_OK
        dst[:] = out
        raw[name] = (t, blocks)
        seed += 1

    for i, lw in enumerate(sm.layers):
        for key, (stem, n, k) in shapes.items():
            put(f"blk.{i}.{stem}.weight", lw[key], n * k)
    put("token_embd.weight", sm.token_embd, c["vocab"] * d)
    return sm, gguf_file.write_llama_gguf(tmp_path / "kquant.gguf", sm, raw=raw)


def test_probe_accepts_k_quant_files(tmp_path):
    sm, path = k_quant_model(tmp_path)
    cfg = llama.gguf_probe(path)
    assert cfg.vocab == sm.dims["vocab"] and cfg.n_layer == sm.dims["n_layer"]


@pytest.mark.gpu
def test_model_from_k_quant_file_equals_model_from_imported_arrays(tmp_path):
    sm, path = k_quant_model(tmp_path)
    a, b = llama.CudaLlama.from_synth(sm), llama.CudaLlama.from_gguf(path)
    ids = synth.token_ids(6, 40, sm.dims["vocab"])
    la, lb = a.forward_tokens(ids), b.forward_tokens(ids)
    assert np.array_equal(la, lb)
    want = O.OracleLlama(sm, threads=2).forward_tokens(ids)
    assert np.abs(la - want).max() < 2e-4 * max(1.0, float(np.abs(want).max()))
    a.close()
    b.close()
