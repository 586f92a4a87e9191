"""Q4_0 and Q5_0 blocks re-blocked exactly to Q8_0 (fc_ggml_to_q8_0): the oracle's decoders on the
reference's known-answer block, the codec against the oracle bit for bit, and a llama GGUF file that
stores its projections in those formats against the model built from the re-blocked arrays."""
import ctypes as C
import struct

import numpy as np
import pytest

from ferrum_cpu_b200 import _lib, gguf_file, llama, synth
from tests import oracle as O

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
