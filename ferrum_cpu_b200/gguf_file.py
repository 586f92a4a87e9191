"""Writes a synthetic model as a gpt2-, llama- or qwen2-architecture GGUF file (version 3).

The container follows the reference's builder (ferrum_core/src/gguf_write/builder.rs and
gguf/header.rs:9-66): magic, version, tensor count, metadata count, metadata key/value pairs,
tensor directory (name, dims with ne0 first, ggml type, offset), padding to general.alignment,
tensor data each padded to the alignment. Key and tensor names are those of
loader/gpt2.rs:100-160. Used by the tests of fc_model_load_gguf and by anyone who wants the
benchmark's synthetic weights as a file.
"""
import struct

import numpy as np

GGML_F32, GGML_Q4_0, GGML_Q5_0, GGML_Q8_0 = 0, 2, 6, 8
VT_U32, VT_F32, VT_STRING = 4, 6, 8


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def write_gpt2_gguf(path, sm, alignment=32, eps=1e-5, version=3, untied_head=None, row_order=None, extra_meta=()):
    """sm: synth.SynthModel. row_order: file row -> model id permutation of the token table (the
    file stores row r = model row row_order[r]), so that a loader needs the inverse to undo it."""
    L, d, H, F, T, V = sm.dims
    meta = [
        ("general.architecture", VT_STRING, "gpt2"),
        ("general.name", VT_STRING, "ferrum-synthetic"),
        ("general.alignment", VT_U32, alignment),
        ("gpt2.context_length", VT_U32, T),
        ("gpt2.embedding_length", VT_U32, d),
        ("gpt2.block_count", VT_U32, L),
        ("gpt2.feed_forward_length", VT_U32, F),
        ("gpt2.attention.head_count", VT_U32, H),
        ("gpt2.attention.layer_norm_epsilon", VT_F32, eps),
    ] + list(extra_meta)
    tensors = []          # (name, dims ne0-first, type, bytes)

    def q8(name, raw, n, k):
        tensors.append((name, (k, n), GGML_Q8_0, np.ascontiguousarray(raw, dtype=np.uint8).tobytes()))

    def f32(name, v, dims):
        tensors.append((name, dims, GGML_F32, np.ascontiguousarray(v, dtype=np.float32).tobytes()))

    tok = np.ascontiguousarray(sm.token_embd, dtype=np.uint8).reshape(V, d // 32 * 34)
    if row_order is not None:
        tok = tok[np.asarray(row_order)]
    q8("token_embd.weight", tok, V, d)
    f32("position_embd.weight", sm.position_embd, (d, T))
    for i, lw in enumerate(sm.layers):
        n = f"blk.{i}."
        f32(n + "attn_norm.weight", lw["ln1_g"], (d,))
        f32(n + "attn_norm.bias", lw["ln1_b"], (d,))
        q8(n + "attn_qkv.weight", lw["attn_qkv_q8"], 3 * d, d)
        f32(n + "attn_qkv.bias", lw["attn_qkv_b"], (3 * d,))
        q8(n + "attn_output.weight", lw["attn_out_q8"], d, d)
        f32(n + "attn_output.bias", lw["attn_out_b"], (d,))
        f32(n + "ffn_norm.weight", lw["ln2_g"], (d,))
        f32(n + "ffn_norm.bias", lw["ln2_b"], (d,))
        q8(n + "ffn_up.weight", lw["ffn_up_q8"], F, d)
        f32(n + "ffn_up.bias", lw["ffn_up_b"], (F,))
        q8(n + "ffn_down.weight", lw["ffn_down_q8"], d, F)
        f32(n + "ffn_down.bias", lw["ffn_down_b"], (d,))
    f32("output_norm.weight", sm.out_norm_g, (d,))
    f32("output_norm.bias", sm.out_norm_b, (d,))
    if untied_head is not None:
        q8("output.weight", untied_head, V, d)

    return _emit(path, meta, tensors, alignment, version)


def _emit(path, meta, tensors, alignment, version):
    out = bytearray()
    out += struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(meta))
    for key, vt, val in meta:
        out += _s(key) + struct.pack("<I", vt)
        if vt == VT_U32:
            out += struct.pack("<I", val)
        elif vt == VT_F32:
            out += struct.pack("<f", val)
        elif vt == VT_STRING:
            out += _s(val)
        else:
            raise ValueError(vt)
    offset = 0
    for name, dims, typ, data in tensors:
        out += _s(name) + struct.pack("<I", len(dims))
        for e in dims:
            out += struct.pack("<Q", e)
        out += struct.pack("<IQ", typ, offset)
        offset += (len(data) + alignment - 1) // alignment * alignment
    out += b"\0" * ((-len(out)) % alignment)
    for _, _, _, data in tensors:
        out += data + b"\0" * ((-len(data)) % alignment)
    with open(path, "wb") as fh:
        fh.write(out)
    return path


def write_llama_gguf(path, sm, arch="llama", alignment=32, version=3, extra_meta=(), extra_tensors=(), drop_meta=(), raw=None):
    """sm: synth.SynthLlama. Keys and tensor names as gguf/llama.rs:164-339 reads them. The file's
    architecture decides the rotation (qwen2: split halves), so write `arch` to match sm's rope_type.
    raw: {tensor name: (ggml type, bytes)} stores a matrix in another block format (Q4_0, Q5_0) instead
    of sm's Q8_0 bytes."""
    raw = raw or {}
    c = sm.dims
    V, d, L, H, KV, hd, F, ctx = (c[k] for k in ("vocab", "d_model", "n_layer", "n_head", "n_kv_head", "head_dim", "d_ff", "ctx"))
    cfg = sm.config
    meta = [
        ("general.architecture", VT_STRING, arch),
        ("general.alignment", VT_U32, alignment),
        (f"{arch}.context_length", VT_U32, ctx),
        (f"{arch}.embedding_length", VT_U32, d),
        (f"{arch}.block_count", VT_U32, L),
        (f"{arch}.feed_forward_length", VT_U32, F),
        (f"{arch}.attention.head_count", VT_U32, H),
        (f"{arch}.attention.head_count_kv", VT_U32, KV),
        (f"{arch}.attention.key_length", VT_U32, hd),
        (f"{arch}.rope.dimension_count", VT_U32, cfg.rope_dim),
        (f"{arch}.rope.freq_base", VT_F32, cfg.rope_base),
        (f"{arch}.attention.layer_norm_rms_epsilon", VT_F32, cfg.norm_eps),
    ]
    if cfg.rope_linear_factor != 1.0:
        meta += [(f"{arch}.rope.scaling.type", VT_STRING, "linear"), (f"{arch}.rope.scaling.factor", VT_F32, cfg.rope_linear_factor)]
    meta = [m for m in meta if m[0] not in drop_meta] + list(extra_meta)
    tensors = []

    def q8(name, data, n, k):
        typ, data = raw.get(name, (GGML_Q8_0, data))
        tensors.append((name, (k, n), typ, np.ascontiguousarray(data, dtype=np.uint8).tobytes()))

    def f32(name, v, dims):
        tensors.append((name, dims, GGML_F32, np.ascontiguousarray(v, dtype=np.float32).tobytes()))

    q8("token_embd.weight", sm.token_embd, V, d)
    if sm.freq_factors is not None:
        f32("rope_freqs.weight", sm.freq_factors, (cfg.rope_dim // 2,))
    qd, kvd = H * hd, KV * hd
    for i, lw in enumerate(sm.layers):
        n = f"blk.{i}."
        f32(n + "attn_norm.weight", lw["attn_norm"], (d,))
        q8(n + "attn_q.weight", lw["wq_q8"], qd, d)
        q8(n + "attn_k.weight", lw["wk_q8"], kvd, d)
        q8(n + "attn_v.weight", lw["wv_q8"], kvd, d)
        q8(n + "attn_output.weight", lw["wo_q8"], d, qd)
        for s_, w_ in (("q", qd), ("k", kvd), ("v", kvd)):
            if "b" + s_ in lw:
                f32(n + f"attn_{s_}.bias", lw["b" + s_], (w_,))
        f32(n + "ffn_norm.weight", lw["ffn_norm"], (d,))
        q8(n + "ffn_gate.weight", lw["gate_q8"], F, d)
        q8(n + "ffn_up.weight", lw["up_q8"], F, d)
        q8(n + "ffn_down.weight", lw["down_q8"], d, F)
    f32("output_norm.weight", sm.output_norm, (d,))
    if sm.output is not None:
        q8("output.weight", sm.output, V, d)
    for name, v, dims in extra_tensors:
        f32(name, v, dims)
    return _emit(path, meta, tensors, alignment, version)
