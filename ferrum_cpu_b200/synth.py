"""Seeded synthetic GPT-2-shaped Q8_0 models and token ids.

Weights are drawn N(0, 0.02^2) with Ferrum's xorshift64* + Box-Muller generator
(ferrum_core/src/rng.rs:29-48, train_transformer/param.rs:24-28) through the library's host
codec, then every matrix is encoded to GGML Q8_0 along its input dimension
(quant.rs:271-280). LayerNorm gain 1 / bias 0 and zero linear biases unless `perturb` is
set, which draws small non-trivial values for them so that tests exercise those terms.
"""
import ctypes as C

import numpy as np

from . import _lib

# name -> (n_layer, d_model, n_head, d_ff, ctx, vocab)
SHAPES = {
    "tiny": (4, 128, 4, 512, 128, 4096),
    "small": (12, 768, 12, 3072, 1024, 50257),
    "medium": (24, 1024, 16, 4096, 1024, 50257),
}


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class Rng:
    """Ferrum's xorshift64* stream (rng.rs)."""

    def __init__(self, seed):
        self.state = C.c_uint64(_lib.lib().fc_rng_seed(seed))

    def normal(self, n, scale):
        out = np.empty(n, dtype=np.float32)
        _lib.lib().fc_rng_fill_normal(C.byref(self.state), scale, n, _ptr(out))
        return out

    def ids(self, n, vocab):
        out = np.empty(n, dtype=np.int32)
        _lib.lib().fc_rng_fill_ids(C.byref(self.state), vocab, n, _ptr(out))
        return out


def q8_0_quantize(x):
    """f32 array (size % 32 == 0) -> uint8 array of 34-byte GGML Q8_0 blocks."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    _lib.check(_lib.lib().fc_q8_0_quantize(_ptr(x), x.size, _ptr(out)))
    return out


def q8_0_dequantize(raw, n):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    _lib.check(_lib.lib().fc_q8_0_dequantize(_ptr(raw), n, _ptr(out)))
    return out


class SynthModel:
    """Host tensors of one model in GGUF order plus the fc_config / fc_weights structs."""

    def __init__(self, n_layer, d_model, n_head, d_ff, ctx, vocab, seed=0, perturb=False, math_mode=0):
        self.dims = (n_layer, d_model, n_head, d_ff, ctx, vocab)
        rng = Rng(seed)
        d, F, V, T = d_model, d_ff, vocab, ctx
        self.keep = []

        def mat(n, k):
            q = q8_0_quantize(rng.normal(n * k, 0.02))
            self.keep.append(q)
            return q

        def vec(n, base, scale):
            v = np.full(n, base, dtype=np.float32)
            if perturb:
                v = v + rng.normal(n, scale)
            v = np.ascontiguousarray(v, dtype=np.float32)
            self.keep.append(v)
            return v

        self.token_embd = mat(V, d)
        self.position_embd = rng.normal(T * d, 0.02)
        self.layers = []
        for _ in range(n_layer):
            L = dict(
                attn_qkv_q8=mat(3 * d, d), attn_out_q8=mat(d, d), ffn_up_q8=mat(F, d), ffn_down_q8=mat(d, F),
                attn_qkv_b=vec(3 * d, 0.0, 0.02), attn_out_b=vec(d, 0.0, 0.02),
                ffn_up_b=vec(F, 0.0, 0.02), ffn_down_b=vec(d, 0.0, 0.02),
                ln1_g=vec(d, 1.0, 0.1), ln1_b=vec(d, 0.0, 0.05), ln2_g=vec(d, 1.0, 0.1), ln2_b=vec(d, 0.0, 0.05))
            self.layers.append(L)
        self.out_norm_g = vec(d, 1.0, 0.1)
        self.out_norm_b = vec(d, 0.0, 0.05)

        self.config = _lib.FcConfig(n_layer, d_model, n_head, d_ff, ctx, vocab, 1, math_mode)
        self._layer_structs = (_lib.FcLayerWeights * n_layer)()
        for i, L in enumerate(self.layers):
            for k, v in L.items():
                setattr(self._layer_structs[i], k, v.ctypes.data)
        self.weights = _lib.FcWeights(
            self.token_embd.ctypes.data, self.position_embd.ctypes.data,
            C.cast(self._layer_structs, C.POINTER(_lib.FcLayerWeights)),
            self.out_norm_g.ctypes.data, self.out_norm_b.ctypes.data, None)

    @property
    def q8_weight_bytes(self):
        """Bytes of Q8_0 matrices one decoded token streams (each matrix once, tied head included)."""
        n_layer, d, _, F, _, V = self.dims
        return (n_layer * (4 * d * d + 2 * d * F) + d * V) * 34 // 32


# name -> (vocab, d_model, n_layer, n_head, n_kv_head, head_dim, d_ff, ctx)
LLAMA_SHAPES = {
    "llama-tiny": (512, 64, 2, 4, 2, 16, 128, 64),
    "llama-mini": (4096, 256, 4, 8, 2, 32, 704, 256),
    # heads of 64 (the width the tensor-core window attention takes), two query heads per key/value head
    "llama-hd64": (1024, 256, 2, 4, 2, 64, 512, 320),
    # widths that are no powers of two, seven query heads on one key/value head (the proportions of a small Qwen2)
    "qwen-odd": (1536, 448, 2, 7, 1, 64, 1216, 160),
    # the shape of a 1B-class GGUF (Llama-3.2-1B: 16 layers, 32 query / 8 key-value heads of 64)
    "llama-1b": (32000, 2048, 16, 32, 8, 64, 8192, 2048),
    # the same depth and head layout at a quarter of the width: what a step costs when the weights are small
    "llama-narrow": (32000, 512, 16, 8, 2, 64, 2048, 2048),
}


class SynthLlama:
    """Host tensors of a Llama / Qwen-shaped model (llm.rs:549-565) with the fc_llama_* structs.
    Matrices N(0, 0.02^2) -> Q8_0; norm weights 1 (+ noise when `perturb`); optional q/k/v biases."""

    def __init__(self, vocab, d_model, n_layer, n_head, n_kv_head, head_dim, d_ff, ctx, seed=0, perturb=False, math_mode=0,
                 rope_dim=None, rope_base=10000.0, rope_type=0, rope_linear_factor=1.0, freq_factors=None, norm_eps=1e-6,
                 tied=True, qkv_bias=False):
        rng = Rng(seed)
        d, F, V = d_model, d_ff, vocab
        qd, kvd = n_head * head_dim, n_kv_head * head_dim
        rope_dim = head_dim if rope_dim is None else rope_dim
        self.dims = dict(vocab=V, d_model=d, n_layer=n_layer, n_head=n_head, n_kv_head=n_kv_head, head_dim=head_dim, d_ff=F, ctx=ctx)
        self.keep = []

        def mat(n, k):
            q = q8_0_quantize(rng.normal(n * k, 0.02))
            self.keep.append(q)
            return q

        def vec(n, base, scale, always=False):
            v = np.full(n, base, dtype=np.float32)
            if perturb or always:
                v = v + rng.normal(n, scale)
            v = np.ascontiguousarray(v, dtype=np.float32)
            self.keep.append(v)
            return v

        self.token_embd = mat(V, d)
        self.layers = []
        for _ in range(n_layer):
            L = dict(attn_norm=vec(d, 1.0, 0.1), wq_q8=mat(qd, d), wk_q8=mat(kvd, d), wv_q8=mat(kvd, d), wo_q8=mat(d, qd),
                     ffn_norm=vec(d, 1.0, 0.1), gate_q8=mat(F, d), up_q8=mat(F, d), down_q8=mat(d, F))
            if qkv_bias:
                L.update(bq=vec(qd, 0.0, 0.02, True), bk=vec(kvd, 0.0, 0.02, True), bv=vec(kvd, 0.0, 0.02, True))
            self.layers.append(L)
        self.output_norm = vec(d, 1.0, 0.1)
        self.output = None if tied else mat(V, d)
        self.freq_factors = None if freq_factors is None else np.ascontiguousarray(freq_factors, dtype=np.float32)

        self.config = _lib.FcLlamaConfig(V, d, n_layer, n_head, n_kv_head, head_dim, F, rope_dim, rope_base, rope_type,
                                         rope_linear_factor, norm_eps, ctx, 1 if tied else 0, math_mode)
        self._layer_structs = (_lib.FcLlamaLayer * n_layer)()
        for i, L in enumerate(self.layers):
            for k, v in L.items():
                setattr(self._layer_structs[i], k, v.ctypes.data)
        self.weights = _lib.FcLlamaWeights(
            self.token_embd.ctypes.data, C.cast(self._layer_structs, C.POINTER(_lib.FcLlamaLayer)),
            self.output_norm.ctypes.data, None if tied else self.output.ctypes.data,
            None if self.freq_factors is None else self.freq_factors.ctypes.data)

    @property
    def q8_weight_bytes(self):
        """Bytes of Q8_0 matrices one decoded token streams (each matrix once, the head included)."""
        c = self.dims
        qd, kvd, d, F = c["n_head"] * c["head_dim"], c["n_kv_head"] * c["head_dim"], c["d_model"], c["d_ff"]
        per_layer = (qd + 2 * kvd) * d + d * qd + 3 * d * F
        return (c["n_layer"] * per_layer + d * c["vocab"]) * 34 // 32


def llama_named(name, **kw):
    return SynthLlama(*LLAMA_SHAPES[name], **kw)


def named(name, **kw):
    return SynthModel(*SHAPES[name], **kw)


def token_ids(seed, n, vocab):
    """n ids uniform in [0, vocab): next_u64() % vocab of the stream seeded with `seed`."""
    return Rng(seed).ids(n, vocab)
