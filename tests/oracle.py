"""ctypes wrapper of the CPU oracle (oracle/libferrum_oracle.so). Test infrastructure:
only tests, the smoke check and the benchmark's CPU-baseline leg import this module."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB_PATH = os.path.join(ORACLE_DIR, "libferrum_oracle.so")

_lib = None


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        # make rebuilds when a source is newer than the library
        subprocess.run(["make", "-C", ORACLE_DIR], check=True, capture_output=True)
        L = C.CDLL(LIB_PATH)
        L.fo_f32_to_f16.restype, L.fo_f32_to_f16.argtypes = C.c_uint16, [C.c_float]
        L.fo_f16_to_f32.restype, L.fo_f16_to_f32.argtypes = C.c_float, [C.c_uint16]
        L.fo_q8_0_encode.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.fo_q8_0_decode.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.fo_rng_seed.restype, L.fo_rng_seed.argtypes = C.c_uint64, [C.c_uint64]
        L.fo_rng_next_u64.restype, L.fo_rng_next_u64.argtypes = C.c_uint64, [C.POINTER(C.c_uint64)]
        L.fo_rng_fill_normal.argtypes = [C.POINTER(C.c_uint64), C.c_float, C.c_size_t, C.c_void_p]
        L.fo_rng_fill_ids.argtypes = [C.POINTER(C.c_uint64), C.c_int32, C.c_size_t, C.c_void_p]
        L.fo_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.fo_linear_naive.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.fo_q8_0_expand_kn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.fo_layernorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.fo_gelu.restype, L.fo_gelu.argtypes = C.c_float, [C.c_float]
        L.fo_softmax_rows.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.fo_argmax_first.restype, L.fo_argmax_first.argtypes = C.c_int, [C.c_void_p, C.c_int]
        L.fo_model_create.restype, L.fo_model_create.argtypes = C.c_void_p, [C.c_void_p, C.c_void_p, C.c_int]
        L.fo_model_free.argtypes = [C.c_void_p]
        L.fo_model_set_threads.argtypes = [C.c_void_p, C.c_int]
        L.fo_forward.restype, L.fo_forward.argtypes = C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.fo_stream_create.restype, L.fo_stream_create.argtypes = C.c_void_p, [C.c_void_p]
        L.fo_stream_free.argtypes = [C.c_void_p]
        L.fo_stream_reset.argtypes = [C.c_void_p]
        L.fo_cached_len.restype, L.fo_cached_len.argtypes = C.c_int, [C.c_void_p]
        L.fo_feed.restype, L.fo_feed.argtypes = C.c_int, [C.c_void_p, C.c_int, C.c_void_p]
        L.fo_prime.restype, L.fo_prime.argtypes = C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.fo_generate_greedy.restype = C.c_int
        L.fo_generate_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.fo_token_logprobs.restype = C.c_int
        L.fo_token_logprobs.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_double),
                                        C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_void_p, C.c_void_p]
        L.fo_pick_by_mass.restype, L.fo_pick_by_mass.argtypes = C.c_int, [C.c_void_p, C.c_int, C.c_float]
        L.fo_rng_next_f32.restype, L.fo_rng_next_f32.argtypes = C.c_float, [C.POINTER(C.c_uint64)]
        L.fo_sample_with_params.restype = C.c_int
        L.fo_sample_with_params.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int,
                                            C.POINTER(C.c_uint64)]
        L.fo_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_void_p]
        L.fo_apply_rope.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p, C.c_int, C.c_float]
        L.fo_silu_mul.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.fo_llama_plan_windows.restype = C.c_int
        L.fo_llama_plan_windows.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.fo_llama_log_prob.restype, L.fo_llama_log_prob.argtypes = C.c_double, [C.c_void_p, C.c_int, C.c_int]
        L.fo_llama_create.restype, L.fo_llama_create.argtypes = C.c_void_p, [C.c_void_p, C.c_void_p, C.c_int]
        L.fo_llama_free.argtypes = [C.c_void_p]
        L.fo_llama_pack.argtypes = [C.c_void_p, C.c_int]
        L.fo_llama_pack.restype = None
        L.fo_llama_set_f32.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int]
        L.fo_llama_forward_tokens.restype = C.c_int
        L.fo_llama_forward_tokens.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.fo_llama_cache_create.restype, L.fo_llama_cache_create.argtypes = C.c_void_p, [C.c_void_p]
        L.fo_llama_cache_free.argtypes = [C.c_void_p]
        L.fo_llama_cache_clear.argtypes = [C.c_void_p]
        L.fo_llama_cache_pos.restype, L.fo_llama_cache_pos.argtypes = C.c_int, [C.c_void_p]
        L.fo_llama_forward_one.restype, L.fo_llama_forward_one.argtypes = C.c_int, [C.c_void_p, C.c_int, C.c_void_p]
        L.fo_llama_score_from.restype = C.c_int
        L.fo_llama_score_from.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_double),
                                          C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_void_p, C.c_void_p]
        L.fo_llama_generate.restype = C.c_int
        L.fo_llama_generate.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float,
                                        C.c_void_p, C.c_int, C.POINTER(C.c_uint64), C.c_void_p]
        L.fo_dequant_q4_0.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.fo_dequant_q5_0.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
        L.fo_nibble_to_i8.restype, L.fo_nibble_to_i8.argtypes = C.c_int, [C.c_int]
        L.fo_rowq_packed_len.restype, L.fo_rowq_packed_len.argtypes = C.c_size_t, [C.c_int, C.c_int, C.c_int]
        L.fo_rowq_from_f32.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.fo_rowq_to_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.fo_rowq_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        _lib = L
    return _lib


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def q8_0_encode(x):
    x = f32(x).ravel()
    out = np.empty(x.size // 32 * 34, dtype=np.uint8)
    lib().fo_q8_0_encode(_ptr(x), x.size, _ptr(out))
    return out


def q8_0_decode(raw, n):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    lib().fo_q8_0_decode(_ptr(raw), n, _ptr(out))
    return out


def fill_normal(seed, n, scale):
    st = C.c_uint64(lib().fo_rng_seed(seed))
    out = np.empty(n, dtype=np.float32)
    lib().fo_rng_fill_normal(C.byref(st), scale, n, _ptr(out))
    return out


def fill_ids(seed, n, vocab):
    st = C.c_uint64(lib().fo_rng_seed(seed))
    out = np.empty(n, dtype=np.int32)
    lib().fo_rng_fill_ids(C.byref(st), vocab, n, _ptr(out))
    return out


def linear(x, w_kn, bias, threads=1, naive=False):
    x, w_kn = f32(x), f32(w_kn)
    m, k = x.shape
    n = w_kn.shape[1]
    b = None if bias is None else f32(bias)
    y = np.empty((m, n), dtype=np.float32)
    if naive:
        lib().fo_linear_naive(_ptr(x), _ptr(w_kn), None if b is None else _ptr(b), m, k, n, _ptr(y))
    else:
        lib().fo_linear(_ptr(x), _ptr(w_kn), None if b is None else _ptr(b), m, k, n, _ptr(y), threads)
    return y


def expand_kn(wq, n, k):
    """Q8_0 [n][k] -> f32 [k][n] exactly as the reference loader expands and transposes it."""
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    out = np.empty((k, n), dtype=np.float32)
    lib().fo_q8_0_expand_kn(_ptr(wq), n, k, _ptr(out))
    return out


def layernorm(x, g, b):
    x, g, b = f32(x), f32(g), f32(b)
    out = np.empty_like(x)
    lib().fo_layernorm(_ptr(x), _ptr(g), _ptr(b), x.shape[0], x.shape[1], _ptr(out))
    return out


def softmax_rows(x):
    x = f32(x)
    out = np.empty_like(x)
    lib().fo_softmax_rows(_ptr(x), x.shape[0], x.shape[1], _ptr(out))
    return out


class Rng:
    """rng.rs xorshift64*: the state travels with the object, as Rng does in the reference."""

    def __init__(self, seed):
        self.state = C.c_uint64(lib().fo_rng_seed(seed))

    def next_u64(self):
        return lib().fo_rng_next_u64(C.byref(self.state))

    def next_f32(self):
        return lib().fo_rng_next_f32(C.byref(self.state))


def pick_by_mass(probs, r):
    probs = f32(probs)
    return lib().fo_pick_by_mass(_ptr(probs), probs.size, r)


def sample_with_params(logits, rng, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0, recent=()):
    """slm/sampling.rs:124-210; advances `rng` exactly as the reference would."""
    logits = f32(logits)
    rec = np.ascontiguousarray(recent, dtype=np.int32)
    return lib().fo_sample_with_params(_ptr(logits), logits.size, temperature, top_k, top_p, repetition_penalty,
                                       _ptr(rec) if rec.size else None, rec.size, C.byref(rng.state))


def argmax_first(x):
    x = f32(x)
    return lib().fo_argmax_first(_ptr(x), x.size)


class OracleModel:
    """The restated reference model built from the same fc_config / fc_weights structs."""

    def __init__(self, synth_model, threads=1):
        self.sm = synth_model
        self.V = synth_model.dims[5]
        self.T = synth_model.dims[4]
        self._m = lib().fo_model_create(C.addressof(synth_model.config), C.addressof(synth_model.weights), threads)
        assert self._m, "oracle rejected the model"
        self._s = lib().fo_stream_create(self._m)

    def set_threads(self, n):
        lib().fo_model_set_threads(self._m, n)

    def forward(self, ids2d):
        ids2d = np.ascontiguousarray(ids2d, dtype=np.int32)
        b, t = ids2d.shape
        probs = np.empty((b * t, self.V), dtype=np.float32)
        assert lib().fo_forward(self._m, _ptr(ids2d), b, t, _ptr(probs)) == 0
        return probs

    def prime(self, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        probs = np.empty(self.V, dtype=np.float32)
        assert lib().fo_prime(self._s, _ptr(ids), ids.size, _ptr(probs)) == 0
        return probs

    def feed(self, token):
        probs = np.empty(self.V, dtype=np.float32)
        rc = lib().fo_feed(self._s, int(token), _ptr(probs))
        return probs if rc == 0 else None

    def reset(self):
        lib().fo_stream_reset(self._s)

    def cached_len(self):
        return lib().fo_cached_len(self._s)

    def generate_greedy(self, prompt, max_new, eos=-1):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(max(1, max_new), dtype=np.int32)
        margin = np.zeros(max(1, max_new), dtype=np.float32)
        n = lib().fo_generate_greedy(self._s, _ptr(prompt), prompt.size, max_new, eos, _ptr(out), _ptr(margin))
        assert n >= 0
        return out[:n].copy(), margin[:max(n, min(max_new, n + 1))].copy()

    def token_logprobs(self, ids, from_=1):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lp = np.zeros(ids.size, dtype=np.float32)
        gr = np.zeros(ids.size, dtype=np.uint8)
        total, n, g = C.c_double(), C.c_int(), C.c_int()
        rc = lib().fo_token_logprobs(self._m, _ptr(ids), ids.size, from_, C.byref(total), C.byref(n), C.byref(g),
                                     _ptr(lp), _ptr(gr))
        assert rc == 0
        return total.value, n.value, bool(g.value), lp, gr

    def close(self):
        if self._s:
            lib().fo_stream_free(self._s)
            self._s = None
        if self._m:
            lib().fo_model_free(self._m)
            self._m = None

    def __del__(self):
        self.close()


# ------------------------------------------------------------------ Llama / Qwen (llm.rs)
def rmsnorm(x, w, eps):
    x = f32(x)
    rows, d = (1, x.size) if x.ndim == 1 else x.shape
    out = np.empty_like(x)
    w = f32(w)
    lib().fo_rmsnorm(_ptr(x), _ptr(w), eps, rows, d, _ptr(out))
    return out


def apply_rope(x, n_heads, head_dim, rope_dim, pos, base=10000.0, neox=False, freq_factors=(), linear_factor=1.0):
    """llm.rs:158-185 on a copy of x."""
    x = f32(x).copy()
    ff = f32(freq_factors)
    lib().fo_apply_rope(_ptr(x), n_heads, head_dim, rope_dim, pos, base, int(neox), _ptr(ff) if ff.size else None, ff.size,
                        linear_factor)
    return x


def silu_mul(g, u):
    g, u = f32(g), f32(u)
    out = np.empty_like(g)
    lib().fo_silu_mul(_ptr(g), _ptr(u), g.size, _ptr(out))
    return out


def llama_plan_windows(n, window, from_):
    buf = np.zeros(3 * (n + 2), dtype=np.int32)
    k = lib().fo_llama_plan_windows(n, window, from_, _ptr(buf), n + 2)
    return [tuple(int(v) for v in buf[3 * i:3 * i + 3]) for i in range(k)]


def llama_log_prob(logits, target):
    logits = f32(logits)
    return lib().fo_llama_log_prob(_ptr(logits), logits.size, target)


class OracleLlama:
    """The restated LlamaModel built from the same fc_llama_config / fc_llama_weights structs."""

    def __init__(self, synth_llama, threads=1, prec=None):
        """prec 0 / 1: every Linear packed to per-row int8 / int4 (Gguf::load_llama(kind), gguf/llama.rs:164-171)."""
        self.sm = synth_llama
        self.V = synth_llama.dims["vocab"]
        self._m = lib().fo_llama_create(C.addressof(synth_llama.config), C.addressof(synth_llama.weights), threads)
        if self._m and prec is not None:
            lib().fo_llama_pack(self._m, int(prec))
        self._c = lib().fo_llama_cache_create(self._m) if self._m else None

    @property
    def ok(self):
        return bool(self._m)

    def set_f32(self, layer, which, w):
        """load_llama_prec(None): matrix `which` (0..6 of `layer`, 7 the head, 8 the embedding table) as decoded f32
        values [n_out][n_in]."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        assert lib().fo_llama_set_f32(self._m, layer, which, _ptr(w), w.shape[0], w.shape[1]) == 0

    def forward_tokens(self, ids):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty((ids.size, self.V), dtype=np.float32)
        assert lib().fo_llama_forward_tokens(self._m, _ptr(ids), ids.size, _ptr(out)) == 0
        return out

    def clear(self):
        lib().fo_llama_cache_clear(self._c)

    def pos(self):
        return lib().fo_llama_cache_pos(self._c)

    def forward_one(self, token):
        out = np.empty(self.V, dtype=np.float32)
        rc = lib().fo_llama_forward_one(self._c, int(token), _ptr(out))
        return out if rc == 0 else None

    def score_from(self, ids, from_, window):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        lp = np.zeros(max(ids.size, 1), dtype=np.float64)
        gr = np.zeros(max(ids.size, 1), dtype=np.uint8)
        total, n, g = C.c_double(), C.c_int(), C.c_int()
        rc = lib().fo_llama_score_from(self._m, _ptr(ids), ids.size, from_, window, C.byref(total), C.byref(n), C.byref(g),
                                       _ptr(lp), _ptr(gr))
        if rc != 0:
            return None
        return total.value, n.value, bool(g.value), lp[:max(ids.size - 1, 0)], gr[:max(ids.size - 1, 0)].astype(bool)

    def generate(self, prompt, max_new, rng, temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0, stops=()):
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        st = np.ascontiguousarray(stops, dtype=np.int32)
        out = np.zeros(max(max_new, 1), dtype=np.int32)
        n = lib().fo_llama_generate(self._c, _ptr(prompt), prompt.size, max_new, temperature, top_k, top_p, repetition_penalty,
                                    _ptr(st) if st.size else None, st.size, C.byref(rng.state), _ptr(out))
        return None if n < 0 else out[:n].copy()

    def close(self):
        if self._c:
            lib().fo_llama_cache_free(self._c)
            self._c = None
        if self._m:
            lib().fo_llama_free(self._m)
            self._m = None

    def __del__(self):
        self.close()


# ------------------------------------------------- per-row-scale QWeight (quant.rs, ops.rs)
def rowq_from_f32(data, kind):
    data = f32(data)
    rows, cols = data.shape
    q = np.zeros(lib().fo_rowq_packed_len(rows, cols, kind), dtype=np.uint8)
    scales = np.zeros(rows, dtype=np.float32)
    lib().fo_rowq_from_f32(_ptr(data), rows, cols, kind, _ptr(scales), _ptr(q))
    return q, scales


def rowq_to_f32(q, scales, rows, cols, kind):
    out = np.empty((rows, cols), dtype=np.float32)
    lib().fo_rowq_to_f32(_ptr(q), _ptr(scales), rows, cols, kind, _ptr(out))
    return out


def rowq_linear(x, q, scales, kind, bias, n):
    x = f32(x)
    m, k = x.shape
    bias = f32(bias)
    y = np.empty((m, n), dtype=np.float32)
    lib().fo_rowq_linear(_ptr(x), _ptr(q), _ptr(scales), kind, _ptr(bias), m, k, n, _ptr(y))
    return y


def dequant_ggml(ggml_type, raw, n):
    """gguf/dequant.rs dequant_q4_0 (type 2) / dequant_q5 without a minimum (type 6)."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    {2: lib().fo_dequant_q4_0, 6: lib().fo_dequant_q5_0}[ggml_type](_ptr(raw), n, _ptr(out))
    return out
