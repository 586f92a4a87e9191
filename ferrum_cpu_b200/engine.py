"""Python face of the C ABI, named after the reference interfaces it stands in for.

CudaSlm mirrors the numeric subset of ferrum_core's GenerativeSLM / CachedTransformer and
the wasm TransformerSLMModel (slm/scoring.rs, slm/cached.rs, slm/token_stream.rs,
slm_wasm/src/lib.rs:217-241) on token ids; text, tokenizer and stop strings stay with the
caller. Every method is a thin ctypes call: the arithmetic lives in libferrum_cuda.so.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import FerrumCudaError, check  # noqa: F401


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _ids(ids):
    return np.ascontiguousarray(ids, dtype=np.int32)


@dataclass
class Score:
    """slm/scoring.rs Score."""
    logprob: float
    n_tokens: int
    greedy: bool


def device_count():
    return _lib.lib().fc_device_count()


def sampling(temperature=1.0, top_k=0, top_p=1.0, repetition_penalty=1.0):
    """slm/sampling.rs SamplingParams (defaults as SamplingParams::default)."""
    return _lib.FcSampling(temperature, top_k, top_p, repetition_penalty)


def sample_logits(logits, rng_state, params, recent=(), device=0):
    """One draw of sample_with_params on the GPU; returns (token, advanced rng state)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    rec = np.ascontiguousarray(recent, dtype=np.int32)
    state = C.c_uint64(rng_state)
    tok = C.c_int32(0)
    check(_lib.lib().fc_sample_logits(device, _ptr(logits), logits.size, C.byref(params), _ptr(rec) if rec.size else None, rec.size,
                                      C.byref(state), C.byref(tok)))
    return tok.value, state.value


def gguf_probe(path, row_perm=None):
    """Dimensions of a gpt2-architecture GGUF file; validates it without a GPU."""
    perm = None if row_perm is None else np.ascontiguousarray(row_perm, dtype=np.int32)
    cfg = _lib.FcConfig()
    check(_lib.lib().fc_gguf_probe(str(path).encode(), None if perm is None else _ptr(perm), 0 if perm is None else perm.size,
                                   C.byref(cfg)))
    return cfg


def take_launch_count():
    return _lib.lib().fc_take_launch_count()


def q8_0_linear(x, wq, bias, n_out, device=0, math_mode=_lib.FC_MATH_FP32):
    """y = x · dequant(wq)ᵀ + bias with host arrays (ops::linear_forward on a packed weight)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    wq = np.ascontiguousarray(wq, dtype=np.uint8)
    y = np.empty((m, n_out), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    check(_lib.lib().fc_q8_0_linear(device, _ptr(x), _ptr(wq), None if b is None else _ptr(b), _ptr(y),
                                    m, k, n_out, math_mode))
    return y


def rowq_from_f32(data, kind):
    """QWeight::from_f32 (quant.rs:164-212) on the host: (packed bytes, scales) of a [rows][cols] matrix."""
    data = np.ascontiguousarray(data, dtype=np.float32)
    rows, cols = data.shape
    q = np.zeros(_lib.lib().fc_rowq_packed_len(rows, cols, kind), dtype=np.uint8)
    scales = np.zeros(rows, dtype=np.float32)
    check(_lib.lib().fc_rowq_from_f32(_ptr(data), rows, cols, kind, _ptr(scales), _ptr(q)))
    return q, scales


def rowq_to_f32(q, scales, rows, cols, kind):
    """QWeight::to_f32 (quant.rs:255-263)."""
    q = np.ascontiguousarray(q, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    out = np.empty((rows, cols), dtype=np.float32)
    check(_lib.lib().fc_rowq_to_f32(_ptr(q), _ptr(scales), rows, cols, kind, _ptr(out)))
    return out


class RowQWeight:
    """A per-row-scale int8 / int4 QWeight resident on a GPU (quant.rs:122-146); `linear` is ops::qlinear."""

    def __init__(self, q, scales, rows, cols, kind, device=0):
        self.rows, self.cols, self.kind = rows, cols, kind
        self._h = C.c_void_p()
        q = np.ascontiguousarray(q, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        check(_lib.lib().fc_rowq_upload(device, _ptr(q), _ptr(scales), rows, cols, kind, C.byref(self._h)))

    @classmethod
    def from_f32(cls, data, kind, device=0):
        data = np.ascontiguousarray(data, dtype=np.float32)
        q, scales = rowq_from_f32(data, kind)
        return cls(q, scales, data.shape[0], data.shape[1], kind, device)

    def linear(self, x, bias):
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim != 2 or x.shape[1] != self.rows:
            raise FerrumCudaError(_lib.FC_E_DIM, f"qlinear: input width {x.shape[-1]} ≠ weight rows {self.rows}")
        bias = np.ascontiguousarray(bias, dtype=np.float32)
        if bias.size != self.cols:
            raise FerrumCudaError(_lib.FC_E_DIM, f"qlinear: bias length {bias.size} ≠ out_features {self.cols}")
        y = np.empty((x.shape[0], self.cols), dtype=np.float32)
        check(_lib.lib().fc_rowq_linear(self._h, _ptr(x), _ptr(bias), _ptr(y), x.shape[0]))
        return y

    def linear_dev(self, x_ptr, bias_ptr, y_ptr, m, stream=None):
        check(_lib.lib().fc_rowq_linear_dev(self._h, C.c_void_p(x_ptr), C.c_void_p(bias_ptr), C.c_void_p(y_ptr), m, stream))

    def close(self):
        if self._h:
            _lib.lib().fc_rowq_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class QWeight:
    """One Q8_0 matrix resident on a GPU (the packed-weight seam of layer/linear.rs:21-35)."""

    def __init__(self, wq, n_out, k_in, device=0):
        wq = np.ascontiguousarray(wq, dtype=np.uint8)
        self._h = C.c_void_p()
        self.n, self.k, self.device = n_out, k_in, device
        check(_lib.lib().fc_qweight_upload(device, _ptr(wq), n_out, k_in, C.byref(self._h)))

    def linear_dev(self, x_dev_ptr, bias_dev_ptr, y_dev_ptr, m, math_mode=_lib.FC_MATH_FP32, stream=None):
        check(_lib.lib().fc_q8_0_linear_dev(self._h, x_dev_ptr, bias_dev_ptr, y_dev_ptr, m, math_mode, stream))

    def linear_dev_noalloc(self, x_dev_ptr, bias_dev_ptr, y_dev_ptr, m, stream=None, wait=True):
        """The tensor-core linear out of the library's fixed scratch array: no device allocation.
        M * K <= 4 Mi; calls that can overlap on the GPU race on the shared scratch."""
        status = C.c_int(0)
        check(_lib.lib().fc_q8_0_linear_dev_noalloc(self._h, x_dev_ptr, bias_dev_ptr, y_dev_ptr, m, stream,
                                                    C.byref(status) if wait else None))

    def close(self):
        if self._h:
            _lib.lib().fc_qweight_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        self.close()


class CudaSlm:
    """A GPT-2-architecture Q8_0 model on one GPU plus one KV-cached stream."""

    def __init__(self, config, weights, device=0, _handle=None):
        self._m = C.c_void_p()
        self._s = C.c_void_p()
        if _handle is not None:
            self._m = _handle
        else:
            check(_lib.lib().fc_model_create(C.byref(config), C.byref(weights), device, C.byref(self._m)))
        cfg = _lib.FcConfig()
        check(_lib.lib().fc_model_config(self._m, C.byref(cfg)))
        self.config = cfg
        self.device = device

    @classmethod
    def from_gguf(cls, path, row_perm=None, device=0, math_mode=_lib.FC_MATH_FP32):
        """loader/gpt2.rs gpt2_from on a file, the tensors uploaded as stored (no f32 expansion)."""
        perm = None if row_perm is None else np.ascontiguousarray(row_perm, dtype=np.int32)
        h = C.c_void_p()
        check(_lib.lib().fc_model_load_gguf(str(path).encode(), None if perm is None else _ptr(perm),
                                            0 if perm is None else perm.size, device, math_mode, C.byref(h)))
        return cls(None, None, device=device, _handle=h)

    # ---- scoring (slm/scoring.rs) ---------------------------------------------------
    def token_logprobs(self, ids, from_=1, per_token=False):
        ids = _ids(ids)
        sc = _lib.FcScore()
        lp = np.zeros(ids.size, dtype=np.float32) if per_token else None
        gr = np.zeros(ids.size, dtype=np.uint8) if per_token else None
        check(_lib.lib().fc_token_logprobs(self._m, _ptr(ids), ids.size, from_, C.byref(sc),
                                           None if lp is None else _ptr(lp), None if gr is None else _ptr(gr)))
        score = Score(sc.logprob, sc.n_tokens, bool(sc.greedy))
        return (score, lp, gr) if per_token else score

    def evaluate_ids(self, ids):
        """scoring.rs:77-87: every id after the first is a target."""
        return self.token_logprobs(ids, 1)

    def score_sequences(self, ids2d, batch_windows=32, lp_out=None):
        ids2d = _ids(ids2d)
        n_seq, seq_len = ids2d.shape
        scores = (_lib.FcScore * n_seq)()
        lp = lp_out if lp_out is not None else np.zeros((n_seq, seq_len), dtype=np.float32)
        check(_lib.lib().fc_score_sequences(self._m, _ptr(ids2d), n_seq, seq_len, batch_windows, scores, _ptr(lp)))
        return [Score(s.logprob, s.n_tokens, bool(s.greedy)) for s in scores], lp

    def score_requests(self, requests, batch_windows=32):
        """Many (ids, first scored target) requests in shared forward passes: one Score per request.
        GenerativeSLM::score(ctx, cont) is (ctx + cont, len(ctx)); score_rolling is (ids, 1)."""
        seqs = [_ids(r[0]) for r in requests]
        offsets = np.zeros(len(seqs) + 1, dtype=np.int64)
        offsets[1:] = np.cumsum([s.size for s in seqs])
        flat = np.concatenate(seqs) if seqs else np.zeros(0, dtype=np.int32)
        start = np.ascontiguousarray([r[1] for r in requests], dtype=np.int32)
        scores = (_lib.FcScore * max(len(seqs), 1))()
        check(_lib.lib().fc_score_requests(self._m, _ptr(flat) if flat.size else None, _ptr(offsets), _ptr(start) if start.size else None,
                                           len(seqs), batch_windows, scores))
        return [Score(s.logprob, s.n_tokens, bool(s.greedy)) for s in scores[:len(seqs)]]

    def score_windows(self, ids2d, targets2d):
        ids2d, targets2d = _ids(ids2d), _ids(targets2d)
        b, t = ids2d.shape
        lp = np.zeros((b, t), dtype=np.float32)
        gr = np.zeros((b, t), dtype=np.uint8)
        check(_lib.lib().fc_score_windows(self._m, _ptr(ids2d), _ptr(targets2d), b, t, _ptr(lp), _ptr(gr)))
        return lp, gr

    def predict_next(self, ids):
        """TransformerSLMModel::predict_next: probabilities after the last of `ids`."""
        ids = _ids(ids)
        probs = np.empty(self.config.vocab, dtype=np.float32)
        check(_lib.lib().fc_predict_next(self._m, _ptr(ids), ids.size, _ptr(probs)))
        return probs

    @property
    def last_score_ms(self):
        return _lib.lib().fc_last_score_ms(self._m)

    # ---- KV-cached decode (slm/cached.rs, slm/token_stream.rs) --------------------------
    def _stream(self):
        if not self._s:
            check(_lib.lib().fc_stream_create(self._m, C.byref(self._s)))
        return self._s

    def prime(self, ids, want_probs=True):
        ids = _ids(ids)
        probs = np.empty(self.config.vocab, dtype=np.float32) if want_probs else None
        check(_lib.lib().fc_prime(self._stream(), _ptr(ids), ids.size, None if probs is None else _ptr(probs)))
        return probs

    def predict_next_cached(self, token, want_probs=True):
        """CachedTransformer::feed / TokenModel::predict_next_cached."""
        probs = np.empty(self.config.vocab, dtype=np.float32) if want_probs else None
        check(_lib.lib().fc_feed(self._stream(), int(token), None if probs is None else _ptr(probs)))
        return probs

    feed = predict_next_cached

    def reset(self):
        check(_lib.lib().fc_stream_reset(self._stream()))

    def set_trace(self, on):
        check(_lib.lib().fc_stream_set_trace(self._stream(), int(on)))

    def read_trace(self, cta=0, absolute=False):
        """Phase timeline (ns) of CTA `cta` for the last traced token: relative to that CTA's
        token start, or the raw timer values when `absolute`."""
        buf = np.zeros(256, dtype=np.uint64)
        n = _lib.lib().fc_stream_read_trace_cta(self._stream(), cta, _ptr(buf), buf.size)
        if n < 0:
            check(n)
        t = buf[:n].astype(np.int64)
        return t if absolute or not n else t - t[0]

    def set_decode_mode(self, mode):
        """0: persistent decode kernel (default), 1: one kernel per layer operation."""
        check(_lib.lib().fc_stream_set_mode(self._stream(), mode))

    def cached_len(self):
        return _lib.lib().fc_cached_len(self._stream())

    def generate_tokens(self, prompt_ids, max_tokens, eos=-1, cancel=None, out=None):
        """generate_tokens with temperature <= 0: greedy ids (token_stream.rs:66-189)."""
        prompt = _ids(prompt_ids)
        buf = out if out is not None else np.empty(max(max_tokens, 1), dtype=np.int32)
        n_out = C.c_int(0)
        rc = _lib.lib().fc_generate_greedy(self._stream(), _ptr(prompt), prompt.size, max_tokens, eos,
                                           None if cancel is None else _ptr(cancel), _ptr(buf), C.byref(n_out))
        if rc == _lib.FC_E_CANCELLED:
            return buf[:n_out.value].copy(), True
        check(rc)
        return buf[:n_out.value].copy(), False

    def generate_sampled(self, prompt_ids, max_tokens, params, rng_state, eos=-1, cancel=None):
        """generate_tokens with a sampler (token_stream.rs:66-189); returns (ids, advanced rng state)."""
        prompt = _ids(prompt_ids)
        buf = np.empty(max(max_tokens, 1), dtype=np.int32)
        n_out = C.c_int(0)
        state = C.c_uint64(rng_state)
        rc = _lib.lib().fc_generate_sampled(self._stream(), _ptr(prompt), prompt.size, max_tokens, eos, C.byref(params),
                                            C.byref(state), None if cancel is None else _ptr(cancel), _ptr(buf), C.byref(n_out))
        if rc != _lib.FC_E_CANCELLED:
            check(rc)
        return buf[:n_out.value].copy(), state.value

    def decode_batch(self, prompts2d, max_tokens, eos=-1):
        """Independent greedy streams (rows of prompts2d) on this GPU; returns a list of id arrays."""
        prompts = _ids(prompts2d)
        n, plen = prompts.shape
        out = np.zeros((n, max(max_tokens, 1)), dtype=np.int32)
        n_out = np.zeros(n, dtype=np.int32)
        check(_lib.lib().fc_decode_batch(self._m, n, _ptr(prompts), plen, max_tokens, eos, _ptr(out), _ptr(n_out)))
        return [out[i, :n_out[i]].copy() for i in range(n)]

    def set_layer_stats(self, on=True):
        """Per-layer min / max / mean / NaN / Inf records of the window forwards (verbose.rs:85-110)."""
        check(_lib.lib().fc_model_set_layer_stats(self._m, 1 if on else 0))

    def layer_stats(self):
        """Records of the last forward pass: embedding, every block, final LayerNorm."""
        n = self.config.n_layer + 2
        buf = (_lib.FcLayerStats * n)()
        got = _lib.lib().fc_model_read_layer_stats(self._m, buf, n)
        if got < 0:
            check(got)
        return [dict(min=b.min, max=b.max, mean=b.mean, nan_count=b.nan_count, inf_count=b.inf_count, n_elements=b.n_elements) for b in buf[:got]]

    @property
    def last_batch_ms(self):
        return _lib.lib().fc_last_batch_ms(self._m)

    @property
    def last_batch_prime_ms(self):
        """Device time of the primes inside the last decode_batch call."""
        return _lib.lib().fc_last_batch_prime_ms(self._m)

    @property
    def last_decode_ms(self):
        return _lib.lib().fc_last_decode_ms(self._stream())

    def close(self):
        if self._s:
            _lib.lib().fc_stream_free(self._s)
            self._s = C.c_void_p()
        if self._m:
            _lib.lib().fc_model_free(self._m)
            self._m = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _handles(models):
    arr = (C.c_void_p * len(models))(*[m._m for m in models])
    return arr


def score_sequences_multi(models, ids2d, batch_windows=32):
    """fc_score_sequences_multi: the sequences split in contiguous blocks over several CudaSlm (one per GPU),
    each driven by its own host thread inside the call. Returns (scores, lp) as CudaSlm.score_sequences."""
    ids2d = _ids(ids2d)
    n_seq, seq_len = ids2d.shape
    scores = (_lib.FcScore * n_seq)()
    lp = np.zeros((n_seq, seq_len), dtype=np.float32)
    check(_lib.lib().fc_score_sequences_multi(_handles(models), len(models), _ptr(ids2d), n_seq, seq_len, batch_windows, scores, _ptr(lp)))
    return [Score(s.logprob, s.n_tokens, bool(s.greedy)) for s in scores], lp


def decode_batch_multi(models, prompts2d, max_tokens, eos=-1):
    """fc_decode_batch_multi: the streams split in contiguous blocks over several CudaSlm."""
    prompts = _ids(prompts2d)
    n, plen = prompts.shape
    out = np.zeros((n, max(max_tokens, 1)), dtype=np.int32)
    n_out = np.zeros(n, dtype=np.int32)
    check(_lib.lib().fc_decode_batch_multi(_handles(models), len(models), n, _ptr(prompts), plen, max_tokens, eos, _ptr(out), _ptr(n_out)))
    return [out[i, :n_out[i]].copy() for i in range(n)]
