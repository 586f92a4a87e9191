"""Python face of the Llama / Qwen part of the C ABI, named after ferrum_core's LlamaModel
(llm.rs:549-766, llm_score.rs:41-96). Token ids in, logits / scores / token ids out; every
method is a thin ctypes call into libferrum_cuda.so.
"""
import ctypes as C
import weakref

import numpy as np

from . import _lib
from ._lib import check
from .engine import Score, _ids, _ptr


def gguf_probe(path):
    """Configuration of a llama / qwen2 GGUF file; validates it without a GPU."""
    cfg = _lib.FcLlamaConfig()
    check(_lib.lib().fc_llama_gguf_probe(str(path).encode(), C.byref(cfg)))
    return cfg


class CudaLlamaCache:
    """LlamaCache (llm.rs:522-546): per-layer KV rows and the position of the next token."""

    def __init__(self, model):
        self.model = model
        self._h = C.c_void_p()
        check(_lib.lib().fc_llama_cache_create(model._h, C.byref(self._h)))
        model._caches.append(weakref.ref(self))

    def close(self):
        if self._h:
            _lib.lib().fc_llama_cache_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def clear(self):
        check(_lib.lib().fc_llama_cache_clear(self._h))

    def pos(self):
        return _lib.lib().fc_llama_cache_pos(self._h)

    @property
    def last_decode_ms(self):
        return _lib.lib().fc_llama_last_decode_ms(self._h)


class CudaLlama:
    """LlamaModel on one GPU."""

    def __init__(self, config, weights, device=0, prec=None):
        self._h = C.c_void_p()
        self._caches = []
        self.config = config
        if prec is None:
            check(_lib.lib().fc_llama_create(C.byref(config), C.byref(weights), device, C.byref(self._h)))
        else:
            check(_lib.lib().fc_llama_create_packed(C.byref(config), C.byref(weights), device, int(prec), C.byref(self._h)))

    @classmethod
    def from_synth(cls, synth, device=0, prec=None):
        """prec: None runs the Q8_0 matrices as stored; 0 / 1 packs every Linear to per-row int8 / int4 as the
        reference's importer does (Gguf::load_llama(kind), gguf/llama.rs:164-171)."""
        return cls(synth.config, synth.weights, device, prec=prec)

    @classmethod
    def from_gguf(cls, path, device=0, math_mode=_lib.FC_MATH_FP32, ctx_cap=0, prec=None):
        """Gguf::load_llama (gguf/llama.rs:164-339) for llama / qwen2 files."""
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        self._caches = []
        self.config = gguf_probe(path)
        if 0 < ctx_cap < self.config.ctx:
            self.config.ctx = ctx_cap
        self.config.math_mode = math_mode
        if prec is None:
            check(_lib.lib().fc_llama_load_gguf(str(path).encode(), device, math_mode, ctx_cap, C.byref(self._h)))
        elif prec == "native":
            # load_llama_prec(None): the file's own blocks, decoded inside the kernels
            check(_lib.lib().fc_llama_load_gguf_native(str(path).encode(), device, ctx_cap, C.byref(self._h)))
        else:
            check(_lib.lib().fc_llama_load_gguf_packed(str(path).encode(), device, ctx_cap, int(prec), C.byref(self._h)))
        return self

    def close(self):
        for ref in self._caches:                 # caches go first: they hold device memory of this model's context
            cache = ref()
            if cache is not None:
                cache.close()
        self._caches = []
        if self._h:
            _lib.lib().fc_llama_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- full-sequence forward and scoring -------------------------------------------------
    def forward_tokens(self, ids):
        """llm.rs:622-635: logits [n][vocab]."""
        ids = _ids(ids)
        out = np.empty((ids.size, self.config.vocab), dtype=np.float32)
        check(_lib.lib().fc_llama_forward_tokens(self._h, _ptr(ids), ids.size, _ptr(out)))
        return out

    def score_from(self, ids, start, window, per_token=False):
        """llm_score.rs:76-96: (Score of ids[start..] given the prefix, all-greedy flag)."""
        ids = _ids(ids)
        sc = _lib.FcScore()
        lp = np.zeros(max(ids.size - 1, 1), dtype=np.float32)
        gr = np.zeros(max(ids.size - 1, 1), dtype=np.uint8)
        check(_lib.lib().fc_llama_score_from(self._h, _ptr(ids), ids.size, start, window, C.byref(sc), _ptr(lp), _ptr(gr)))
        score = Score(sc.logprob, sc.n_tokens, bool(sc.greedy))
        if per_token:
            return score, lp[:max(ids.size - 1, 0)], gr[:max(ids.size - 1, 0)].astype(bool)
        return score

    def score_rolling(self, ids, window):
        """llm_score.rs:61-69: every token but the first; at least two ids."""
        ids = _ids(ids)
        if ids.size < 2:
            raise _lib.FerrumCudaError(_lib.FC_E_DIM, "scoring needs at least two tokens (one to condition on, one to predict)")
        return self.score_from(ids, 1, window)

    def score_sequences(self, ids, batch_windows=8, per_token=False):
        """One window per row of ids [n_seq][seq_len], several windows per forward."""
        ids = _ids(ids)
        n_seq, seq_len = ids.shape
        scores = (_lib.FcScore * max(n_seq, 1))()
        lp = np.zeros((n_seq, seq_len - 1), dtype=np.float32)
        check(_lib.lib().fc_llama_score_sequences(self._h, _ptr(ids), n_seq, seq_len, batch_windows, scores, _ptr(lp)))
        out = [Score(s.logprob, s.n_tokens, bool(s.greedy)) for s in scores[:n_seq]]
        return (out, lp) if per_token else out

    @property
    def last_score_ms(self):
        return _lib.lib().fc_llama_last_score_ms(self._h)

    # ---- KV-cached decode ------------------------------------------------------------------
    def new_cache(self):
        return CudaLlamaCache(self)

    def forward_one(self, token, cache, want_logits=True):
        """llm.rs:610-618: next-token logits; advances the cache."""
        out = np.empty(self.config.vocab, dtype=np.float32) if want_logits else None
        check(_lib.lib().fc_llama_forward_one(cache._h, int(token), None if out is None else _ptr(out)))
        return out

    def prime(self, ids, cache, want_logits=True):
        """Clear the cache and feed a prompt (llm.rs:733-738); logits after its last token."""
        ids = _ids(ids)
        out = np.empty(self.config.vocab, dtype=np.float32) if want_logits else None
        check(_lib.lib().fc_llama_prime(cache._h, _ptr(ids), ids.size, None if out is None else _ptr(out)))
        return out

    def generate(self, prompt, max_new, params, stops=(), rng_state=1, cache=None, cancel=None):
        """llm.rs:643-754: (new token ids, advanced generator state)."""
        prompt = _ids(prompt)
        cache = cache or self.new_cache()
        stops_a = np.ascontiguousarray(stops, dtype=np.int32)
        out = np.zeros(max(max_new, 1), dtype=np.int32)
        n_out = C.c_int(0)
        state = C.c_uint64(rng_state)
        cancel_p = None if cancel is None else C.cast(C.byref(cancel), C.c_void_p)
        check(_lib.lib().fc_llama_generate(cache._h, _ptr(prompt), prompt.size, max_new, C.byref(params),
                                           _ptr(stops_a) if stops_a.size else None, stops_a.size, C.byref(state), cancel_p,
                                           _ptr(out), C.byref(n_out)))
        self.last_cache_pos = cache.pos()
        return out[:n_out.value].copy(), state.value
