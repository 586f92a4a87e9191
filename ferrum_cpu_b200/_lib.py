"""ctypes binding of libferrum_cuda.so (the C ABI declared in include/ferrum_cuda.h).

The library is the product; there is no Python or CPU implementation behind it. Loading
fails loudly when the shared object has not been built (python -m ferrum_cpu_b200.build).
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libferrum_cuda.so")

FC_OK = 0
FC_E_SHAPE, FC_E_DIM, FC_E_FORMAT, FC_E_CUDA, FC_E_TIMEOUT, FC_E_CANCELLED, FC_E_ARG = -1, -2, -3, -4, -5, -6, -7
FC_MATH_FP32, FC_MATH_BF16X3 = 0, 1


class FcConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "d_model", "n_head", "d_ff", "ctx", "vocab", "tied", "math_mode")]


class FcLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "attn_qkv_q8", "attn_qkv_b", "attn_out_q8", "attn_out_b", "ln1_g", "ln1_b", "ln2_g", "ln2_b",
        "ffn_up_q8", "ffn_up_b", "ffn_down_q8", "ffn_down_b")]


class FcWeights(C.Structure):
    _fields_ = [("token_embd_q8", C.c_void_p), ("position_embd", C.c_void_p), ("layers", C.POINTER(FcLayerWeights)),
                ("out_norm_g", C.c_void_p), ("out_norm_b", C.c_void_p), ("output_q8", C.c_void_p)]


class FcSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("repetition_penalty", C.c_float)]


class FcLlamaConfig(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("d_model", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32),
                ("n_kv_head", C.c_int32), ("head_dim", C.c_int32), ("d_ff", C.c_int32), ("rope_dim", C.c_int32),
                ("rope_base", C.c_float), ("rope_type", C.c_int32), ("rope_linear_factor", C.c_float),
                ("norm_eps", C.c_float), ("ctx", C.c_int32), ("tied", C.c_int32), ("math_mode", C.c_int32)]


class FcLlamaLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "attn_norm", "wq_q8", "wk_q8", "wv_q8", "wo_q8", "bq", "bk", "bv", "ffn_norm", "gate_q8", "up_q8", "down_q8")]


class FcLlamaWeights(C.Structure):
    _fields_ = [("token_embd_q8", C.c_void_p), ("layers", C.POINTER(FcLlamaLayer)), ("output_norm", C.c_void_p),
                ("output_q8", C.c_void_p), ("rope_freqs", C.c_void_p)]


FC_ROPE_NORM, FC_ROPE_NEOX = 0, 1
FC_Q_INT8, FC_Q_INT4 = 0, 1


class FcScore(C.Structure):
    _fields_ = [("logprob", C.c_double), ("n_tokens", C.c_int64), ("greedy", C.c_int32)]


class FcLayerStats(C.Structure):
    _fields_ = [("min", C.c_float), ("max", C.c_float), ("mean", C.c_float), ("nan_count", C.c_int64), ("inf_count", C.c_int64),
                ("n_elements", C.c_int64)]


# name -> (restype, argtypes); every symbol include/ferrum_cuda.h declares
SIGNATURES = {
    "fc_last_error": (C.c_char_p, []),
    "fc_device_count": (C.c_int, []),
    "fc_q8_0_quantize": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "fc_q8_0_dequantize": (C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p]),
    "fc_ggml_block_bytes": (C.c_size_t, [C.c_int]),
    "fc_ggml_to_q8_0": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]),
    "fc_ggml_type_bytes": (C.c_size_t, [C.c_int, C.c_size_t]),
    "fc_ggml_dequantize": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "fc_ggml_requantize_q8_0": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "fc_ggml_weight_upload": (C.c_int, [C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_ggml_weight_free": (None, [C.c_void_p]),
    "fc_ggml_linear": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "fc_ggml_linear_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fc_f32_to_f16": (C.c_uint16, [C.c_float]),
    "fc_f16_to_f32": (C.c_float, [C.c_uint16]),
    "fc_rng_seed": (C.c_uint64, [C.c_uint64]),
    "fc_rng_fill_normal": (None, [C.POINTER(C.c_uint64), C.c_float, C.c_size_t, C.c_void_p]),
    "fc_rng_fill_ids": (None, [C.POINTER(C.c_uint64), C.c_int32, C.c_size_t, C.c_void_p]),
    "fc_q8_0_linear": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "fc_qweight_upload": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_qweight_free": (None, [C.c_void_p]),
    "fc_q8_0_linear_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "fc_q8_0_linear_dev_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.POINTER(C.c_int)]),
    "fc_model_create": (C.c_int, [C.POINTER(FcConfig), C.POINTER(FcWeights), C.c_int, C.POINTER(C.c_void_p)]),
    "fc_model_load_gguf": (C.c_int, [C.c_char_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_gguf_probe": (C.c_int, [C.c_char_p, C.c_void_p, C.c_int, C.POINTER(FcConfig)]),
    "fc_model_free": (None, [C.c_void_p]),
    "fc_model_config": (C.c_int, [C.c_void_p, C.POINTER(FcConfig)]),
    "fc_score_windows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "fc_token_logprobs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(FcScore), C.c_void_p, C.c_void_p]),
    "fc_score_sequences": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(FcScore), C.c_void_p]),
    "fc_score_requests": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(FcScore)]),
    "fc_predict_next": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fc_stream_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "fc_stream_free": (None, [C.c_void_p]),
    "fc_stream_reset": (C.c_int, [C.c_void_p]),
    "fc_cached_len": (C.c_int, [C.c_void_p]),
    "fc_stream_set_mode": (C.c_int, [C.c_void_p, C.c_int]),
    "fc_stream_set_trace": (C.c_int, [C.c_void_p, C.c_int]),
    "fc_stream_read_trace": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "fc_stream_read_trace_cta": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int]),
    "fc_feed": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "fc_prime": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fc_generate_greedy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int32, C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "fc_sample_logits": (C.c_int, [C.c_int, C.c_void_p, C.c_int, C.POINTER(FcSampling), C.c_void_p, C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_int32)]),
    "fc_generate_sampled": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int32, C.POINTER(FcSampling), C.POINTER(C.c_uint64), C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "fc_decode_batch": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int32, C.c_void_p, C.c_void_p]),
    "fc_last_batch_ms": (C.c_float, [C.c_void_p]),
    "fc_last_batch_prime_ms": (C.c_float, [C.c_void_p]),
    "fc_debug_set_wait_budget": (C.c_int, [C.c_longlong, C.c_int]),
    "fc_score_sequences_multi": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "fc_decode_batch_multi": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int32, C.c_void_p, C.c_void_p]),
    "fc_model_set_layer_stats": (C.c_int, [C.c_void_p, C.c_int]),
    "fc_model_read_layer_stats": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "fc_llama_create": (C.c_int, [C.POINTER(FcLlamaConfig), C.POINTER(FcLlamaWeights), C.c_int, C.POINTER(C.c_void_p)]),
    "fc_llama_free": (None, [C.c_void_p]),
    "fc_llama_load_gguf": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_llama_load_gguf_packed": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_llama_load_gguf_native": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_llama_create_packed": (C.c_int, [C.POINTER(FcLlamaConfig), C.POINTER(FcLlamaWeights), C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_llama_gguf_probe": (C.c_int, [C.c_char_p, C.POINTER(FcLlamaConfig)]),
    "fc_llama_forward_tokens": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fc_llama_score_from": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(FcScore), C.c_void_p, C.c_void_p]),
    "fc_llama_score_sequences": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(FcScore), C.c_void_p]),
    "fc_llama_last_score_ms": (C.c_float, [C.c_void_p]),
    "fc_llama_cache_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "fc_llama_cache_free": (None, [C.c_void_p]),
    "fc_llama_cache_clear": (C.c_int, [C.c_void_p]),
    "fc_llama_cache_pos": (C.c_int, [C.c_void_p]),
    "fc_llama_forward_one": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "fc_llama_prime": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fc_llama_generate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(FcSampling), C.c_void_p, C.c_int,
                                    C.POINTER(C.c_uint64), C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]),
    "fc_llama_last_decode_ms": (C.c_float, [C.c_void_p]),
    "fc_rowq_packed_len": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "fc_rowq_from_f32": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "fc_rowq_to_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fc_rowq_upload": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "fc_rowq_free": (None, [C.c_void_p]),
    "fc_rowq_linear": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "fc_rowq_linear_dev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "fc_take_launch_count": (C.c_int64, []),
    "fc_last_decode_ms": (C.c_float, [C.c_void_p]),
    "fc_last_score_ms": (C.c_float, [C.c_void_p]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ferrum_cpu_b200.build`. "
                "There is no fallback implementation.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


class FerrumCudaError(RuntimeError):
    """A negative status from the C ABI; `.code` is the FC_E_* value (InferError kinds)."""

    def __init__(self, code, message):
        super().__init__(f"[{code}] {message}")
        self.code = code


def check(rc):
    if rc != FC_OK:
        raise FerrumCudaError(rc, lib().fc_last_error().decode("utf-8", "replace"))
