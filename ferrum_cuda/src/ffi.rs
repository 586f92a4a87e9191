//! Raw bindings of libferrum_cuda.so: every entry point include/ferrum_cuda.h declares, with the same
//! argument order and meaning. This is the only module of the crate (and of Ferrum) that is `unsafe` to
//! call; `lib.rs` wraps it in owned handles that map statuses back to `InferError`.
//!
//! Not compiled in the environment this file was written in (no Rust toolchain there); the same ABI is
//! exercised symbol by symbol through the ctypes table of ferrum_cpu_b200/_lib.py, and tests/test_abi.py
//! checks that this file names every symbol of the header with the right number of arguments.
#![allow(non_camel_case_types, non_snake_case, clippy::too_many_arguments)]
use std::os::raw::{c_char, c_int, c_void};

pub const FC_OK: c_int = 0;
pub const FC_E_SHAPE: c_int = -1;
pub const FC_E_DIM: c_int = -2;
pub const FC_E_FORMAT: c_int = -3;
pub const FC_E_CUDA: c_int = -4;
pub const FC_E_TIMEOUT: c_int = -5;
pub const FC_E_CANCELLED: c_int = -6;
pub const FC_E_ARG: c_int = -7;
pub const FC_MATH_FP32: c_int = 0;
pub const FC_MATH_BF16X3: c_int = 1;
pub const FC_DECODE_PERSISTENT: c_int = 0;
pub const FC_DECODE_PER_KERNEL: c_int = 1;
pub const FC_ROPE_NORM: c_int = 0;
pub const FC_ROPE_NEOX: c_int = 1;
pub const FC_GGML_Q4_0: c_int = 2;
pub const FC_GGML_Q5_0: c_int = 6;
pub const FC_GGML_Q8_0: c_int = 8;
pub const FC_GGML_F32: c_int = 0;
pub const FC_GGML_F16: c_int = 1;
pub const FC_GGML_Q4_1: c_int = 3;
pub const FC_GGML_Q5_1: c_int = 7;
pub const FC_GGML_Q8_1: c_int = 9;
pub const FC_GGML_Q2_K: c_int = 10;
pub const FC_GGML_Q3_K: c_int = 11;
pub const FC_GGML_Q4_K: c_int = 12;
pub const FC_GGML_Q5_K: c_int = 13;
pub const FC_GGML_Q6_K: c_int = 14;
pub const FC_Q_INT8: c_int = 0;
pub const FC_Q_INT4: c_int = 1;

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct fc_config {
    pub n_layer: i32, pub d_model: i32, pub n_head: i32, pub d_ff: i32, pub ctx: i32, pub vocab: i32,
    pub tied: i32, pub math_mode: i32,
}
#[repr(C)]
pub struct fc_layer_weights {
    pub attn_qkv_q8: *const c_void, pub attn_qkv_b: *const f32,
    pub attn_out_q8: *const c_void, pub attn_out_b: *const f32,
    pub ln1_g: *const f32, pub ln1_b: *const f32, pub ln2_g: *const f32, pub ln2_b: *const f32,
    pub ffn_up_q8: *const c_void, pub ffn_up_b: *const f32,
    pub ffn_down_q8: *const c_void, pub ffn_down_b: *const f32,
}
#[repr(C)]
pub struct fc_weights {
    pub token_embd_q8: *const c_void, pub position_embd: *const f32, pub layers: *const fc_layer_weights,
    pub out_norm_g: *const f32, pub out_norm_b: *const f32, pub output_q8: *const c_void,
}
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct fc_score { pub logprob: f64, pub n_tokens: i64, pub greedy: i32 }
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct fc_layer_stats { pub min: f32, pub max: f32, pub mean: f32, pub nan_count: i64, pub inf_count: i64, pub n_elements: i64 }
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct fc_sampling { pub temperature: f32, pub top_k: i32, pub top_p: f32, pub repetition_penalty: f32 }
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct fc_llama_config {
    pub vocab: i32, pub d_model: i32, pub n_layer: i32, pub n_head: i32, pub n_kv_head: i32, pub head_dim: i32, pub d_ff: i32,
    pub rope_dim: i32, pub rope_base: f32, pub rope_type: i32, pub rope_linear_factor: f32, pub norm_eps: f32, pub ctx: i32,
    pub tied: i32, pub math_mode: i32,
}
#[repr(C)]
pub struct fc_llama_layer {
    pub attn_norm: *const f32,
    pub wq_q8: *const c_void, pub wk_q8: *const c_void, pub wv_q8: *const c_void, pub wo_q8: *const c_void,
    pub bq: *const f32, pub bk: *const f32, pub bv: *const f32,
    pub ffn_norm: *const f32,
    pub gate_q8: *const c_void, pub up_q8: *const c_void, pub down_q8: *const c_void,
}
#[repr(C)]
pub struct fc_llama_weights {
    pub token_embd_q8: *const c_void, pub layers: *const fc_llama_layer, pub output_norm: *const f32,
    pub output_q8: *const c_void, pub rope_freqs: *const f32,
}

/// Opaque handles: the library owns what is behind them until the matching `*_free`.
pub enum fc_model {}
pub enum fc_stream {}
pub enum fc_qweight {}
pub enum fc_ggml_weight {}
pub enum fc_llama {}
pub enum fc_llama_cache {}
pub enum fc_rowq {}

#[link(name = "ferrum_cuda")]
extern "C" {
    pub fn fc_last_error() -> *const c_char;
    pub fn fc_device_count() -> c_int;
    pub fn fc_q8_0_quantize(x: *const f32, n: usize, out: *mut c_void) -> c_int;
    pub fn fc_q8_0_dequantize(raw: *const c_void, n: usize, out: *mut f32) -> c_int;
    pub fn fc_ggml_block_bytes(ggml_type: c_int) -> usize;
    pub fn fc_ggml_to_q8_0(ggml_type: c_int, raw: *const c_void, n: usize, out: *mut c_void) -> c_int;
    pub fn fc_ggml_type_bytes(ggml_type: c_int, n: usize) -> usize;
    pub fn fc_ggml_dequantize(ggml_type: c_int, raw: *const c_void, nbytes: usize, n: usize, out: *mut f32) -> c_int;
    pub fn fc_ggml_requantize_q8_0(ggml_type: c_int, raw: *const c_void, nbytes: usize, n: usize, out: *mut c_void) -> c_int;
    pub fn fc_ggml_weight_upload(device: c_int, ggml_type: c_int, raw: *const c_void, nbytes: usize, n: c_int, k: c_int, out: *mut *mut fc_ggml_weight) -> c_int;
    pub fn fc_ggml_weight_free(w: *mut fc_ggml_weight);
    pub fn fc_ggml_linear(w: *const fc_ggml_weight, x: *const f32, bias: *const f32, y: *mut f32, m: c_int) -> c_int;
    pub fn fc_ggml_linear_dev(w: *const fc_ggml_weight, x_dev: *const f32, bias_dev: *const f32, y_dev: *mut f32, m: c_int, cuda_stream: *mut c_void) -> c_int;
    pub fn fc_f32_to_f16(v: f32) -> u16;
    pub fn fc_f16_to_f32(h: u16) -> f32;
    pub fn fc_rng_seed(seed: u64) -> u64;
    pub fn fc_rng_fill_normal(state: *mut u64, scale: f32, n: usize, out: *mut f32);
    pub fn fc_rng_fill_ids(state: *mut u64, vocab: i32, n: usize, out: *mut i32);
    pub fn fc_q8_0_linear(device: c_int, x: *const f32, wq: *const c_void, bias: *const f32, y: *mut f32, M: c_int, K: c_int, N: c_int, math_mode: c_int) -> c_int;
    pub fn fc_qweight_upload(device: c_int, wq: *const c_void, N: c_int, K: c_int, out: *mut *mut fc_qweight) -> c_int;
    pub fn fc_qweight_free(w: *mut fc_qweight);
    pub fn fc_q8_0_linear_dev(w: *const fc_qweight, x_dev: *const f32, bias_dev: *const f32, y_dev: *mut f32, M: c_int, math_mode: c_int, cuda_stream: *mut c_void) -> c_int;
    pub fn fc_q8_0_linear_dev_noalloc(w: *const fc_qweight, x_dev: *const f32, bias_dev: *const f32, y_dev: *mut f32, M: c_int, cuda_stream: *mut c_void, timed_out: *mut c_int) -> c_int;
    pub fn fc_model_create(cfg: *const fc_config, w: *const fc_weights, device: c_int, out: *mut *mut fc_model) -> c_int;
    pub fn fc_model_load_gguf(path: *const c_char, row_perm: *const i32, n_perm: c_int, device: c_int, math_mode: c_int, out: *mut *mut fc_model) -> c_int;
    pub fn fc_gguf_probe(path: *const c_char, row_perm: *const i32, n_perm: c_int, out: *mut fc_config) -> c_int;
    pub fn fc_model_free(m: *mut fc_model);
    pub fn fc_model_config(m: *const fc_model, out: *mut fc_config) -> c_int;
    pub fn fc_model_set_layer_stats(m: *mut fc_model, on: c_int) -> c_int;
    pub fn fc_model_read_layer_stats(m: *mut fc_model, out: *mut fc_layer_stats, cap: c_int) -> c_int;
    pub fn fc_score_windows(m: *mut fc_model, ids: *const i32, targets: *const i32, B: c_int, T: c_int, logprob: *mut f32, is_greedy: *mut u8) -> c_int;
    pub fn fc_token_logprobs(m: *mut fc_model, ids: *const i32, n: c_int, from_: c_int, score: *mut fc_score, lp: *mut f32, is_greedy: *mut u8) -> c_int;
    pub fn fc_score_sequences(m: *mut fc_model, ids: *const i32, n_seq: c_int, seq_len: c_int, batch_windows: c_int, scores: *mut fc_score, lp: *mut f32) -> c_int;
    pub fn fc_score_requests(m: *mut fc_model, ids: *const i32, offsets: *const i64, from_: *const i32, n_req: c_int, batch_windows: c_int, scores: *mut fc_score) -> c_int;
    pub fn fc_predict_next(m: *mut fc_model, ids: *const i32, n: c_int, probs: *mut f32) -> c_int;
    pub fn fc_stream_create(m: *mut fc_model, out: *mut *mut fc_stream) -> c_int;
    pub fn fc_stream_free(s: *mut fc_stream);
    pub fn fc_stream_reset(s: *mut fc_stream) -> c_int;
    pub fn fc_stream_set_mode(s: *mut fc_stream, mode: c_int) -> c_int;
    pub fn fc_stream_set_trace(s: *mut fc_stream, on: c_int) -> c_int;
    pub fn fc_stream_read_trace(s: *mut fc_stream, out: *mut u64, cap: c_int) -> c_int;
    pub fn fc_stream_read_trace_cta(s: *mut fc_stream, cta: c_int, out: *mut u64, cap: c_int) -> c_int;
    pub fn fc_cached_len(s: *const fc_stream) -> c_int;
    pub fn fc_feed(s: *mut fc_stream, token: i32, probs: *mut f32) -> c_int;
    pub fn fc_prime(s: *mut fc_stream, ids: *const i32, n: c_int, probs: *mut f32) -> c_int;
    pub fn fc_generate_greedy(s: *mut fc_stream, prompt: *const i32, n: c_int, max_new: c_int, eos: i32, cancel: *const i32, out: *mut i32, n_out: *mut c_int) -> c_int;
    pub fn fc_sample_logits(device: c_int, logits: *const f32, n: c_int, params: *const fc_sampling, recent: *const i32, n_recent: c_int, rng_state: *mut u64, token: *mut i32) -> c_int;
    pub fn fc_generate_sampled(s: *mut fc_stream, prompt: *const i32, n: c_int, max_new: c_int, eos: i32, params: *const fc_sampling, rng_state: *mut u64, cancel: *const i32, out: *mut i32, n_out: *mut c_int) -> c_int;
    pub fn fc_decode_batch(m: *mut fc_model, n_streams: c_int, prompts: *const i32, prompt_len: c_int, max_new: c_int, eos: i32, out: *mut i32, n_out: *mut c_int) -> c_int;
    pub fn fc_last_batch_ms(m: *const fc_model) -> f32;
    pub fn fc_last_batch_prime_ms(m: *const fc_model) -> f32;
    pub fn fc_score_sequences_multi(models: *const *mut fc_model, n_models: c_int, ids: *const i32, n_seq: c_int, seq_len: c_int, batch_windows: c_int, scores: *mut fc_score, lp: *mut f32) -> c_int;
    pub fn fc_decode_batch_multi(models: *const *mut fc_model, n_models: c_int, n_streams: c_int, prompts: *const i32, prompt_len: c_int, max_new: c_int, eos: i32, out: *mut i32, n_out: *mut c_int) -> c_int;
    pub fn fc_llama_create(cfg: *const fc_llama_config, w: *const fc_llama_weights, device: c_int, out: *mut *mut fc_llama) -> c_int;
    pub fn fc_llama_free(m: *mut fc_llama);
    pub fn fc_llama_load_gguf(path: *const c_char, device: c_int, math_mode: c_int, ctx_cap: c_int, out: *mut *mut fc_llama) -> c_int;
    pub fn fc_llama_load_gguf_packed(path: *const c_char, device: c_int, ctx_cap: c_int, kind: c_int, out: *mut *mut fc_llama) -> c_int;
    pub fn fc_llama_load_gguf_native(path: *const c_char, device: c_int, ctx_cap: c_int, out: *mut *mut fc_llama) -> c_int;
    pub fn fc_llama_create_packed(cfg: *const fc_llama_config, w: *const fc_llama_weights, device: c_int, kind: c_int, out: *mut *mut fc_llama) -> c_int;
    pub fn fc_llama_gguf_probe(path: *const c_char, out: *mut fc_llama_config) -> c_int;
    pub fn fc_llama_forward_tokens(m: *mut fc_llama, ids: *const i32, n: c_int, logits: *mut f32) -> c_int;
    pub fn fc_llama_score_from(m: *mut fc_llama, ids: *const i32, n: c_int, from_: c_int, window: c_int, score: *mut fc_score, lp: *mut f32, is_greedy: *mut u8) -> c_int;
    pub fn fc_llama_score_sequences(m: *mut fc_llama, ids: *const i32, n_seq: c_int, seq_len: c_int, batch_windows: c_int, scores: *mut fc_score, lp: *mut f32) -> c_int;
    pub fn fc_llama_last_score_ms(m: *const fc_llama) -> f32;
    pub fn fc_llama_cache_create(m: *mut fc_llama, out: *mut *mut fc_llama_cache) -> c_int;
    pub fn fc_llama_cache_free(c: *mut fc_llama_cache);
    pub fn fc_llama_cache_clear(c: *mut fc_llama_cache) -> c_int;
    pub fn fc_llama_cache_pos(c: *const fc_llama_cache) -> c_int;
    pub fn fc_llama_forward_one(c: *mut fc_llama_cache, token: i32, logits: *mut f32) -> c_int;
    pub fn fc_llama_prime(c: *mut fc_llama_cache, ids: *const i32, n: c_int, logits: *mut f32) -> c_int;
    pub fn fc_llama_generate(c: *mut fc_llama_cache, prompt: *const i32, n: c_int, max_new: c_int, params: *const fc_sampling, stops: *const i32, n_stops: c_int, rng_state: *mut u64, cancel: *const i32, out: *mut i32, n_out: *mut c_int) -> c_int;
    pub fn fc_llama_last_decode_ms(c: *const fc_llama_cache) -> f32;
    pub fn fc_rowq_packed_len(rows: c_int, cols: c_int, kind: c_int) -> usize;
    pub fn fc_rowq_from_f32(data: *const f32, rows: c_int, cols: c_int, kind: c_int, scales: *mut f32, q: *mut u8) -> c_int;
    pub fn fc_rowq_to_f32(q: *const u8, scales: *const f32, rows: c_int, cols: c_int, kind: c_int, out: *mut f32) -> c_int;
    pub fn fc_rowq_upload(device: c_int, q: *const u8, scales: *const f32, rows: c_int, cols: c_int, kind: c_int, out: *mut *mut fc_rowq) -> c_int;
    pub fn fc_rowq_free(w: *mut fc_rowq);
    pub fn fc_rowq_linear(w: *const fc_rowq, x: *const f32, bias: *const f32, y: *mut f32, M: c_int) -> c_int;
    pub fn fc_rowq_linear_dev(w: *const fc_rowq, x_dev: *const f32, bias_dev: *const f32, y_dev: *mut f32, M: c_int, stream: *mut c_void) -> c_int;
    pub fn fc_take_launch_count() -> i64;
    pub fn fc_last_decode_ms(s: *const fc_stream) -> f32;
    pub fn fc_last_score_ms(m: *const fc_model) -> f32;
    pub fn fc_debug_set_wait_budget(cycles: i64, withhold_producers: c_int) -> c_int;
}
