/* ferrum_cuda.h — C ABI of libferrum_cuda.so: the Q8_0 GPT-2 forward path of Ferrum
 * on NVIDIA B200 (sm_100a).
 *
 * The reference (thomascherickal/ferrum-cpu, 100 % safe Rust) has no FFI surface; the
 * entry points below are what a `ferrum_cuda` crate binds to replace the Rust items
 * cited beside each declaration (paths are relative to the reference repository).
 *
 * Conventions
 *  - every call returns an int status: FC_OK (0) or a negative FC_E_* code; the text of
 *    the last error on the calling thread is returned by fc_last_error();
 *  - no call aborts, throws or traps; bad ids, shapes and full caches are FC_E_DIM as
 *    the reference's InferError::DimMismatch (ferrum_core/src/error.rs:6-26);
 *  - the caller owns every host buffer it passes; the library copies at create time and
 *    owns all device memory until the matching *_free;
 *  - one handle is used by one host thread at a time (the reference model is !Send,
 *    ferrum_core/src/layer/transformer.rs:82; the server keeps it on one thread,
 *    slm_server/src/model_thread.rs:111-143);
 *  - there is no CPU fallback: a call fails with FC_E_CUDA when no sm_100 device exists.
 */
#ifndef FERRUM_CUDA_H
#define FERRUM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FC_OK 0
#define FC_E_SHAPE (-1)     /* InferError::ShapeMismatch / NotAMatrix */
#define FC_E_DIM (-2)       /* InferError::DimMismatch: id >= vocab, cache full, width mismatch */
#define FC_E_FORMAT (-3)    /* InferError::Format: K % 32 != 0, null tensor */
#define FC_E_CUDA (-4)      /* a CUDA runtime call failed, or no sm_100 device */
#define FC_E_TIMEOUT (-5)   /* a bounded device-side wait ran out */
#define FC_E_CANCELLED (-6) /* the cancel flag was seen set */
#define FC_E_ARG (-7)       /* null handle / null required pointer */

/* Math modes of the prefill GEMM. Decode always runs fp32 FMA on CUDA cores. */
#define FC_MATH_FP32 0      /* fp32 CUDA-core GEMM (exactly rounded products) */
#define FC_MATH_BF16X3 1    /* tcgen05 kind::f16 bf16 operands, 3-term split, fp32 TMEM accumulate */

/* Dimensions of a gpt2-architecture GGUF (ferrum_core/src/loader/gpt2.rs:201-215). */
typedef struct fc_config {
    int32_t n_layer, d_model, n_head, d_ff, ctx, vocab;
    int32_t tied;       /* 1: no output.weight, the head is token_embd (gpt2.rs:228-233) */
    int32_t math_mode;  /* FC_MATH_* */
} fc_config;

/* One transformer block's tensors in GGUF order (loader/gpt2.rs:236-262). A `*_q8`
 * pointer is the raw GGML Q8_0 tensor: rows of K/32 blocks of 34 bytes
 * [u16 f16 scale, little endian][32 x i8] (gguf_write/blocks.rs:132-140). */
typedef struct fc_layer_weights {
    const void* attn_qkv_q8;  const float* attn_qkv_b;   /* [3d][d] rows Q,K,V ; [3d] */
    const void* attn_out_q8;  const float* attn_out_b;   /* [d][d] ; [d] */
    const float *ln1_g, *ln1_b, *ln2_g, *ln2_b;          /* attn_norm, ffn_norm ; [d] each */
    const void* ffn_up_q8;    const float* ffn_up_b;     /* [F][d] ; [F] */
    const void* ffn_down_q8;  const float* ffn_down_b;   /* [d][F] ; [d] */
} fc_layer_weights;

typedef struct fc_weights {
    const void* token_embd_q8;      /* [V][d] */
    const float* position_embd;     /* [ctx][d] f32 */
    const fc_layer_weights* layers; /* n_layer entries */
    const float *out_norm_g, *out_norm_b;
    const void* output_q8;          /* [V][d] or NULL when tied */
} fc_weights;

typedef struct fc_model fc_model;     /* Sequential + weights on one GPU (model.rs:51-71) */
typedef struct fc_stream fc_stream;   /* CachedTransformer: KV caches + position (slm/cached.rs:45-64) */
typedef struct fc_qweight fc_qweight; /* one Q8_0 matrix resident on a GPU (precedent: quant.rs:130-146 QWeight) */

/* Result of scoring, as ferrum_core/src/slm/scoring.rs Score {logprob, n_tokens, greedy}. */
typedef struct fc_score {
    double logprob;
    int64_t n_tokens;
    int32_t greedy;
} fc_score;

const char* fc_last_error(void);
/* Number of visible sm_100 devices (0 when none; never fails). */
int fc_device_count(void);

/* ---- host-side codecs (load time; not part of the forward pass) ------------------- */
/* quant.rs:271-280 q8_0_block over n values (n % 32 == 0) -> n/32*34 bytes. */
int fc_q8_0_quantize(const float* x, size_t n, void* out);
/* gguf/dequant.rs:37-49 dequant_q8_0. */
int fc_q8_0_dequantize(const void* raw, size_t n, float* out);
/* GGML block formats whose values are an f16 scale times a small integer re-blocked, exactly, to
 * Q8_0 (same scale, the integer as the int8 level): type 8 Q8_0 (copied), 2 Q4_0 (level = nibble
 * - 8, gguf/dequant.rs:66-83), 6 Q5_0 (level = 5-bit value - 16, gguf/dequant.rs:105-130). n
 * values (n % 32 == 0) -> n/32*34 bytes. d * level is then the very product the reference's
 * dequantiser forms, so every kernel here serves these files unchanged (at Q8_0's footprint).
 * Formats with a minimum or sub-block scales (Q4_1, Q5_1, K-quants) are FC_E_FORMAT here; they go through
 * fc_ggml_requantize_q8_0 below. */
#define FC_GGML_Q4_0 2
#define FC_GGML_Q5_0 6
#define FC_GGML_Q8_0 8
size_t fc_ggml_block_bytes(int ggml_type);   /* bytes of one 32-value block, 0 if not covered */
int fc_ggml_to_q8_0(int ggml_type, const void* raw, size_t n, void* out);
/* Every tensor type the reference's importer reads (gguf/format.rs:10-42, gguf/dequant.rs:37-315), decoded to
 * f32 with the reference's own order of operations (bit-identical): F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1
 * and the K-quants Q2_K .. Q6_K (super-blocks of 256). fc_ggml_type_bytes: storage of n values, 0 for an unknown
 * type or an n that is not a whole number of blocks (gguf/format.rs:107-130). fc_ggml_dequantize refuses data
 * shorter than n values (FC_E_FORMAT). fc_ggml_requantize_q8_0 is the import route for matrices: the exact
 * re-blocking above where it exists, else decode and re-encode with the Q8_0 block encoder along the row
 * (quant.rs:271-280) - what a wrapper beside the untouched loader does with the f32 layers it is handed, and the
 * counterpart of the reference re-packing every imported matrix to int8 / int4 (gguf/llama.rs:13-27). */
#define FC_GGML_F32 0
#define FC_GGML_F16 1
#define FC_GGML_Q4_1 3
#define FC_GGML_Q5_1 7
#define FC_GGML_Q8_1 9
#define FC_GGML_Q2_K 10
#define FC_GGML_Q3_K 11
#define FC_GGML_Q4_K 12
#define FC_GGML_Q5_K 13
#define FC_GGML_Q6_K 14
size_t fc_ggml_type_bytes(int ggml_type, size_t n);
int fc_ggml_dequantize(int ggml_type, const void* raw, size_t nbytes, size_t n, float* out);
int fc_ggml_requantize_q8_0(int ggml_type, const void* raw, size_t nbytes, size_t n, void* out);
/* A matrix [N = out][K = in] kept on the device in its GGML block format (its file footprint: 4.5 bits per weight for
 * Q4_0 / Q4_K, 5.5 for Q5_0 / Q5_K, 6.56 for Q6_K, ...) and multiplied with the blocks decoded inside the kernel:
 * y[M][N] = x[M][K] · dequant(W)ᵀ + bias. The decoded weights are bit-identical to gguf/dequant.rs (each value is
 * formed in the reference's order of operations), so this is Linear::forward on the f32 weights of the reference's
 * precision-preserving import (load_llama_prec(None), gguf/llama.rs:171-176) up to the order of the sum over k.
 * K must hold whole blocks of the type and be a multiple of 32; bias may be NULL. A format-generic kernel (one warp
 * per output row): the Q8_0 entries above are the fast path for Q8_0. */
typedef struct fc_ggml_weight fc_ggml_weight;
int fc_ggml_weight_upload(int device, int ggml_type, const void* raw, size_t nbytes, int N, int K, fc_ggml_weight** out);
void fc_ggml_weight_free(fc_ggml_weight* w);
int fc_ggml_linear(const fc_ggml_weight* w, const float* x, const float* bias, float* y, int M);
/* Device pointers (x_dev 16-byte aligned); returns after the launch. */
int fc_ggml_linear_dev(const fc_ggml_weight* w, const float* x_dev, const float* bias_dev, float* y_dev, int M, void* cuda_stream);
uint16_t fc_f32_to_f16(float v);  /* gguf_write/blocks.rs:12-61 */
float fc_f16_to_f32(uint16_t h);  /* gguf/dequant.rs:7-35 */
/* rng.rs:9-48 xorshift64*: seed -> state (0 is remapped), draws advance *state. */
uint64_t fc_rng_seed(uint64_t seed);
void fc_rng_fill_normal(uint64_t* state, float scale, size_t n, float* out);
void fc_rng_fill_ids(uint64_t* state, int32_t vocab, size_t n, int32_t* out);

/* ---- standalone Q8_0 linear: the matmul-engine entry ------------------------------ */
/* y[M][N] = x[M][K] · dequant(wq[N][K])ᵀ + bias — replaces ops::linear_forward
 * (ops.rs:233-256) on a weight kept packed (the seam Linear::forward dispatches on,
 * layer/linear.rs:191-194). Host buffers; copies in and out. M == 1 runs the decode
 * GEMV, M >= 2 the prefill GEMM in `math_mode`. bias may be NULL. */
int fc_q8_0_linear(int device, const float* x, const void* wq, const float* bias, float* y,
                   int M, int K, int N, int math_mode);
/* The same with the weight resident: upload once, multiply many times on device
 * pointers (x_dev, bias_dev, y_dev are device memory on the weight's GPU). The kernels read and
 * write them with 16-byte vector accesses: a pointer that is not 16-byte aligned (a sub-view at an
 * odd element offset, say) is refused with FC_E_ARG before anything is launched. This entry cannot
 * report a device-side timeout (it returns before the kernel ends); an fc_qweight handle is used
 * by one host thread at a time, like every other handle. */
int fc_qweight_upload(int device, const void* wq, int N, int K, fc_qweight** out);
void fc_qweight_free(fc_qweight* w);
int fc_q8_0_linear_dev(const fc_qweight* w, const float* x_dev, const float* bias_dev, float* y_dev,
                       int M, int math_mode, void* cuda_stream);

/* The same product as fc_q8_0_linear_dev in FC_MATH_BF16X3, for callers that must not
 * allocate device memory. No counterpart in the reference (it never leaves the host heap).
 *
 * Who needs it: a serving loop that handed all free device memory to its own pool at
 * start-up, so a cudaMalloc inside the library would fail; or a latency-critical thread that
 * cannot afford cudaMalloc taking the driver's allocation lock and synchronising with other
 * work on the device. fc_q8_0_linear_dev grows its scratch (the two bf16 planes the
 * activations are split into, plus a status word) with cudaMalloc on demand; this entry point
 * keeps that scratch in a fixed array inside the library instead and calls no cudaMalloc,
 * cudaFree or allocating library routine.
 *
 * Limits and rules:
 *  - M * K <= 4 194 304 activations per call (FC_E_SHAPE beyond that: split the rows over
 *    several calls, or use fc_q8_0_linear_dev); K % 64 == 0; the weight handle is uploaded
 *    beforehand with fc_qweight_upload (which does allocate);
 *  - the array is 16 MiB per GPU. The CUDA runtime loads the library's device code lazily, so the
 *    array (and the kernel images) are allocated by the driver at the FIRST call on a device, not
 *    when the library is loaded, and then held until the process exits: make one warm-up call per
 *    device before the host reserves the remaining device memory for its own pool (or run with
 *    CUDA_MODULE_LOADING=EAGER). From the second call on nothing is allocated;
 *  - that first call also looks up the array's device address; make it before any stream capture;
 *  - x_dev, y_dev and bias_dev must be 16-byte aligned (FC_E_ARG otherwise);
 *  - all calls on a device share the one array: two calls whose kernels can overlap on the
 *    GPU (different streams, no ordering between them) race on it. Issue them on one stream
 *    or order them with events;
 *  - x_dev, bias_dev (may be NULL) and y_dev are device pointers on the weight's GPU; the
 *    caller still provides input and output.
 * timed_out: NULL for a fully asynchronous call; otherwise the call waits for the stream and
 * stores the kernel's status word there (0, or FC_E_TIMEOUT, which is then also returned). */
int fc_q8_0_linear_dev_noalloc(const fc_qweight* w, const float* x_dev, const float* bias_dev, float* y_dev,
                               int M, void* cuda_stream, int* timed_out);

/* ---- model ------------------------------------------------------------------------ */
/* Validates as loader/gpt2.rs + loader/mod.rs:147-154 (d % n_head == 0, K % 32 == 0),
 * uploads and repacks the weights on `device`. */
int fc_model_create(const fc_config* cfg, const fc_weights* w, int device, fc_model** out);
/* The same from a GGUF file, without the f32 expansion of the matrices (the direct path the
 * reference names as future work, loader/decode.rs:99-100). Reads a gpt2-architecture GGUF
 * (version 2 or 3, gguf/header.rs:9-66) as loader/gpt2.rs:201-262 does: gpt2.context_length /
 * embedding_length / block_count / feed_forward_length / attention.head_count, and
 * gpt2.attention.layer_norm_epsilon, which must be 1e-5; tensors token_embd.weight,
 * position_embd.weight, blk.N.{attn_norm,attn_qkv,attn_output,ffn_norm,ffn_up,ffn_down}.
 * {weight,bias}, output_norm.{weight,bias}, optional output.weight (absent: tied head).
 * Matrices must be stored as Q8_0 (they are uploaded as stored), vectors and the position
 * table as F32; anything else is FC_E_FORMAT. row_perm (may be NULL) is the tokenizer's row
 * order, row_perm[model id] = row of the file (the `perm` of gpt2.rs:221-231, which stays with
 * the tokenizer on the caller's side); n_perm becomes the vocabulary size. */
int fc_model_load_gguf(const char* path, const int32_t* row_perm, int n_perm, int device, int math_mode, fc_model** out);
/* Parses and validates the same file without touching a GPU; fills the dimensions. */
int fc_gguf_probe(const char* path, const int32_t* row_perm, int n_perm, fc_config* out);
void fc_model_free(fc_model* m);
int fc_model_config(const fc_model* m, fc_config* out);

/* Per-layer statistics of a window forward: the device-side counterpart of the reference's verbose log
 * (model.rs:58-68 prints verbose::stats and check_nan_inf of every layer's output, verbose.rs:85-110).
 * When switched on (also by the environment variable FERRUM_CUDA_TRACE=1 at fc_model_create), every
 * scoring / predict_next forward leaves one record per layer output - the embedding, each transformer
 * block, the final LayerNorm - of the LAST forward pass the call ran: min, max, mean (f64 sum), and the
 * counts of NaN and Inf (NaN never enters min / max, as in the reference's comparisons). The head's logits
 * and the softmax are not materialised on this path and have no record. fc_model_read_layer_stats
 * copies up to cap records and returns how many (n_layer + 2 at most), or a negative status. */
typedef struct fc_layer_stats {
    float min, max, mean;
    int64_t nan_count, inf_count, n_elements;
} fc_layer_stats;
int fc_model_set_layer_stats(fc_model* m, int on);
int fc_model_read_layer_stats(fc_model* m, fc_layer_stats* out, int cap);

/* ---- scoring: Sequential::forward + the Softmax tail, fused ------------------------ */
/* B windows of exactly T <= ctx ids each (right-padded by the caller as scoring.rs:184-193
 * pads with id 0). For row t of window b the target is targets[b][t] (or -1: skip).
 * logprob = ln(max(p, 1e-12)) of the target under the model's softmax (f32 prob, f64 ln:
 * scoring.rs:175-181, loss.rs:12-18); is_greedy = argmax_first(row) == target. Outputs are
 * host arrays [B][T]; skipped rows get 0. */
int fc_score_windows(fc_model* m, const int32_t* ids, const int32_t* targets, int B, int T,
                     float* logprob, uint8_t* is_greedy);
/* GenerativeSLM::token_logprobs (scoring.rs:151-213): window plan, <= 32 windows per
 * forward, f64 sum. lp / is_greedy are optional host arrays of length n (entries below
 * `from` are left untouched). */
int fc_token_logprobs(fc_model* m, const int32_t* ids, int n, int from, fc_score* score,
                      float* lp, uint8_t* is_greedy);
/* n_seq independent sequences of seq_len ids each, all scored from target 1; windows of
 * different sequences share forward batches of `batch_windows` windows. */
int fc_score_sequences(fc_model* m, const int32_t* ids, int n_seq, int seq_len, int batch_windows,
                       fc_score* scores, float* lp);
/* Many scoring requests in shared forward passes (the reference's server scores them one by one,
 * slm_server/src/model_thread.rs:29-38): request r is ids[offsets[r] .. offsets[r+1]) scored from
 * target from[r] (GenerativeSLM::score(ctx, cont) is from = len(ctx), score_rolling from = 1;
 * slm/scoring.rs:95-140). Each request keeps its own window plan; the windows of all requests are
 * sorted by length and run batch_windows (0: 32) at a time. scores [n_req]. */
int fc_score_requests(fc_model* m, const int32_t* ids, const int64_t* offsets, const int32_t* from, int n_req, int batch_windows,
                      fc_score* scores);
/* Full-window next-token distributions, as TransformerSLMModel::predict_next
 * (slm_wasm/src/lib.rs:217-241): probs[V] of the last of n <= ctx ids. */
int fc_predict_next(fc_model* m, const int32_t* ids, int n, float* probs);

/* ---- KV-cached decode: CachedTransformer ----------------------------------------- */
int fc_stream_create(fc_model* m, fc_stream** out);   /* cached.rs:45-64 try_new */
void fc_stream_free(fc_stream* s);
int fc_stream_reset(fc_stream* s);                    /* cached.rs:93-98 */
/* How fc_feed / fc_prime / fc_generate_greedy run a token on the GPU. Both compute the same
 * CachedTransformer::feed; the per-kernel form exists to cross-check the persistent one.
 *   FC_DECODE_PERSISTENT: one cooperative kernel per batch of tokens (default when the model
 *                         shape fits it: d_model <= 1024, d_ff <= 4096, ctx <= 1024);
 *   FC_DECODE_PER_KERNEL: one kernel per layer operation, replayed from a CUDA graph. */
#define FC_DECODE_PERSISTENT 0
#define FC_DECODE_PER_KERNEL 1
int fc_stream_set_mode(fc_stream* s, int mode);
/* Tracing (the reference's per-layer verbose log, verbose.rs:11-110, has no timing; this is
 * its device-side counterpart). When on, the persistent decode kernel records the GPU's
 * nanosecond timer at every phase boundary of the last token of each launch:
 * entry 0 = token start, then 15 entries per block (LayerNorm1, QKV, barrier, attention,
 * barrier, combine, out-proj, barrier, LayerNorm2, up, barrier, load, down, barrier, load),
 * then the head phases. Every CTA of the kernel keeps its own
 * timeline (up to 256 entries): fc_stream_read_trace copies CTA 0's, fc_stream_read_trace_cta
 * that of CTA `cta`; both return the number of entries copied (or < 0). */
int fc_stream_set_trace(fc_stream* s, int on);
int fc_stream_read_trace(fc_stream* s, uint64_t* out, int cap);
int fc_stream_read_trace_cta(fc_stream* s, int cta, uint64_t* out, int cap);
int fc_cached_len(const fc_stream* s);
/* cached.rs:100-125 feed: one token; probs (host [V]) may be NULL. FC_E_DIM on id >= vocab
 * or a full cache (transformer.rs:237-242). */
int fc_feed(fc_stream* s, int32_t token, float* probs);
/* cached.rs:129-136 prime: reset, then feed every id. */
int fc_prime(fc_stream* s, const int32_t* ids, int n, float* probs);
/* token_stream.rs:66-189 with temperature <= 0: keep the last ctx prompt ids, prime, then
 * per step argmax_first(ln(max(p,1e-12))) (sampling.rs:96-104,147), stop before emitting
 * `eos` (pass -1 for none), re-prime on the last ctx/2 ids when the window outgrows ctx,
 * else feed. `cancel` (may be NULL) is polled on the host between steps
 * (sampling.rs:69-73); when seen set the call returns FC_E_CANCELLED with *n_out tokens
 * valid. out: host [max_new]. */
int fc_generate_greedy(fc_stream* s, const int32_t* prompt, int n, int max_new, int32_t eos,
                       const volatile int32_t* cancel, int32_t* out, int* n_out);

/* Decoding controls of slm/sampling.rs:26-39 SamplingParams (the cancel flag is a separate
 * argument). temperature <= 0: greedy argmax of the penalised logits, no draw. top_k 0 and
 * top_p 1.0 disable those filters, repetition_penalty 1.0 disables the penalty. */
typedef struct fc_sampling {
    float temperature;
    int32_t top_k;
    float top_p;
    float repetition_penalty;
} fc_sampling;
/* sample_with_params (slm/sampling.rs:124-210) on the device for one row of `n` logits (host
 * buffer): penalty over `recent` (once per occurrence), temperature softmax, top-k, top-p,
 * renormalise, one xorshift64* draw (rng.rs:29-40). *rng_state is advanced exactly as the
 * reference advances its Rng. Sums are block reductions, so a draw can differ from the
 * sequential reference only when r lands within rounding of a cumulative boundary; probabilities
 * tying exactly at the top-p cut are all kept. n <= 51200. */
int fc_sample_logits(int device, const float* logits, int n, const fc_sampling* params, const int32_t* recent, int n_recent,
                     uint64_t* rng_state, int32_t* token);
/* generate_tokens / stream_next (slm/token_stream.rs:66-189) with sampling: prime the last ctx
 * prompt ids, then per token draw from ln(max(p, 1e-12)) of the current distribution with the
 * window's ids as `recent`, stop on eos, re-prime on the last ctx/2 ids when the window
 * outgrows the context. The sampler and the generator state stay on the device between
 * tokens; *rng_state returns advanced. */
int fc_generate_sampled(fc_stream* s, const int32_t* prompt, int n, int max_new, int32_t eos, const fc_sampling* params,
                        uint64_t* rng_state, const volatile int32_t* cancel, int32_t* out, int* n_out);
/* n_streams independent greedy generations on one GPU: prompts [n_streams][prompt_len], out
 * [n_streams][max_new], n_out [n_streams]. Each is token_stream.rs:66-189 with temperature <= 0
 * on its own KV caches (a CachedTransformer per stream, slm/cached.rs:45-64). The streams advance
 * in lock step, up to 64 at a time: the prompts are primed as one batch of windows, then every
 * step takes all streams through each Q8_0 matrix at once, so the weights are read once per step
 * whatever the number of streams. A stream that picks `eos` (-1: none) stops emitting; the others
 * go on. The extra feed after the last sampled token (token_stream.rs:181-186) is not run. Streams
 * that would outgrow the context (prompt_len + max_new > ctx: they need the re-prime of
 * token_stream.rs:162-165) and single streams run one after the other as fc_generate_greedy.
 * More than 16 streams of a wave run as groups of 16 on parallel branches of the step's CUDA graph (each group
 * reads the weights once); the environment variable FERRUM_LOCKSTEP_GROUP=<n> sets another group size (a
 * tuning aid: tokens do not depend on it beyond the summation order of the kernels it selects).
 * Device time of the whole call: fc_last_batch_ms; of its primes alone: fc_last_batch_prime_ms. */
int fc_decode_batch(fc_model* m, int n_streams, const int32_t* prompts, int prompt_len, int max_new, int32_t eos,
                    int32_t* out, int* n_out);
float fc_last_batch_ms(const fc_model* m);
float fc_last_batch_prime_ms(const fc_model* m);

/* ---- several GPUs behind one call ---------------------------------------------------- */
/* The reference's server owns ONE model on one thread and serialises jobs (slm_server/src/model_thread.rs:
 * 111-143); scoring sequences and decode streams are independent, so a box of N GPUs serves them N at a
 * time with the weights replicated. These calls take N model handles (normally fc_model_create with the
 * same weights on devices 0..N-1), give each a contiguous block of the items - item i goes to model
 * i * N / n_items - on a host thread of its own, and write every block's results straight into the
 * caller's arrays: there is nothing to gather and no collective. Results are identical to the single-
 * model calls on the same items. The first failing model's status and message are returned. */
int fc_score_sequences_multi(fc_model* const* models, int n_models, const int32_t* ids, int n_seq, int seq_len, int batch_windows,
                             fc_score* scores, float* lp);
int fc_decode_batch_multi(fc_model* const* models, int n_models, int n_streams, const int32_t* prompts, int prompt_len, int max_new,
                          int32_t eos, int32_t* out, int* n_out);

/* ---- imported Llama / Qwen models (ferrum_core/src/llm.rs, llm_score.rs) ---------- */
/* The decoder family of llm.rs on the same Q8_0 kernels: RMSNorm (llm.rs:57-64), rotary
 * positions in both pairings with the GGUF's frequency scaling (llm.rs:126-185), grouped-query
 * attention over f32 KV caches (llm.rs:305-341), the SwiGLU feed-forward (llm.rs:417-428) and
 * the exact log-softmax scorer (llm_score.rs:21-96). */
#define FC_ROPE_NORM 0 /* rotate interleaved pairs (2i, 2i+1) — RopeType::Norm, llm.rs:97-98 */
#define FC_ROPE_NEOX 1 /* rotate split halves (i, i + rope_dim/2) — RopeType::Neox, llm.rs:99-100 */

/* LlamaConfig (llm.rs:491-519). */
typedef struct fc_llama_config {
    int32_t vocab, d_model, n_layer, n_head, n_kv_head, head_dim, d_ff;
    int32_t rope_dim;          /* even, <= head_dim */
    float rope_base;
    int32_t rope_type;         /* FC_ROPE_* */
    float rope_linear_factor;  /* RopeScaling::linear_factor; 1.0 = none */
    float norm_eps;
    int32_t ctx;
    int32_t tied;              /* 1: the head is token_embd (llm.rs:560-564) */
    int32_t math_mode;         /* FC_MATH_* of the window forward */
} fc_llama_config;

/* One LlamaBlock (llm.rs:438-447). Projections are raw GGML Q8_0 tensors [out][in]; the
 * optional f32 biases of the q, k, v projections (Qwen) may be NULL. */
typedef struct fc_llama_layer {
    const float* attn_norm;                          /* [d] */
    const void *wq_q8, *wk_q8, *wv_q8, *wo_q8;       /* [H*hd][d], [KV*hd][d] x2, [d][H*hd] */
    const float *bq, *bk, *bv;                       /* NULL or [H*hd], [KV*hd], [KV*hd] */
    const float* ffn_norm;                           /* [d] */
    const void *gate_q8, *up_q8, *down_q8;           /* [F][d] x2, [d][F] */
} fc_llama_layer;

typedef struct fc_llama_weights {
    const void* token_embd_q8;     /* [V][d]; rows are dequantised as they are looked up */
    const fc_llama_layer* layers;  /* n_layer entries */
    const float* output_norm;      /* [d] */
    const void* output_q8;         /* [V][d] or NULL when tied */
    const float* rope_freqs;       /* RopeScaling::freq_factors: NULL or [rope_dim/2] */
} fc_llama_weights;

typedef struct fc_llama fc_llama;             /* LlamaModel on one GPU (llm.rs:549-565) */
typedef struct fc_llama_cache fc_llama_cache; /* LlamaCache: per-layer KV rows + position (llm.rs:522-546) */

/* Validates as Attention::new (llm.rs:243-252: n_head % n_kv_head, rope_dim even and <=
 * head_dim) and RopeScaling::check (llm.rs:135-150: factors finite and > 0): FC_E_DIM. */
int fc_llama_create(const fc_llama_config* cfg, const fc_llama_weights* w, int device, fc_llama** out);
/* The same model with every Linear packed the way the reference's importer packs it (Gguf::load_llama(kind),
 * gguf/llama.rs:13-27,164-171): each Q8_0 matrix is decoded, transposed to [in][out] and packed by
 * QWeight::from_f32 (quant.rs:164-212) to per-input-row int8 (FC_Q_INT8) or int4 (FC_Q_INT4) - the LM head too, the
 * tied one from the transposed embedding (gguf/llama.rs:304-311) - and every forward runs ops::qlinear
 * (ops.rs:316-377) on them; the embedding table stays as stored. All fc_llama_* calls work on the result; the decode
 * step runs one kernel per operation. */
int fc_llama_create_packed(const fc_llama_config* cfg, const fc_llama_weights* w, int device, int kind, fc_llama** out);
void fc_llama_free(fc_llama* m);
/* Gguf::load_llama (gguf/llama.rs:164-339) for `llama` and `qwen2` files whose projections are
 * Q8_0 (they stay packed) and whose norms are F32: the same metadata keys, defaults and refusals
 * (yarn / longrope scaling, attn_factor != 1, biases other than q/k/v, FC_E_FORMAT). qwen2 rotates
 * split halves, llama interleaved pairs. ctx_cap > 0 lowers the context (and with it the KV
 * caches) below the file's context_length. fc_llama_gguf_probe validates without a GPU. */
int fc_llama_load_gguf(const char* path, int device, int math_mode, int ctx_cap, fc_llama** out);
/* Gguf::load_llama(kind) (gguf/llama.rs:164-171) from the file: fc_llama_load_gguf followed by the packing of
 * fc_llama_create_packed. */
int fc_llama_load_gguf_packed(const char* path, int device, int ctx_cap, int kind, fc_llama** out);
/* The reference's precision-preserving import (load_llama_prec(None), gguf/llama.rs:171-176: every tensor decoded to
 * f32, nothing re-quantised) without the expansion: every matrix stays on the device in the file's own block format
 * (Q4_0, Q5_0, Q8_0, Q4_1, Q5_1, Q2_K .. Q6_K, f16, f32: its file footprint, no Q8_0 copy), the embedding rows and
 * the Linears decode it inside their kernels (fc_ggml_linear), bit-identical weights, fp32 arithmetic. Rows must hold
 * whole blocks of their type (256 for the K-quants). All fc_llama_* calls work on the result; one kernel per
 * operation, the decode step captured in a CUDA graph. */
int fc_llama_load_gguf_native(const char* path, int device, int ctx_cap, fc_llama** out);
int fc_llama_gguf_probe(const char* path, fc_llama_config* out);
/* LlamaModel::forward_tokens (llm.rs:622-635): n ids -> logits [n][vocab] (host buffer). */
int fc_llama_forward_tokens(fc_llama* m, const int32_t* ids, int n, float* logits);
/* LlamaModel::score_from (llm_score.rs:76-96) with the windows of plan_windows
 * (llm_score.rs:21-32): score ids[from..] given what precedes them. lp (may be NULL) receives
 * ln softmax(logits)[target] of target i at lp[i - 1] (entries before `from` are 0);
 * is_greedy likewise. score_rolling (llm_score.rs:61-69) is from = 1. window must lie in
 * 2..=ctx (FC_E_DIM, llm_score.rs:42-50). */
int fc_llama_score_from(fc_llama* m, const int32_t* ids, int n, int from, int window, fc_score* score, float* lp,
                        uint8_t* is_greedy);
/* The same for n_seq sequences of seq_len ids each that fit one window (seq_len <= ctx),
 * several windows per forward: scores [n_seq], lp (may be NULL) [n_seq][seq_len - 1]. */
int fc_llama_score_sequences(fc_llama* m, const int32_t* ids, int n_seq, int seq_len, int batch_windows, fc_score* scores,
                             float* lp);
float fc_llama_last_score_ms(const fc_llama* m);

int fc_llama_cache_create(fc_llama* m, fc_llama_cache** out);
void fc_llama_cache_free(fc_llama_cache* c);
int fc_llama_cache_clear(fc_llama_cache* c);   /* LlamaCache::clear, llm.rs:536-541 */
int fc_llama_cache_pos(const fc_llama_cache* c);
/* LlamaModel::forward_one (llm.rs:610-618): one token at the cache position; logits (host
 * [vocab]) may be NULL. FC_E_DIM on id >= vocab or a full context. */
int fc_llama_forward_one(fc_llama_cache* c, int32_t token, float* logits);
/* The prompt loop of generate_inner (llm.rs:733-738) on its own: clears the cache, feeds ids[n]
 * and returns the logits after the last one (host [vocab], may be NULL). Prompts of 8 ids or
 * more run as one fp32 window forward that fills the caches (same values to fp32 rounding). */
int fc_llama_prime(fc_llama_cache* c, const int32_t* ids, int n, float* logits);
/* LlamaModel::generate_cancellable (llm.rs:658-754): prime the prompt token by token, then
 * draw up to min(max_new, ctx - n) tokens with sample_with_params over `recent` = prompt +
 * tokens so far, stopping after a token found in stops[n_stops] (it is kept in out). The
 * sampler and generator state stay on the device; *rng_state returns advanced. A prompt that
 * fills the context is FC_E_DIM (llm.rs:724-729). */
int fc_llama_generate(fc_llama_cache* c, const int32_t* prompt, int n, int max_new, const fc_sampling* params,
                      const int32_t* stops, int n_stops, uint64_t* rng_state, const volatile int32_t* cancel,
                      int32_t* out, int* n_out);
float fc_llama_last_decode_ms(const fc_llama_cache* c);

/* ---- per-row-scale int8 / int4 weights (quant.rs:122-263 QWeight, ops.rs:268-377 qlinear) ---- */
/* The in-memory quantised weight of the reference: [rows = in_features][cols = out_features]
 * row-major, one f32 scale per row. Int8: one i8 per weight. Int4: ceil(cols/2) bytes per row in
 * the split-half layout — byte b holds column b in its low nibble and column half + b in its
 * high nibble (quant.rs:137-144). */
#define FC_Q_INT8 0
#define FC_Q_INT4 1
/* Bytes of the packed matrix (QKind::packed_len). */
size_t fc_rowq_packed_len(int rows, int cols, int kind);
/* QWeight::from_f32 (quant.rs:164-212) on the host: scales [rows], q [fc_rowq_packed_len]. */
int fc_rowq_from_f32(const float* data, int rows, int cols, int kind, float* scales, uint8_t* q);
/* QWeight::to_f32 (quant.rs:226-263): out [rows][cols]. */
int fc_rowq_to_f32(const uint8_t* q, const float* scales, int rows, int cols, int kind, float* out);
typedef struct fc_rowq fc_rowq;   /* one QWeight resident on a GPU */
int fc_rowq_upload(int device, const uint8_t* q, const float* scales, int rows, int cols, int kind, fc_rowq** out);
void fc_rowq_free(fc_rowq* w);
/* ops::qlinear (ops.rs:316-377): y[M][cols] = bias + (x[M][rows] * scale) · levels, the scale
 * folded into the activations, never expanding the weights. Host buffers; bias [cols] is
 * required as in the reference. FC_E_DIM on a width mismatch is the caller's check (rows and
 * cols are the handle's). */
int fc_rowq_linear(const fc_rowq* w, const float* x, const float* bias, float* y, int M);
/* The same on device pointers, asynchronous on `stream` (a cudaStream_t, or NULL). x_dev, bias_dev and
 * y_dev must be 16-byte aligned (FC_E_ARG otherwise). */
int fc_rowq_linear_dev(const fc_rowq* w, const float* x_dev, const float* bias_dev, float* y_dev, int M, void* stream);

/* ---- introspection used by the benchmark ----------------------------------------- */
/* Kernel launches issued by this library on the calling thread since the last call
 * (returns the count and resets it). */
int64_t fc_take_launch_count(void);
/* Device time in ms of the decode steps of the last fc_generate_greedy on this stream
 * (CUDA events on the launching stream around the feeds after the prime). */
float fc_last_decode_ms(const fc_stream* s);
/* Device time in ms of the forward passes of the last scoring call on this model. */
float fc_last_score_ms(const fc_model* m);

/* ---- test hook ------------------------------------------------------------------------ */
/* Every device-side wait of the pipelined kernels (mbarriers of the tensor-core GEMM and of the
 * persistent decode kernel, its grid barrier) is bounded by a cycle budget (default 4e9, about two
 * seconds); when it runs out the kernel raises a status word, drains what it has in flight and
 * returns, and the call reports FC_E_TIMEOUT (the device-side counterpart of the reference's
 * request timeout, slm_server/src/model_thread.rs:48-56). This hook sets that budget for launches
 * made afterwards by this process and, with withhold_producers != 0, makes the producer warps of
 * those kernels copy nothing, so that a test can watch a wait run out and the handle stay usable.
 * Nothing faults, traps or waits without a limit. Not for production use: restore
 * (4000000000, 0) afterwards. */
int fc_debug_set_wait_budget(long long cycles, int withhold_producers);

#ifdef __cplusplus
}
#endif
#endif /* FERRUM_CUDA_H */
