// Shared declarations of libferrum_cuda: error plumbing, the device layout of a Q8_0
// matrix, and the launch wrappers of every kernel file.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <vector>

#include "../../include/ferrum_cuda.h"

namespace fc {

// ---- errors -------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);
int fail(int code, const char* fmt, ...);
const char* g_err_text();   // the calling thread's last error text
extern thread_local int64_t g_launches;

#define FC_CUDA(expr)                                                               \
    do {                                                                            \
        cudaError_t e__ = (expr);                                                   \
        if (e__ != cudaSuccess) return fc::cuda_fail(e__, #expr, __FILE__, __LINE__); \
    } while (0)
#define FC_TRY(expr)                \
    do {                            \
        int rc__ = (expr);          \
        if (rc__ != FC_OK) return rc__; \
    } while (0)
// After a kernel launch: count it and surface launch-configuration errors.
#define FC_LAUNCHED()                \
    do {                             \
        ++fc::g_launches;            \
        FC_CUDA(cudaGetLastError()); \
    } while (0)

// Device pointers a caller hands to the *_dev entry points are read and written with 16-byte
// vector accesses: anything else is refused on the host before a kernel is launched.
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// Test hooks (fc_debug_set_wait_budget): the cycle budget of every bounded device-side wait, and a
// switch that makes the producers of the pipelined kernels withhold their copies, so that a test can
// make a wait run out without faulting, trapping or hanging anything.
struct DebugKnobs {
    long long wait_cycles = 4000000000LL;   // ~2 s at 1.9 GHz
    int withhold = 0;
};
extern DebugKnobs g_debug;

// ---- host helpers shared by the API files (defined in api.cu) ---------------------------
// Owns device allocations until release().
struct Arena {
    std::vector<void*> ptrs;
    int alloc(void** p, size_t bytes) {
        FC_CUDA(cudaMalloc(p, bytes ? bytes : 16));
        ptrs.push_back(*p);
        return FC_OK;
    }
    template <class T>
    int alloc_n(T** p, size_t n) { return alloc((void**)p, n * sizeof(T)); }
    void release() {
        for (void* p : ptrs) cudaFree(p);
        ptrs.clear();
    }
};
struct QMat;
// Makes `device` current; refuses anything but an sm_100 part (there is no other code path).
int select_device(int device);
int upload_f32(Arena& ar, const float* host, size_t n, float** dev, cudaStream_t st);
// Raw GGML Q8_0 rows [N][K/32 x 34 B] -> the device planes of QMat.
int upload_q8(Arena& ar, const void* host, int N, int K, QMat* out, cudaStream_t st);

// ---- device layout of one Q8_0 matrix [N][K] ----------------------------------------
// The 34-byte GGML blocks are split at upload into two planes so that every row starts
// on a 16-byte boundary:
//   qu [N_pad][K]      uint8  = int8 quant XOR 0x80 (i.e. q + 128), K contiguous
//   d  [N_pad][K/32]   f16    block scales
// Rows N..N_pad-1 are zero scale / 0x80 quants (value 0) so tiles may read them.
struct QMat {
    const uint8_t* qu = nullptr;
    const __half* d = nullptr;
    int N = 0, K = 0, N_pad = 0;
};
constexpr int kRowPad = 128;

enum Epilogue : int { EPI_NONE = 0, EPI_GELU = 1, EPI_SWIGLU = 2, EPI_SCORE = 3 };

// activation.rs:9-12 (tanh GELU), same constants and association as the reference.
__device__ __forceinline__ float gelu_f(float x) {
    const float K = 0.7978846f;
    return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}

// ---- decode-step device state (one per stream) ----------------------------------------
// The "window" of token_stream.rs lives on the device: ids fed so far and ids waiting to
// be fed, so that a whole greedy generation runs without a host round trip.
struct StepState {
    int pos;       // cache position of the next fed token (== cached_len)
    int fed;       // index in queue of the next token to feed
    int tail;      // number of ids in queue
    int done;      // set when eos was selected: later steps do nothing
    int eos;       // -1: none
    int error;     // non-zero: bad id / cache full seen on device (FC_E_DIM)
    int pad[2];
};

// ---- kernel launchers (each returns FC_OK or FC_E_CUDA) --------------------------------
// repack.cu
int launch_repack_q8(const uint8_t* raw, int N, int K, int N_pad, uint8_t* qu, __half* d, cudaStream_t st);

// gemv.cu — y = W·x + bias (+GELU) (+residual), one activation row.
struct GemvOut {
    // Row n of the result goes to out[n / seg][n % seg]; segments 1 and 2 (K and V rows of
    // the fused QKV matrix) are offset by pos * pos_stride floats, pos read from `state`.
    float* out[3] = {nullptr, nullptr, nullptr};
    int seg = 0;
    size_t pos_stride = 0;
};
int launch_gemv_q8(const QMat& w, const float* x, const float* bias, const float* residual, int epi,
                   const GemvOut& out, const StepState* state, cudaStream_t st);

// Split-K form for wide matrices: optional RMSNorm of x (norm_w, eps) as it is staged; epi
// EPI_SWIGLU pairs rows (2i, 2i+1) as (gate, up) and writes out[i] = silu(gate) * up.
int launch_gemv_q8_wide(const QMat& w, const float* x, const float* norm_w, float eps, const float* bias, const float* residual,
                        int epi, float* out, const StepState* state, cudaStream_t st);

// gemv_stream.cu — the same contract on a persistent kernel that streams row tiles through a
// shared-memory ring with bulk async copies; `status` (device int) is raised to FC_E_TIMEOUT when
// a bounded wait runs out. Shapes the ring does not cover take launch_gemv_q8_wide.
int launch_gemv_q8_stream(const QMat& w, const float* x, const float* norm_w, float eps, const float* bias, const float* residual,
                          int epi, float* out, const StepState* state, int* status, cudaStream_t st);

// gemm_simt.cu — Y[M][N] = X[M][K]·Wᵀ + bias (+GELU) (+residual[M][N]), fp32 CUDA cores.
int launch_gemm_q8_fp32(const QMat& w, const float* x, const float* bias, const float* residual, int epi,
                        float* y, int M, int ldy, cudaStream_t st);

// gemm_tc.cu — the same product on tcgen05 tensor cores (bf16 3-term split, fp32 TMEM
// accumulate). x_hi / x_lo are bf16 planes [M][K] made by launch_split_bf16; K % 64 == 0.
// `status` is a device int raised to FC_E_TIMEOUT when a bounded wait runs out.
int launch_split_bf16(const float* x, void* hi, void* lo, size_t n, cudaStream_t st);
int launch_gemm_q8_bf16x3(const QMat& w, const void* x_hi, const void* x_lo, const float* bias, const float* residual,
                          int epi, float* y, int M, int ldy, int* status, cudaStream_t st);
// The same with a choice of output: f32 rows y, or (y == nullptr) bf16 hi / lo planes for the next GEMM.
int launch_gemm_q8_bf16x3_ex(const QMat& w, const void* x_hi, const void* x_lo, const float* bias, const float* residual,
                             int epi, float* y, void* y_hi, void* y_lo, int M, int ldy, int* status, cudaStream_t st);

// The LM head fused with the statistics of the softmax tail (math mode FC_MATH_BF16X3): instead of logits the
// epilogue leaves, per (row, 128-column tile), the tile's largest logit, the sum of exp(logit - that) and the first
// column that attains it in stats [M][ceil(N / 128)] (16-byte records), and the logit of the row's target
// (targets[M], -1: none) in tlogit [M]. launch_score_combine folds the records of a row in tile order into
// ln(max(softmax(row)[target], 1e-12)) (f32 probability, f64 logarithm) and argmax_first(row) == target.
int launch_gemm_q8_bf16x3_score(const QMat& w, const void* x_hi, const void* x_lo, const int* targets, void* stats, float* tlogit,
                                int M, int* status, cudaStream_t st);
int launch_score_combine(const void* stats, const float* tlogit, const int* targets, int M, int n_tiles, int V, double* logprob,
                         uint8_t* is_greedy, cudaStream_t st);

// api.cu — the matrix and device behind a resident-weight handle.
const QMat* qweight_matrix(const fc_qweight* w, int* device);

// rowops.cu
int launch_embed_step(const QMat& tok, const float* pos_emb, int ctx, const int* queue, StepState* state,
                      float* x, cudaStream_t st);
int launch_embed_rows(const QMat& tok, const float* pos_emb, const int* ids, int R, int T, float* x,
                      int* error_flag, cudaStream_t st);
int launch_layernorm(const float* x, const float* g, const float* b, int rows, int d, float* y,
                     const StepState* state, cudaStream_t st);
// LayerNorm written as bf16 hi / lo planes [rows][d] for the tensor-core GEMM.
int launch_layernorm_planes(const float* x, const float* g, const float* b, int rows, int d, void* hi, void* lo, cudaStream_t st);
// Decode tail over logits[V]: softmax statistics, optional probs[V], optional greedy select
// (append to queue) — and always the end-of-step bookkeeping (pos, fed).
int launch_step_tail(const float* logits, int V, float* probs_or_null, int do_select, int* queue, int queue_cap,
                     StepState* state, float* sel_logit_or_null, cudaStream_t st);
// End-of-step bookkeeping alone (steps that skip the head).
int launch_step_advance(StepState* state, cudaStream_t st);
int launch_step_advance_pdl(StepState* state, cudaStream_t st);
// Scoring tail: per row of logits[R][ldl], target id (or -1) -> logprob, is_greedy.
// `status` (device int, may be null) is raised to FC_E_TIMEOUT when a bounded wait runs out.
int launch_score_rows(const float* logits, int ldl, int V, const int* targets, int R, double* logprob,
                      uint8_t* is_greedy, int* status, cudaStream_t st);
int launch_softmax_row(const float* logits, int V, float* probs, cudaStream_t st);
// sample.cu — one draw of sample_with_params on the device; see the kernel for the arguments.
int launch_sample(const float* in, int V, int from_probs, const fc_sampling& prm, const int* recent, int n_recent,
                  unsigned long long* rng_state, int* queue, int queue_cap, StepState* state, int* token_out, cudaStream_t st);

// Per-layer statistics of a window forward (the device-side counterpart of verbose.rs:85-110): one record per layer.
// Linear on a matrix kept in its GGML block format, decoded in the kernel (ggml_linear.cu): y[M][ldy] = [residual +] bias +
// x · dequant(W)ᵀ; rows of the same kind of table decoded by id (ids, or the queue entry at state->fed when ids is null).
int launch_ggml_linear(const fc_ggml_weight* w, const float* x, const float* bias, const float* residual, float* y, int ldy, int M,
                       cudaStream_t st);
int launch_ggml_rows(const fc_ggml_weight* w, const int* ids, StepState* state, const int* queue, int ctx, int R, float* x,
                     int* error_flag, cudaStream_t st);
int ggml_weight_rows(const fc_ggml_weight* w);
int ggml_weight_cols(const fc_ggml_weight* w);

// Per-row-scale int8 / int4 linear on a packed matrix (rowq.cu): y[M][ldy] = [residual +] bias + x · W; bias and residual may
// be null, residual may be y itself.
int launch_rowq_linear(fc_rowq* w, const float* x, const float* bias, const float* residual, float* y, int ldy, int M, cudaStream_t st);
int rowq_in(const fc_rowq* w);
int rowq_out(const fc_rowq* w);

struct LayerStatsDev {
    float min, max, mean, pad;
    long long nan_count, inf_count, n;
};
size_t layer_stats_scratch_bytes();
// x (f32), or (x == nullptr) bf16 hi / lo planes whose sum is the value; n elements; scratch: layer_stats_scratch_bytes().
int launch_layer_stats(const float* x, const void* hi, const void* lo, size_t n, void* scratch, LayerStatsDev* out, cudaStream_t st);

// attn.cu
int launch_attn_decode(const float* q, const float* kcache, const float* vcache, int d, int H, int ctx,
                       const StepState* state, float* out, cudaStream_t st);
// qkv [R][3d] (q | k | v per row), R = B·T, causal within each window of T rows.
int launch_attn_prefill(const float* qkv, int B, int T, int d, int H, float* out, cudaStream_t st);
// Grouped-query forms (llm.rs:305-341): H query heads share KV key/value heads of width hd.
// Decode: q [H*hd], caches [ctx][KV*hd]. Window: q, k, v rows ld floats apart, out rows ldo apart.
int launch_attn_decode_gqa(const float* q, const float* kcache, const float* vcache, int H, int KV, int hd, int ctx,
                           const StepState* state, float* out, cudaStream_t st);
int launch_attn_prefill_gqa(const float* q, const float* k, const float* v, int B, int T, int ld, int H, int KV, int hd,
                            int ldo, float* out, cudaStream_t st);
// attn_tc.cu — the same on tcgen05 (head_dim 64): bf16 hi / lo planes of qkv [B*T][3d] in,
// planes of the attention output [B*T][d] out; `status` is raised on a timeout.
int launch_attn_prefill_tc(const void* qkv_hi, const void* qkv_lo, int B, int T, int d, int H, void* out_hi, void* out_lo,
                           int* status, cudaStream_t st);
// Grouped-query form: planes [B*T][(H + 2 KV) * 64] in (q heads | k heads | v heads), [B*T][H * 64] out.
int launch_attn_prefill_tc_gqa(const void* qkv_hi, const void* qkv_lo, int B, int T, int H, int KV, void* out_hi, void* out_lo,
                               int* status, cudaStream_t st);

// decode_batch.cu — one lock-step decode step for S <= kBatchMaxStreams streams.
// Fragment-major copy of a Q8_0 matrix for the warp-level tensor-core product: per (16 rows,
// 32-wide block) 512 bytes of biased quants in lane order (q) and 8 pairs of f16 scales (d).
struct QFrag {
    const void* q = nullptr;
    const void* d = nullptr;
    int N = 0, K = 0, N_pad = 0;
};
constexpr int kBatchMaxStreams = 64;
size_t frag_quant_bytes(const QMat& w);
size_t frag_scale_bytes(const QMat& w);
int launch_repack_frag(const QMat& w, void* fq, void* fd, cudaStream_t st);
// Columns of the activation planes for S streams (two f16 rows per stream, padded to the MMA tiling).
int batch_cols(int S);
// Y = X · Wᵀ for S streams. xp: f16 rows [batch_cols(S)][K], row 2s = hi and row 2s + 1 = lo of stream s (rows past
// 2S zero).
// Where the result goes: f32 rows (optionally residual + result; residual may be y) and / or f16 hi / lo rows (after
// bias and epilogue), or raw partial sums part[splits][S][N] of K ranges (no bias; the consumer adds them in order,
// then the bias and the residual).
struct SkinnyOut {
    float* y = nullptr;
    int ldy = 0;
    const float* residual = nullptr;
    void* planes = nullptr;
    int ldp = 0;
    float* part = nullptr;
    int max_warps = 16;   // warps per CTA; 8 when several chains of step kernels share the GPU (two or three CTAs per SM then)
    bool long_k_block = true;   // 32 warps on the 16-row tile for long K (up to 16 streams); off when more than two chains share the GPU
};
int skinny_max_splits();
int launch_skinny_q8(const QFrag& w, int S, const void* xp, const float* bias, int epi, const SkinnyOut& out, int* splits_used,
                     cudaStream_t st);
int launch_embed_batch(const QMat& tok, const float* pos_emb, const int* cur, const int* pos, int S, float* x, cudaStream_t st);
// LayerNorm rows as f16 hi / lo rows; with partials (part != null) the row is first completed, x_new = x + (sum of the
// n_part partial products part[n_part][S][d] + part_bias), and stored to x_out.
int launch_ln_rows_f16(const float* x, const float* part, int n_part, const float* part_bias, float* x_out, const float* g,
                       const float* b, int S, int d, void* xp, cudaStream_t st);
// qkv [S][3d] of this step; kcs / vcs: per-stream cache base pointers (device array), layer_off floats into each.
int launch_attn_decode_batch(const float* qkv, float* const* kcs, float* const* vcs, size_t layer_off, int d, int H, int ctx,
                             const int* pos, int S, void* ap, cudaStream_t st);
int launch_pick_batch(const float* logits, int ldl, int V, int S, int eos, int* cur, int* done, int* n_out, int* out, int out_cap,
                      int* pos, int advance, cudaStream_t st);
int launch_scatter_kv(const float* qkv, float* const* kcs, float* const* vcs, size_t layer_off, int S, int n, int d, cudaStream_t st);
int launch_gather_last_rows(const float* x, int S, int n, int d, float* out, cudaStream_t st);
int launch_batch_init(int S, int pos0, int* done, int* n_out, int* cur, int* pos, cudaStream_t st);
int launch_gather_first(int* const* queues, StepState* const* states, int prompt_len, int S, int* cur, int* done, int* n_out,
                        int* out, int out_cap, int* pos, cudaStream_t st);

}  // namespace fc
