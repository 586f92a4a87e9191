// C ABI of the imported Llama / Qwen decoder (ferrum_core/src/llm.rs, llm_score.rs) on the
// Q8_0 kernels of this library: upload, the full-sequence forward and exact log-softmax
// scorer, and the KV-cached decode driver with on-device sampling.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include "llama_native.h"
#include "llama_ops.cuh"

using namespace fc;

namespace {

struct LlamaLayerDev {
    QMat qkv, wo, gateup, down;      // wq|wk|wv rows fused; gate and up rows interleaved (g0, u0, g1, u1, ...)
    float* qkv_b = nullptr;          // fused q|k|v bias, or null when the file has none
    float *attn_norm = nullptr, *ffn_norm = nullptr;
};

}  // namespace

struct fc_llama {
    fc_llama_config cfg;
    int device = 0;
    cudaStream_t st = nullptr;
    Arena arena, ws_arena;
    QMat tok, head;
    float* out_norm = nullptr;
    float2* ftab = nullptr;          // per rotary pair: {frequency, frequency divisor}
    float inv_linear = 1.0f;
    std::vector<LlamaLayerDev> layers;
    int q_dim = 0, kv_dim = 0, qkv_dim = 0;
    // window-forward workspace for ws_rows rows
    int ws_rows = 0, head_chunk = 0;
    float *x = nullptr, *n = nullptr, *qkv = nullptr, *att = nullptr, *gu = nullptr, *hid = nullptr, *logits = nullptr;
    int *ids_d = nullptr, *targets_d = nullptr, *err_d = nullptr, *tc_status = nullptr;
    double* lp_d = nullptr;
    uint8_t* gr_d = nullptr;
    uint16_t *xhi = nullptr, *xlo = nullptr;
    uint16_t *qkvhi = nullptr, *qkvlo = nullptr, *atthi = nullptr, *attlo = nullptr;   // planes around the tensor-core attention
    uint16_t *hidhi = nullptr, *hidlo = nullptr;                                       // gated hidden state, written by the gate/up GEMM
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_score_ms = 0.0f;
    bool force_fp32 = false;         // the batched prime keeps the cache rows at fp32 rounding
    // prec < 0: the Q8_0 matrices above are what runs. FC_Q_INT8 / FC_Q_INT4: every Linear packed as the reference's
    // importer packs it (Gguf::load_llama(kind), gguf/llama.rs:13-27,164-171) to a per-input-row QWeight, run by
    // ops::qlinear. kNative: every matrix kept in the file's own block format and decoded inside the product, which is
    // the reference's f32 import (load_llama_prec(None), gguf/llama.rs:171-176) without the expansion; no Q8_0 copies.
    static constexpr int kNative = 2;
    int prec = -1;
    struct Lin {                      // one Linear of the packed / native model: exactly one of the two is set
        fc_rowq* rq = nullptr;
        fc_ggml_weight* gw = nullptr;
    };
    struct PackedLayer { Lin wq, wk, wv, wo, gate, up, down; };
    std::vector<PackedLayer> packed;
    Lin packed_head;
    fc_ggml_weight* native_tok = nullptr;   // the embedding table in its block format (kNative)
};

struct fc_llama_cache {
    fc_llama* m = nullptr;
    int device = 0;                       // kept here so that freeing does not read the model
    Arena arena;
    float *kc = nullptr, *vc = nullptr;   // [L][ctx][kv_dim]
    float *x = nullptr, *n = nullptr, *qkv = nullptr, *att = nullptr, *gu = nullptr, *hid = nullptr, *logits = nullptr;
    int* queue = nullptr;
    int queue_cap = 0;
    StepState* state = nullptr;
    int* status = nullptr;                // raised by a kernel whose bounded wait ran out
    int host_pos = 0;
    cudaGraphExec_t graph[2] = {nullptr, nullptr};   // [0]: step without the head, [1]: with it
    int graph_nodes[2] = {0, 0};
    bool packed_warm[2] = {false, false};   // packed model: the uncaptured first step of each kind has run
    unsigned long long* rng_d = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_decode_ms = 0.0f;
};

namespace {

constexpr size_t q8_row_bytes(int K) { return (size_t)(K / 32) * 34; }

// Rows of several raw Q8_0 tensors with the same row length, one after the other.
int upload_fused(Arena& ar, std::initializer_list<std::pair<const void*, int>> parts, int K, QMat* out, cudaStream_t st) {
    if (K <= 0 || K % 32) return fail(FC_E_FORMAT, "Q8_0 row length %d must be a positive multiple of 32", K);
    size_t rows = 0;
    for (auto& p : parts) {
        if (!p.first) return fail(FC_E_FORMAT, "a required Q8_0 tensor is null");
        rows += (size_t)p.second;
    }
    std::vector<uint8_t> buf(rows * q8_row_bytes(K));
    size_t at = 0;
    for (auto& p : parts) {
        const size_t bytes = (size_t)p.second * q8_row_bytes(K);
        std::memcpy(buf.data() + at, p.first, bytes);
        at += bytes;
    }
    return upload_q8(ar, buf.data(), (int)rows, K, out, st);
}

// Rows of two raw Q8_0 tensors [rows][K] interleaved: a0, b0, a1, b1, ...
int upload_interleaved(Arena& ar, const void* a, const void* b, int rows, int K, QMat* out, cudaStream_t st) {
    if (!a || !b) return fail(FC_E_FORMAT, "a required Q8_0 tensor is null");
    if (K <= 0 || K % 32) return fail(FC_E_FORMAT, "Q8_0 row length %d must be a positive multiple of 32", K);
    const size_t rb = q8_row_bytes(K);
    std::vector<uint8_t> buf((size_t)2 * rows * rb);
    for (int r = 0; r < rows; ++r) {
        std::memcpy(buf.data() + (size_t)(2 * r) * rb, (const uint8_t*)a + (size_t)r * rb, rb);
        std::memcpy(buf.data() + (size_t)(2 * r + 1) * rb, (const uint8_t*)b + (size_t)r * rb, rb);
    }
    return upload_q8(ar, buf.data(), 2 * rows, K, out, st);
}

int gemm(fc_llama* m, const QMat& w, const float* x, const float* bias, const float* res, float* y, int M, int ldy) {
    if (m->cfg.math_mode == FC_MATH_BF16X3 && !m->force_fp32 && w.K % 64 == 0) {
        FC_TRY(launch_split_bf16(x, m->xhi, m->xlo, (size_t)M * w.K, m->st));
        return launch_gemm_q8_bf16x3(w, m->xhi, m->xlo, bias, res, EPI_NONE, y, M, ldy, m->tc_status, m->st);
    }
    return launch_gemm_q8_fp32(w, x, bias, res, EPI_NONE, y, M, ldy, m->st);
}

// The window attention runs on tcgen05 when the math mode allows it and heads are 64 wide (the
// rotated q | k | v rows are split into bf16 planes for it; its output planes feed the wo GEMM).
bool tensor_attention(const fc_llama* m) {
    return m->cfg.math_mode == FC_MATH_BF16X3 && m->cfg.head_dim == 64 && m->cfg.d_model % 64 == 0;
}

int ensure_workspace(fc_llama* m, int rows) {
    if (rows <= m->ws_rows) return FC_OK;
    m->ws_arena.release();
    m->ws_rows = 0;
    const fc_llama_config& c = m->cfg;
    const size_t R = rows, d = c.d_model, F = c.d_ff;
    size_t chunk = ((size_t)1 << 28) / (size_t)m->head.N_pad;   // logits for head_chunk rows at a time (<= 1 GiB)
    chunk = std::max<size_t>(1, std::min<size_t>(chunk, R));
    Arena& a = m->ws_arena;
    FC_TRY(a.alloc_n(&m->x, R * d));
    FC_TRY(a.alloc_n(&m->n, R * d));
    FC_TRY(a.alloc_n(&m->qkv, R * (size_t)m->qkv_dim));
    FC_TRY(a.alloc_n(&m->att, R * (size_t)m->q_dim));
    FC_TRY(a.alloc_n(&m->gu, R * 2 * F));
    FC_TRY(a.alloc_n(&m->hid, R * F));
    FC_TRY(a.alloc_n(&m->logits, chunk * (size_t)m->head.N_pad));
    FC_TRY(a.alloc_n(&m->ids_d, R));
    FC_TRY(a.alloc_n(&m->targets_d, R));
    FC_TRY(a.alloc_n(&m->lp_d, R));
    FC_TRY(a.alloc_n(&m->gr_d, R));
    FC_TRY(a.alloc_n(&m->err_d, 1));
    FC_TRY(a.alloc_n(&m->tc_status, 1));
    FC_CUDA(cudaMemsetAsync(m->tc_status, 0, sizeof(int), m->st));
    if (c.math_mode == FC_MATH_BF16X3) {
        const size_t widest = std::max({d, F, (size_t)m->q_dim});
        FC_TRY(a.alloc_n(&m->xhi, R * widest));
        FC_TRY(a.alloc_n(&m->xlo, R * widest));
        if (d % 64 == 0 && F % 64 == 0) {
            FC_TRY(a.alloc_n(&m->hidhi, R * F));
            FC_TRY(a.alloc_n(&m->hidlo, R * F));
        }
        if (tensor_attention(m)) {
            FC_TRY(a.alloc_n(&m->qkvhi, R * (size_t)m->qkv_dim)); FC_TRY(a.alloc_n(&m->qkvlo, R * (size_t)m->qkv_dim));
            FC_TRY(a.alloc_n(&m->atthi, R * (size_t)m->q_dim));   FC_TRY(a.alloc_n(&m->attlo, R * (size_t)m->q_dim));
        }
    }
    m->ws_rows = rows;
    m->head_chunk = (int)chunk;
    return FC_OK;
}

// LlamaModel::forward_tokens (llm.rs:622-635) up to the final norm, for B windows of T rows
// whose ids are in m->ids_d: every row r sits at position r % T. Leaves RMSNorm(h) in m->n.
// With `fill` (B == 1) the rotated keys and the values of every block become the cache's rows 0..T-1.
int forward_rows_packed(fc_llama* m, int B, int T, fc_llama_cache* fill);
int forward_rows(fc_llama* m, int B, int T, fc_llama_cache* fill = nullptr) {
    if (m->prec >= 0) return forward_rows_packed(m, B, T, fill);
    const fc_llama_config& c = m->cfg;
    const int R = B * T, d = c.d_model, F = c.d_ff;
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemsetAsync(m->err_d, 0, sizeof(int), st));
    FC_TRY(launch_llama_embed_rows(m->tok, m->ids_d, R, m->x, m->err_d, st));
    for (int l = 0; l < c.n_layer; ++l) {
        const LlamaLayerDev& L = m->layers[l];
        // LlamaBlock::forward_full (llm.rs:464-482)
        const bool planes = m->cfg.math_mode == FC_MATH_BF16X3 && !m->force_fp32 && d % 64 == 0 && F % 64 == 0;
        if (planes) {
            // norms and the gate write the planes the next GEMM reads: no f32 copy of them, no split pass
            FC_TRY(launch_llama_rmsnorm_planes(m->x, L.attn_norm, c.norm_eps, R, d, m->xhi, m->xlo, st));
            FC_TRY(launch_gemm_q8_bf16x3(L.qkv, m->xhi, m->xlo, L.qkv_b, nullptr, EPI_NONE, m->qkv, R, m->qkv_dim, m->tc_status, st));
        } else {
            FC_TRY(launch_llama_rmsnorm(m->x, L.attn_norm, c.norm_eps, R, d, m->n, nullptr, st));
            FC_TRY(gemm(m, L.qkv, m->n, L.qkv_b, nullptr, m->qkv, R, m->qkv_dim));
        }
        const bool tc_attn = tensor_attention(m) && !m->force_fp32 && !fill && (size_t)m->qkv_dim * 4 <= 48 * 1024;
        if (tc_attn) {
            // rotate and split in one pass: the attention reads planes, nothing reads the rotated f32 rows
            FC_TRY(launch_llama_rope_planes(m->qkv, R, m->qkv_dim, T, c.n_head, c.n_kv_head, m->q_dim, c.head_dim, c.rope_dim,
                                            c.rope_type == FC_ROPE_NEOX, m->ftab, m->inv_linear, m->qkvhi, m->qkvlo, st));
        } else {
            FC_TRY(launch_llama_rope_rows(m->qkv, R, m->qkv_dim, T, c.n_head, c.n_kv_head, m->q_dim, c.head_dim, c.rope_dim,
                                          c.rope_type == FC_ROPE_NEOX, m->ftab, m->inv_linear, st));
        }
        if (fill) {
            const size_t layer_stride = (size_t)c.ctx * m->kv_dim;
            FC_TRY(launch_llama_store_kv_rows(m->qkv, R, m->qkv_dim, m->q_dim, m->kv_dim, fill->kc + l * layer_stride,
                                              fill->vc + l * layer_stride, st));
        }
        if (tc_attn) {
            FC_TRY(launch_attn_prefill_tc_gqa(m->qkvhi, m->qkvlo, B, T, c.n_head, c.n_kv_head, m->atthi, m->attlo, m->tc_status, st));
            FC_TRY(launch_gemm_q8_bf16x3(L.wo, m->atthi, m->attlo, nullptr, m->x, EPI_NONE, m->x, R, d, m->tc_status, st));
        } else {
            FC_TRY(launch_attn_prefill_gqa(m->qkv, m->qkv + m->q_dim, m->qkv + m->q_dim + m->kv_dim, B, T, m->qkv_dim, c.n_head,
                                           c.n_kv_head, c.head_dim, m->q_dim, m->att, st));
            FC_TRY(gemm(m, L.wo, m->att, nullptr, m->x, m->x, R, d));
        }
        if (planes) {
            FC_TRY(launch_llama_rmsnorm_planes(m->x, L.ffn_norm, c.norm_eps, R, d, m->xhi, m->xlo, st));
            // the gate is the GEMM's epilogue: interleaved (gate, up) columns -> planes of the gated hidden state
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.gateup, m->xhi, m->xlo, nullptr, nullptr, EPI_SWIGLU, nullptr, m->hidhi, m->hidlo, R, F,
                                            m->tc_status, st));
            FC_TRY(launch_gemm_q8_bf16x3(L.down, m->hidhi, m->hidlo, nullptr, m->x, EPI_NONE, m->x, R, d, m->tc_status, st));
        } else {
            FC_TRY(launch_llama_rmsnorm(m->x, L.ffn_norm, c.norm_eps, R, d, m->n, nullptr, st));
            FC_TRY(gemm(m, L.gateup, m->n, nullptr, nullptr, m->gu, R, 2 * F));
            FC_TRY(launch_llama_swiglu(m->gu, R, F, m->hid, nullptr, st));
            FC_TRY(gemm(m, L.down, m->hid, nullptr, m->x, m->x, R, d));
        }
    }
    return launch_llama_rmsnorm(m->x, m->out_norm, c.norm_eps, R, d, m->n, nullptr, st);
}

int lin_apply(const fc_llama::Lin& l, const float* x, const float* bias, const float* residual, float* y, int ldy, int M, cudaStream_t st) {
    return l.rq ? launch_rowq_linear(l.rq, x, bias, residual, y, ldy, M, st) : launch_ggml_linear(l.gw, x, bias, residual, y, ldy, M, st);
}

// FeedForward::forward (llm.rs:417-428) on separate gate and up rows: h = silu(gate) * up.
__global__ void silu_mul_kernel(const float* __restrict__ g, const float* __restrict__ u, size_t n, float* __restrict__ h) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float a = g[i];
        h[i] = __fmul_rn(__fdiv_rn(a, __fadd_rn(1.0f, expf(-a))), u[i]);
    }
}
int launch_silu_mul(const float* g, const float* u, size_t n, float* h, cudaStream_t st) {
    const size_t want = (n + 255) / 256;
    silu_mul_kernel<<<(unsigned)std::min<size_t>(std::max<size_t>(want, 1), 148 * 8), 256, 0, st>>>(g, u, n, h);
    FC_LAUNCHED();
    return FC_OK;
}

// One block of the packed model on R rows: LlamaBlock::forward_full / forward_one (llm.rs:451-482) with every
// Linear an ops::qlinear (ops.rs:316-377). x: residual stream [R][d]; n: scratch [R][d]; qkv: [R][qkv_dim]; att:
// [R][q_dim]; gu: [R][2 F] (gate rows, then up rows); hid: [R][F]. `attend` runs between the projections and wo.
template <class Attend>
int packed_block(fc_llama* m, int l, int R, float* x, float* n, float* qkv, float* att, float* gu, float* hid,
                 const StepState* state, Attend attend) {
    const fc_llama_config& c = m->cfg;
    const LlamaLayerDev& L = m->layers[l];
    const fc_llama::PackedLayer& P = m->packed[l];
    const int d = c.d_model, F = c.d_ff;
    cudaStream_t st = m->st;
    FC_TRY(launch_llama_rmsnorm(x, L.attn_norm, c.norm_eps, R, d, n, state, st));
    const float* b = L.qkv_b;
    FC_TRY(lin_apply(P.wq, n, b, nullptr, qkv, m->qkv_dim, R, st));
    FC_TRY(lin_apply(P.wk, n, b ? b + m->q_dim : nullptr, nullptr, qkv + m->q_dim, m->qkv_dim, R, st));
    FC_TRY(lin_apply(P.wv, n, b ? b + m->q_dim + m->kv_dim : nullptr, nullptr, qkv + m->q_dim + m->kv_dim, m->qkv_dim, R, st));
    FC_TRY(attend());
    FC_TRY(lin_apply(P.wo, att, nullptr, x, x, d, R, st));
    FC_TRY(launch_llama_rmsnorm(x, L.ffn_norm, c.norm_eps, R, d, n, state, st));
    FC_TRY(lin_apply(P.gate, n, nullptr, nullptr, gu, F, R, st));
    FC_TRY(lin_apply(P.up, n, nullptr, nullptr, gu + (size_t)R * F, F, R, st));
    FC_TRY(launch_silu_mul(gu, gu + (size_t)R * F, (size_t)R * F, hid, st));
    return lin_apply(P.down, hid, nullptr, x, x, d, R, st);
}

int forward_rows_packed(fc_llama* m, int B, int T, fc_llama_cache* fill) {
    const fc_llama_config& c = m->cfg;
    const int R = B * T, d = c.d_model;
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemsetAsync(m->err_d, 0, sizeof(int), st));
    if (m->native_tok) FC_TRY(launch_ggml_rows(m->native_tok, m->ids_d, nullptr, nullptr, c.ctx, R, m->x, m->err_d, st));
    else FC_TRY(launch_llama_embed_rows(m->tok, m->ids_d, R, m->x, m->err_d, st));
    for (int l = 0; l < c.n_layer; ++l) {
        FC_TRY(packed_block(m, l, R, m->x, m->n, m->qkv, m->att, m->gu, m->hid, nullptr, [&]() -> int {
            FC_TRY(launch_llama_rope_rows(m->qkv, R, m->qkv_dim, T, c.n_head, c.n_kv_head, m->q_dim, c.head_dim, c.rope_dim,
                                          c.rope_type == FC_ROPE_NEOX, m->ftab, m->inv_linear, st));
            if (fill) {
                const size_t layer_stride = (size_t)c.ctx * m->kv_dim;
                FC_TRY(launch_llama_store_kv_rows(m->qkv, R, m->qkv_dim, m->q_dim, m->kv_dim, fill->kc + l * layer_stride,
                                                  fill->vc + l * layer_stride, st));
            }
            return launch_attn_prefill_gqa(m->qkv, m->qkv + m->q_dim, m->qkv + m->q_dim + m->kv_dim, B, T, m->qkv_dim, c.n_head,
                                           c.n_kv_head, c.head_dim, m->q_dim, m->att, st);
        }));
    }
    return launch_llama_rmsnorm(m->x, m->out_norm, c.norm_eps, R, d, m->n, nullptr, st);
}

int check_ids(const fc_llama* m, const int32_t* ids, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (ids[i] < 0 || ids[i] >= m->cfg.vocab) return fail(FC_E_DIM, "token %d ≥ vocab_size %d", ids[i], m->cfg.vocab);
    return FC_OK;
}

int check_status(fc_llama* m) {
    int err = 0, status = 0;
    FC_CUDA(cudaMemcpyAsync(&err, m->err_d, sizeof(int), cudaMemcpyDeviceToHost, m->st));
    FC_CUDA(cudaMemcpyAsync(&status, m->tc_status, sizeof(int), cudaMemcpyDeviceToHost, m->st));
    FC_CUDA(cudaStreamSynchronize(m->st));
    if (status != 0) {
        cudaMemsetAsync(m->tc_status, 0, sizeof(int), m->st);
        return fail(FC_E_TIMEOUT, "a bounded wait inside a tensor-core kernel ran out (status %d)", status);
    }
    if (err != 0) return fail(err, "a token id was rejected on the device");
    return FC_OK;
}

// Head + scoring tail over the R rows whose normalised state is in m->n; targets in m->targets_d.
int score_tail(fc_llama* m, int R) {
    const int d = m->cfg.d_model, ldl = m->head.N_pad;
    for (int r0 = 0; r0 < R; r0 += m->head_chunk) {
        const int rows = std::min(m->head_chunk, R - r0);
        if (m->prec >= 0) FC_TRY(lin_apply(m->packed_head, m->n + (size_t)r0 * d, nullptr, nullptr, m->logits, ldl, rows, m->st));
        else FC_TRY(gemm(m, m->head, m->n + (size_t)r0 * d, nullptr, nullptr, m->logits, rows, ldl));
        FC_TRY(launch_llama_score_rows(m->logits, ldl, m->cfg.vocab, m->targets_d + r0, rows, m->lp_d + r0, m->gr_d + r0, m->st));
    }
    return FC_OK;
}

// plan_windows (llm_score.rs:21-32).
struct Window { int start, first, end; };
void plan_windows(int n, int window, int from, std::vector<Window>* out) {
    const int half = std::max(window / 2, 1);
    int next = std::max(from, 1);
    while (next < n) {
        const int start = next <= window ? 0 : next - half;
        const int end = std::min(start + window + 1, n);
        out->push_back({start, next, end});
        next = end;
    }
}

int check_window(const fc_llama* m, int window) {
    if (window < 2 || window > m->cfg.ctx)
        return fail(FC_E_DIM, "window must be between 2 and the model's context length %d (got %d)", m->cfg.ctx, window);
    return FC_OK;
}

// ---------------------------------------------------------------------------- decode step
// LlamaModel::forward_one (llm.rs:610-618) -> LlamaBlock::forward_one (llm.rs:451-461) as a
// kernel sequence; every per-step quantity is read from device state so the captured graph is
// replayed unchanged.
int launch_step(fc_llama_cache* s, int with_head) {
    fc_llama* m = s->m;
    const fc_llama_config& c = m->cfg;
    cudaStream_t st = m->st;
    const size_t layer_stride = (size_t)c.ctx * m->kv_dim;
    FC_TRY(launch_llama_embed_step(m->tok, c.ctx, s->queue, s->state, s->x, st));
    for (int l = 0; l < c.n_layer; ++l) {
        const LlamaLayerDev& L = m->layers[l];
        float* kc = s->kc + l * layer_stride;
        float* vc = s->vc + l * layer_stride;
        // RMSNorm rides in the prologue of the projection that reads it, SwiGLU in the epilogue of gate/up
        FC_TRY(launch_gemv_q8_stream(L.qkv, s->x, L.attn_norm, c.norm_eps, L.qkv_b, nullptr, EPI_NONE, s->qkv, s->state, s->status, st));
        FC_TRY(launch_llama_attn_decode(s->qkv, c.n_head, c.n_kv_head, c.head_dim, c.rope_dim, c.rope_type == FC_ROPE_NEOX, m->ftab,
                                        m->inv_linear, kc, vc, c.ctx, s->state, s->att, st));
        FC_TRY(launch_gemv_q8_stream(L.wo, s->att, nullptr, 0.0f, nullptr, s->x, EPI_NONE, s->x, s->state, s->status, st));
        FC_TRY(launch_gemv_q8_stream(L.gateup, s->x, L.ffn_norm, c.norm_eps, nullptr, nullptr, EPI_SWIGLU, s->hid, s->state, s->status, st));
        FC_TRY(launch_gemv_q8_stream(L.down, s->hid, nullptr, 0.0f, nullptr, s->x, EPI_NONE, s->x, s->state, s->status, st));
    }
    if (with_head)
        FC_TRY(launch_gemv_q8_stream(m->head, s->x, m->out_norm, c.norm_eps, nullptr, nullptr, EPI_NONE, s->logits, s->state, s->status, st));
    return launch_step_advance_pdl(s->state, st);
}

// The same step on the packed model, one kernel per operation. The first step of a cache runs uncaptured, so that the
// packed linears' single-row scratch exists before the step is captured.
int launch_step_packed(fc_llama_cache* s, int with_head) {
    fc_llama* m = s->m;
    const fc_llama_config& c = m->cfg;
    cudaStream_t st = m->st;
    const size_t layer_stride = (size_t)c.ctx * m->kv_dim;
    if (m->native_tok) FC_TRY(launch_ggml_rows(m->native_tok, nullptr, s->state, s->queue, c.ctx, 1, s->x, nullptr, st));
    else FC_TRY(launch_llama_embed_step(m->tok, c.ctx, s->queue, s->state, s->x, st));
    for (int l = 0; l < c.n_layer; ++l) {
        float* kc = s->kc + l * layer_stride;
        float* vc = s->vc + l * layer_stride;
        FC_TRY(packed_block(m, l, 1, s->x, s->n, s->qkv, s->att, s->gu, s->hid, nullptr, [&]() -> int {
            return launch_llama_attn_decode(s->qkv, c.n_head, c.n_kv_head, c.head_dim, c.rope_dim, c.rope_type == FC_ROPE_NEOX, m->ftab,
                                            m->inv_linear, kc, vc, c.ctx, s->state, s->att, st);
        }));
    }
    if (with_head) {
        FC_TRY(launch_llama_rmsnorm(s->x, m->out_norm, c.norm_eps, 1, c.d_model, s->n, nullptr, st));
        FC_TRY(lin_apply(m->packed_head, s->n, nullptr, nullptr, s->logits, m->head.N_pad, 1, st));
    }
    return launch_step_advance_pdl(s->state, st);
}

int run_step(fc_llama_cache* s, int with_head) {
    const bool packed = s->m->prec >= 0;
    if (packed && !s->packed_warm[with_head]) {
        s->packed_warm[with_head] = true;
        return launch_step_packed(s, with_head);
    }
    if (!s->graph[with_head]) {
        cudaStream_t st = s->m->st;
        cudaGraph_t g = nullptr;
        const int64_t before = g_launches;
        FC_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        const int rc = packed ? launch_step_packed(s, with_head) : launch_step(s, with_head);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        s->graph_nodes[with_head] = (int)(g_launches - before);
        g_launches = before;
        if (rc != FC_OK) { if (g) cudaGraphDestroy(g); return rc; }
        FC_CUDA(e);
        const cudaError_t ei = cudaGraphInstantiate(&s->graph[with_head], g, 0);
        cudaGraphDestroy(g);
        FC_CUDA(ei);
    }
    FC_CUDA(cudaGraphLaunch(s->graph[with_head], s->m->st));
    g_launches += s->graph_nodes[with_head];
    return FC_OK;
}

__global__ void llama_set_state_kernel(StepState* st, int pos, int fed, int tail) {
    st->pos = pos; st->fed = fed; st->tail = tail; st->done = 0; st->eos = -1; st->error = 0;
}

int read_state(fc_llama_cache* s, StepState* out) {
    int status = 0;
    FC_CUDA(cudaMemcpyAsync(out, s->state, sizeof(StepState), cudaMemcpyDeviceToHost, s->m->st));
    FC_CUDA(cudaMemcpyAsync(&status, s->status, sizeof(int), cudaMemcpyDeviceToHost, s->m->st));
    FC_CUDA(cudaStreamSynchronize(s->m->st));
    if (status != 0) {
        cudaMemsetAsync(s->status, 0, sizeof(int), s->m->st);
        return fail(FC_E_TIMEOUT, "a bounded wait inside the streaming GEMV ran out (status %d)", status);
    }
    return FC_OK;
}

// Queues ids behind what the queue holds and feeds them; the last one with the head when asked.
int feed_ids(fc_llama_cache* s, const int32_t* ids, int n, int head_on_last) {
    fc_llama* m = s->m;
    if (s->host_pos + n > m->cfg.ctx)
        return fail(FC_E_DIM, "%d more tokens do not fit the model's %d-token context window (position %d)", n, m->cfg.ctx, s->host_pos);
    FC_CUDA(cudaMemcpyAsync(s->queue + s->host_pos, ids, (size_t)n * 4, cudaMemcpyHostToDevice, m->st));
    llama_set_state_kernel<<<1, 1, 0, m->st>>>(s->state, s->host_pos, s->host_pos, s->host_pos + n);
    FC_LAUNCHED();
    for (int i = 0; i < n; ++i) FC_TRY(run_step(s, head_on_last && i + 1 == n));
    s->host_pos += n;
    return FC_OK;
}

// The prompt of an empty cache as one fp32 window forward instead of n decode steps: the same
// cache rows and last-row logits to fp32 rounding (the order of the sums differs), at a fraction of
// the launches. Short prompts keep the step path.
constexpr int kPrimeBatchMin = 8;
int prime_window(fc_llama_cache* s, const int32_t* ids, int n) {
    fc_llama* m = s->m;
    const fc_llama_config& c = m->cfg;
    if (n > c.ctx) return fail(FC_E_DIM, "%d tokens do not fit the model's %d-token context window", n, c.ctx);
    FC_TRY(ensure_workspace(m, n));
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemcpyAsync(m->ids_d, ids, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    FC_CUDA(cudaMemcpyAsync(s->queue, ids, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    m->force_fp32 = true;
    const int rc = forward_rows(m, 1, n, s);
    m->force_fp32 = false;
    FC_TRY(rc);
    llama_set_state_kernel<<<1, 1, 0, st>>>(s->state, n, n, n);
    FC_LAUNCHED();
    // logits of the last row: the final norm was applied by forward_rows
    if (m->prec >= 0)
        FC_TRY(lin_apply(m->packed_head, m->n + (size_t)(n - 1) * c.d_model, nullptr, nullptr, s->logits, m->head.N_pad, 1, st));
    else
        FC_TRY(launch_gemv_q8_stream(m->head, m->n + (size_t)(n - 1) * c.d_model, nullptr, 0.0f, nullptr, nullptr, EPI_NONE, s->logits,
                                     s->state, s->status, st));
    FC_TRY(check_status(m));
    s->host_pos = n;
    return FC_OK;
}

}  // namespace

extern "C" {

// `matrices`: upload the Q8_0 matrices (false for the model that keeps them in their file formats).
static int create_impl(const fc_llama_config* cfg, const fc_llama_weights* w, int device, bool matrices, fc_llama** out) {
    if (!cfg || !w || !out || !w->layers) return fail(FC_E_ARG, "fc_llama_create: null argument");
    *out = nullptr;
    const fc_llama_config& c = *cfg;
    if (c.vocab <= 0 || c.d_model <= 0 || c.n_layer <= 0 || c.n_head <= 0 || c.head_dim <= 0 || c.d_ff <= 0 || c.ctx <= 0)
        return fail(FC_E_SHAPE, "fc_llama_create: non-positive dimension");
    // Attention::new (llm.rs:243-252)
    if (c.n_kv_head <= 0 || c.n_head % c.n_kv_head)
        return fail(FC_E_DIM, "n_heads %d must be a multiple of n_kv_heads %d", c.n_head, c.n_kv_head);
    if (c.rope_dim > c.head_dim || c.rope_dim < 0 || c.rope_dim % 2)
        return fail(FC_E_DIM, "rope_dim %d must be even and ≤ head_dim %d", c.rope_dim, c.head_dim);
    // RopeScaling::check (llm.rs:135-150)
    auto ok = [](float v) { return std::isfinite(v) && v > 0.0f; };
    if (!ok(c.rope_linear_factor)) return fail(FC_E_DIM, "RoPE scaling factors must be finite and > 0");
    if (w->rope_freqs)
        for (int i = 0; i < c.rope_dim / 2; ++i)
            if (!ok(w->rope_freqs[i])) return fail(FC_E_DIM, "RoPE scaling factors must be finite and > 0");
    if (c.rope_type != FC_ROPE_NORM && c.rope_type != FC_ROPE_NEOX) return fail(FC_E_ARG, "rope_type %d", c.rope_type);
    if (c.math_mode != FC_MATH_FP32 && c.math_mode != FC_MATH_BF16X3) return fail(FC_E_ARG, "math_mode %d", c.math_mode);
    if (c.head_dim > 256 || c.head_dim % 4) return fail(FC_E_SHAPE, "head_dim %d must be a multiple of 4, at most 256", c.head_dim);
    if (c.d_model % 32 || c.d_ff % 32 || (c.n_head * c.head_dim) % 32)
        return fail(FC_E_FORMAT, "d_model, d_ff and n_head * head_dim must be multiples of 32 for Q8_0 rows");
    FC_TRY(select_device(device));
    fc_llama* m = new fc_llama();
    m->cfg = c;
    m->device = device;
    m->q_dim = c.n_head * c.head_dim;
    m->kv_dim = c.n_kv_head * c.head_dim;
    m->qkv_dim = m->q_dim + 2 * m->kv_dim;
    auto build = [&]() -> int {
        FC_CUDA(cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking));
        FC_CUDA(cudaEventCreate(&m->ev0));
        FC_CUDA(cudaEventCreate(&m->ev1));
        cudaStream_t st = m->st;
        const int d = c.d_model, F = c.d_ff;
        if (matrices) {
            FC_TRY(upload_q8(m->arena, w->token_embd_q8, c.vocab, d, &m->tok, st));
            if (c.tied || !w->output_q8) m->head = m->tok;
            else FC_TRY(upload_q8(m->arena, w->output_q8, c.vocab, d, &m->head, st));
        } else {
            // only the shape of the head is used (the row stride of the logits)
            m->head.N = c.vocab; m->head.K = d; m->head.N_pad = (c.vocab + 127) & ~127;
            m->tok = m->head;
        }
        FC_TRY(upload_f32(m->arena, w->output_norm, d, &m->out_norm, st));
        // apply_rope (llm.rs:172): freq_i = (base as f64).powf(-2 i / rope_dim) as f32
        const int half = c.rope_dim / 2;
        std::vector<float2> ftab(std::max(half, 1));
        for (int i = 0; i < half; ++i) {
            ftab[i].x = (float)std::pow((double)c.rope_base, -2.0 * (double)i / (double)c.rope_dim);
            ftab[i].y = w->rope_freqs ? w->rope_freqs[i] : 1.0f;
        }
        FC_TRY(m->arena.alloc_n(&m->ftab, ftab.size()));
        FC_CUDA(cudaMemcpyAsync(m->ftab, ftab.data(), ftab.size() * sizeof(float2), cudaMemcpyHostToDevice, st));
        FC_CUDA(cudaStreamSynchronize(st));
        m->inv_linear = 1.0f / c.rope_linear_factor;
        m->layers.resize(c.n_layer);
        for (int l = 0; l < c.n_layer; ++l) {
            const fc_llama_layer& h = w->layers[l];
            LlamaLayerDev& L = m->layers[l];
            if (matrices) {
                FC_TRY(upload_fused(m->arena, {{h.wq_q8, m->q_dim}, {h.wk_q8, m->kv_dim}, {h.wv_q8, m->kv_dim}}, d, &L.qkv, st));
                FC_TRY(upload_q8(m->arena, h.wo_q8, d, m->q_dim, &L.wo, st));
                FC_TRY(upload_interleaved(m->arena, h.gate_q8, h.up_q8, F, d, &L.gateup, st));
                FC_TRY(upload_q8(m->arena, h.down_q8, d, F, &L.down, st));
            }
            FC_TRY(upload_f32(m->arena, h.attn_norm, d, &L.attn_norm, st));
            FC_TRY(upload_f32(m->arena, h.ffn_norm, d, &L.ffn_norm, st));
            if (h.bq || h.bk || h.bv) {
                std::vector<float> b((size_t)m->qkv_dim, 0.0f);
                if (h.bq) std::memcpy(b.data(), h.bq, (size_t)m->q_dim * 4);
                if (h.bk) std::memcpy(b.data() + m->q_dim, h.bk, (size_t)m->kv_dim * 4);
                if (h.bv) std::memcpy(b.data() + m->q_dim + m->kv_dim, h.bv, (size_t)m->kv_dim * 4);
                FC_TRY(upload_f32(m->arena, b.data(), b.size(), &L.qkv_b, st));
                FC_CUDA(cudaStreamSynchronize(st));
            }
        }
        FC_CUDA(cudaStreamSynchronize(st));
        return FC_OK;
    };
    const int rc = build();
    if (rc != FC_OK) { fc_llama_free(m); return rc; }
    *out = m;
    return FC_OK;
}

int fc_llama_create(const fc_llama_config* cfg, const fc_llama_weights* w, int device, fc_llama** out) {
    return create_impl(cfg, w, device, true, out);
}

// A Q8_0 tensor [n_out][n_in] as the reference's importer packs it: decoded (gguf/dequant.rs:37-49), transposed to
// Ferrum's [n_in][n_out] (gguf/llama.rs:143-144) and packed by QWeight::from_f32 (quant.rs:164-212), then uploaded.
static int pack_linear(int device, const void* q8, int n_out, int n_in, int kind, fc_rowq** out) {
    if (!q8) return fail(FC_E_FORMAT, "a required Q8_0 tensor is null");
    std::vector<float> w((size_t)n_out * n_in), t((size_t)n_out * n_in);
    FC_TRY(fc_q8_0_dequantize(q8, w.size(), w.data()));
    for (int o = 0; o < n_out; ++o)
        for (int i = 0; i < n_in; ++i) t[(size_t)i * n_out + o] = w[(size_t)o * n_in + i];
    std::vector<float> scales((size_t)n_in);
    std::vector<uint8_t> q(fc_rowq_packed_len(n_in, n_out, kind));
    FC_TRY(fc_rowq_from_f32(t.data(), n_in, n_out, kind, scales.data(), q.data()));
    return fc_rowq_upload(device, q.data(), scales.data(), n_in, n_out, kind, out);
}

int fc_llama_create_packed(const fc_llama_config* cfg, const fc_llama_weights* w, int device, int kind, fc_llama** out) {
    if (kind != FC_Q_INT8 && kind != FC_Q_INT4) return fail(FC_E_ARG, "fc_llama_create_packed: kind %d", kind);
    FC_TRY(fc_llama_create(cfg, w, device, out));
    fc_llama* m = *out;
    const fc_llama_config& c = m->cfg;
    auto build = [&]() -> int {
        m->packed.resize(c.n_layer);
        for (int l = 0; l < c.n_layer; ++l) {
            const fc_llama_layer& h = w->layers[l];
            fc_llama::PackedLayer& P = m->packed[l];
            FC_TRY(pack_linear(device, h.wq_q8, m->q_dim, c.d_model, kind, &P.wq.rq));
            FC_TRY(pack_linear(device, h.wk_q8, m->kv_dim, c.d_model, kind, &P.wk.rq));
            FC_TRY(pack_linear(device, h.wv_q8, m->kv_dim, c.d_model, kind, &P.wv.rq));
            FC_TRY(pack_linear(device, h.wo_q8, c.d_model, m->q_dim, kind, &P.wo.rq));
            FC_TRY(pack_linear(device, h.gate_q8, c.d_ff, c.d_model, kind, &P.gate.rq));
            FC_TRY(pack_linear(device, h.up_q8, c.d_ff, c.d_model, kind, &P.up.rq));
            FC_TRY(pack_linear(device, h.down_q8, c.d_model, c.d_ff, kind, &P.down.rq));
        }
        // the LM head: `output.weight`, or the token embedding transposed when tied (gguf/llama.rs:304-311)
        FC_TRY(pack_linear(device, (c.tied || !w->output_q8) ? w->token_embd_q8 : w->output_q8, c.vocab, c.d_model, kind, &m->packed_head.rq));
        m->prec = kind;
        return FC_OK;
    };
    const int rc = build();
    if (rc != FC_OK) { fc_llama_free(m); *out = nullptr; }
    return rc;
}

void fc_llama_free(fc_llama* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->st) cudaStreamSynchronize(m->st);
    auto drop = [](fc_llama::Lin& l) { fc_rowq_free(l.rq); fc_ggml_weight_free(l.gw); l = fc_llama::Lin(); };
    for (auto& P : m->packed)
        for (fc_llama::Lin* l : {&P.wq, &P.wk, &P.wv, &P.wo, &P.gate, &P.up, &P.down}) drop(*l);
    drop(m->packed_head);
    fc_ggml_weight_free(m->native_tok);
    m->ws_arena.release();
    m->arena.release();
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->st) cudaStreamDestroy(m->st);
    delete m;
}

int fc_llama_forward_tokens(fc_llama* m, const int32_t* ids, int n, float* logits) {
    if (!m || !ids || !logits) return fail(FC_E_ARG, "fc_llama_forward_tokens: null argument");
    if (n <= 0) return fail(FC_E_SHAPE, "fc_llama_forward_tokens: n = %d", n);
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, ids, (size_t)n));
    FC_TRY(ensure_workspace(m, n));
    const int d = m->cfg.d_model, V = m->cfg.vocab, ldl = m->head.N_pad;
    FC_CUDA(cudaMemcpyAsync(m->ids_d, ids, (size_t)n * 4, cudaMemcpyHostToDevice, m->st));
    FC_TRY(forward_rows(m, 1, n));
    for (int r0 = 0; r0 < n; r0 += m->head_chunk) {
        const int rows = std::min(m->head_chunk, n - r0);
        if (m->prec >= 0) FC_TRY(lin_apply(m->packed_head, m->n + (size_t)r0 * d, nullptr, nullptr, m->logits, ldl, rows, m->st));
        else FC_TRY(gemm(m, m->head, m->n + (size_t)r0 * d, nullptr, nullptr, m->logits, rows, ldl));
        FC_CUDA(cudaMemcpy2DAsync(logits + (size_t)r0 * V, (size_t)V * 4, m->logits, (size_t)ldl * 4, (size_t)V * 4, rows,
                                  cudaMemcpyDeviceToHost, m->st));
    }
    return check_status(m);
}

int fc_llama_score_from(fc_llama* m, const int32_t* ids, int n, int from, int window, fc_score* score, float* lp,
                        uint8_t* is_greedy) {
    if (!m || !ids || !score) return fail(FC_E_ARG, "fc_llama_score_from: null argument");
    if (n < 0 || from < 0) return fail(FC_E_SHAPE, "fc_llama_score_from: n = %d, from = %d", n, from);
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_window(m, window));
    FC_TRY(check_ids(m, ids, (size_t)n));
    score->logprob = 0.0; score->n_tokens = 0; score->greedy = 1;
    if (lp) std::fill(lp, lp + std::max(n - 1, 0), 0.0f);
    if (is_greedy) std::fill(is_greedy, is_greedy + std::max(n - 1, 0), (uint8_t)0);
    std::vector<Window> plan;
    plan_windows(n, window, from, &plan);
    if (plan.empty()) return FC_OK;
    FC_TRY(ensure_workspace(m, std::min(window, n)));
    m->last_score_ms = 0.0f;
    std::vector<int32_t> targets;
    std::vector<double> lps;
    std::vector<uint8_t> grs;
    for (const Window& wd : plan) {
        // the window feeds ids[start .. min(start + window, n)); row r predicts id start + r + 1
        const int rows = std::min(wd.start + window, n) - wd.start;
        targets.assign(rows, -1);
        for (int t = wd.first; t < wd.end; ++t) targets[t - 1 - wd.start] = ids[t];
        FC_CUDA(cudaMemcpyAsync(m->ids_d, ids + wd.start, (size_t)rows * 4, cudaMemcpyHostToDevice, m->st));
        FC_CUDA(cudaMemcpyAsync(m->targets_d, targets.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, m->st));
        FC_CUDA(cudaEventRecord(m->ev0, m->st));
        FC_TRY(forward_rows(m, 1, rows));
        FC_TRY(score_tail(m, rows));
        FC_CUDA(cudaEventRecord(m->ev1, m->st));
        lps.resize(rows); grs.resize(rows);
        FC_CUDA(cudaMemcpyAsync(lps.data(), m->lp_d, (size_t)rows * 8, cudaMemcpyDeviceToHost, m->st));
        FC_CUDA(cudaMemcpyAsync(grs.data(), m->gr_d, (size_t)rows, cudaMemcpyDeviceToHost, m->st));
        FC_TRY(check_status(m));
        float ms = 0.0f;
        FC_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
        m->last_score_ms += ms;
        for (int t = wd.first; t < wd.end; ++t) {           // ascending targets, f64 sum (llm_score.rs:88-93)
            const int r = t - 1 - wd.start;
            score->logprob += lps[r];
            score->n_tokens += 1;
            if (!grs[r]) score->greedy = 0;
            if (lp) lp[t - 1] = (float)lps[r];
            if (is_greedy) is_greedy[t - 1] = grs[r];
        }
    }
    return FC_OK;
}

int fc_llama_score_sequences(fc_llama* m, const int32_t* ids, int n_seq, int seq_len, int batch_windows, fc_score* scores,
                             float* lp) {
    if (!m || !ids || !scores) return fail(FC_E_ARG, "fc_llama_score_sequences: null argument");
    if (n_seq < 0 || seq_len < 2) return fail(FC_E_SHAPE, "fc_llama_score_sequences: n_seq = %d, seq_len = %d", n_seq, seq_len);
    if (seq_len > m->cfg.ctx) return fail(FC_E_DIM, "sequences of %d ids do not fit one window of %d", seq_len, m->cfg.ctx);
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, ids, (size_t)n_seq * seq_len));
    const int T = seq_len, Bmax = std::max(1, std::min(batch_windows > 0 ? batch_windows : 8, std::max(n_seq, 1)));
    FC_TRY(ensure_workspace(m, Bmax * T));
    m->last_score_ms = 0.0f;
    std::vector<int32_t> targets((size_t)Bmax * T);
    std::vector<double> lps((size_t)Bmax * T);
    std::vector<uint8_t> grs((size_t)Bmax * T);
    for (int s0 = 0; s0 < n_seq; s0 += Bmax) {
        const int B = std::min(Bmax, n_seq - s0), R = B * T;
        for (int b = 0; b < B; ++b) {
            const int32_t* seq = ids + (size_t)(s0 + b) * T;
            for (int t = 0; t < T; ++t) targets[(size_t)b * T + t] = t + 1 < T ? seq[t + 1] : -1;
        }
        FC_CUDA(cudaMemcpyAsync(m->ids_d, ids + (size_t)s0 * T, (size_t)R * 4, cudaMemcpyHostToDevice, m->st));
        FC_CUDA(cudaMemcpyAsync(m->targets_d, targets.data(), (size_t)R * 4, cudaMemcpyHostToDevice, m->st));
        FC_CUDA(cudaEventRecord(m->ev0, m->st));
        FC_TRY(forward_rows(m, B, T));
        FC_TRY(score_tail(m, R));
        FC_CUDA(cudaEventRecord(m->ev1, m->st));
        FC_CUDA(cudaMemcpyAsync(lps.data(), m->lp_d, (size_t)R * 8, cudaMemcpyDeviceToHost, m->st));
        FC_CUDA(cudaMemcpyAsync(grs.data(), m->gr_d, (size_t)R, cudaMemcpyDeviceToHost, m->st));
        FC_TRY(check_status(m));
        float ms = 0.0f;
        FC_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
        m->last_score_ms += ms;
        for (int b = 0; b < B; ++b) {
            fc_score& sc = scores[s0 + b];
            sc.logprob = 0.0; sc.n_tokens = 0; sc.greedy = 1;
            for (int t = 0; t + 1 < T; ++t) {
                const size_t r = (size_t)b * T + t;
                sc.logprob += lps[r];
                sc.n_tokens += 1;
                if (!grs[r]) sc.greedy = 0;
                if (lp) lp[(size_t)(s0 + b) * (T - 1) + t] = (float)lps[r];
            }
        }
    }
    return FC_OK;
}

float fc_llama_last_score_ms(const fc_llama* m) { return m ? m->last_score_ms : 0.0f; }

int fc_llama_cache_create(fc_llama* m, fc_llama_cache** out) {
    if (!m || !out) return fail(FC_E_ARG, "fc_llama_cache_create: null argument");
    *out = nullptr;
    FC_CUDA(cudaSetDevice(m->device));
    const fc_llama_config& c = m->cfg;
    fc_llama_cache* s = new fc_llama_cache();
    s->m = m;
    s->device = m->device;
    auto build = [&]() -> int {
        const size_t kv = (size_t)c.n_layer * c.ctx * m->kv_dim;
        Arena& a = s->arena;
        FC_TRY(a.alloc_n(&s->kc, kv));
        FC_TRY(a.alloc_n(&s->vc, kv));
        FC_TRY(a.alloc_n(&s->x, (size_t)c.d_model));
        FC_TRY(a.alloc_n(&s->n, (size_t)c.d_model));
        FC_TRY(a.alloc_n(&s->qkv, (size_t)m->qkv_dim));
        FC_TRY(a.alloc_n(&s->att, (size_t)m->q_dim));
        FC_TRY(a.alloc_n(&s->gu, (size_t)2 * c.d_ff));
        FC_TRY(a.alloc_n(&s->hid, (size_t)c.d_ff));
        FC_TRY(a.alloc_n(&s->logits, (size_t)m->head.N_pad));
        s->queue_cap = c.ctx + 1;
        FC_TRY(a.alloc_n(&s->queue, (size_t)s->queue_cap));
        FC_TRY(a.alloc_n(&s->state, 1));
        FC_TRY(a.alloc_n(&s->status, 1));
        FC_CUDA(cudaMemsetAsync(s->status, 0, sizeof(int), m->st));
        FC_TRY(a.alloc_n(&s->rng_d, 1));
        FC_CUDA(cudaEventCreate(&s->ev0));
        FC_CUDA(cudaEventCreate(&s->ev1));
        return fc_llama_cache_clear(s);
    };
    const int rc = build();
    if (rc != FC_OK) { fc_llama_cache_free(s); return rc; }
    *out = s;
    return FC_OK;
}

void fc_llama_cache_free(fc_llama_cache* s) {
    if (!s) return;
    cudaSetDevice(s->device);
    cudaDeviceSynchronize();              // the model (and its stream) may already be gone
    for (auto& g : s->graph) if (g) cudaGraphExecDestroy(g);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    s->arena.release();
    delete s;
}

int fc_llama_cache_clear(fc_llama_cache* s) {
    if (!s) return fail(FC_E_ARG, "fc_llama_cache_clear: null cache");
    FC_CUDA(cudaSetDevice(s->m->device));
    llama_set_state_kernel<<<1, 1, 0, s->m->st>>>(s->state, 0, 0, 0);
    FC_LAUNCHED();
    s->host_pos = 0;
    return FC_OK;
}

int fc_llama_cache_pos(const fc_llama_cache* s) { return s ? s->host_pos : 0; }

int fc_llama_forward_one(fc_llama_cache* s, int32_t token, float* logits) {
    if (!s) return fail(FC_E_ARG, "fc_llama_forward_one: null cache");
    fc_llama* m = s->m;
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, &token, 1));
    FC_TRY(feed_ids(s, &token, 1, logits != nullptr));
    if (logits) FC_CUDA(cudaMemcpyAsync(logits, s->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->st));
    StepState hs;
    FC_TRY(read_state(s, &hs));
    if (hs.error) { s->host_pos -= 1; return fail(hs.error, "the decode step rejected a token or position on the device"); }
    return FC_OK;
}

int fc_llama_prime(fc_llama_cache* s, const int32_t* ids, int n, float* logits) {
    if (!s || !ids) return fail(FC_E_ARG, "fc_llama_prime: null argument");
    if (n <= 0) return fail(FC_E_DIM, "prompt must be non-empty");
    fc_llama* m = s->m;
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, ids, (size_t)n));
    FC_TRY(fc_llama_cache_clear(s));
    if (n >= kPrimeBatchMin) FC_TRY(prime_window(s, ids, n));
    else FC_TRY(feed_ids(s, ids, n, 1));
    if (logits) FC_CUDA(cudaMemcpyAsync(logits, s->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, m->st));
    StepState hs;
    FC_TRY(read_state(s, &hs));
    if (hs.error) return fail(hs.error, "the decode step rejected a token or position on the device");
    return FC_OK;
}

int fc_llama_generate(fc_llama_cache* s, const int32_t* prompt, int n, int max_new, const fc_sampling* params,
                      const int32_t* stops, int n_stops, uint64_t* rng_state, const volatile int32_t* cancel,
                      int32_t* out, int* n_out) {
    if (!s || !prompt || !params || !rng_state || !n_out || (max_new > 0 && !out) || (n_stops > 0 && !stops))
        return fail(FC_E_ARG, "fc_llama_generate: null argument");
    *n_out = 0;
    if (n <= 0) return fail(FC_E_DIM, "prompt must be non-empty");
    if (max_new < 0 || n_stops < 0) return fail(FC_E_SHAPE, "fc_llama_generate: max_new = %d, n_stops = %d", max_new, n_stops);
    fc_llama* m = s->m;
    const fc_llama_config& c = m->cfg;
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, prompt, (size_t)n));
    // llm.rs:723-730: the context window bounds the prompt and the generation
    if (n >= c.ctx) return fail(FC_E_DIM, "prompt of %d tokens does not fit the model's %d-token context window", n, c.ctx);
    max_new = std::min(max_new, c.ctx - n);
    cudaStream_t st = m->st;
    if (cancel && *cancel) return FC_OK;                     // cancelled while reading the prompt: nothing (llm.rs:734-736)
    FC_TRY(fc_llama_cache_clear(s));
    FC_CUDA(cudaMemcpyAsync(s->rng_d, rng_state, 8, cudaMemcpyHostToDevice, st));
    if (n >= kPrimeBatchMin) FC_TRY(prime_window(s, prompt, n));
    else FC_TRY(feed_ids(s, prompt, n, 1));
    // greedy without a penalty needs neither the sampler's sort nor, without stop ids, the host
    const bool plain_greedy = params->temperature <= 0.0f && params->repetition_penalty == 1.0f;
    const bool free_run = plain_greedy && n_stops == 0 && !cancel;
    FC_CUDA(cudaEventRecord(s->ev0, st));
    int made = 0;
    int rc = FC_OK;
    bool cancelled = false, timed = false;
    while (made < max_new) {
        if (cancel && *cancel) { cancelled = true; break; }
        // recent = prompt + tokens so far = the queue (llm.rs:740-751)
        rc = plain_greedy ? launch_llama_pick(s->logits, c.vocab, s->queue, s->queue_cap, s->state, st)
                          : launch_sample(s->logits, c.vocab, 0, *params, s->queue, 0, s->rng_d, s->queue, s->queue_cap, s->state,
                                          nullptr, st);
        if (rc != FC_OK) break;
        ++made;
        bool stop = false;
        if (!free_run) {
            int32_t tok = 0;
            if (cudaMemcpyAsync(&tok, s->queue + n + made - 1, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
                cudaStreamSynchronize(st) != cudaSuccess) { rc = fail(FC_E_CUDA, "token download failed"); break; }
            out[made - 1] = tok;
            for (int i = 0; i < n_stops; ++i) stop |= stops[i] == tok;
        }
        if (stop) break;                                     // a stop id is kept in out and not fed (llm.rs:747-749)
        // the forward of the last requested token keeps the cache continuable (llm.rs:750-751); its logits are not used
        // here, so it stays outside the timed region
        if (made == max_new) { FC_CUDA(cudaEventRecord(s->ev1, st)); timed = true; }
        rc = run_step(s, 1);                                 // forward_one(next), the last token included (llm.rs:750-751)
        if (rc != FC_OK) break;
        s->host_pos += 1;
    }
    if (rc == FC_OK) {
        if (!timed) FC_CUDA(cudaEventRecord(s->ev1, st));
        if (free_run && made > 0) FC_CUDA(cudaMemcpyAsync(out, s->queue + n, (size_t)made * 4, cudaMemcpyDeviceToHost, st));
        StepState hs;
        rc = read_state(s, &hs);
        if (rc == FC_OK && hs.error) rc = fail(hs.error, "the decode step rejected a token or position on the device");
        if (rc == FC_OK) FC_CUDA(cudaEventElapsedTime(&s->last_decode_ms, s->ev0, s->ev1));
    }
    FC_CUDA(cudaMemcpy(rng_state, s->rng_d, 8, cudaMemcpyDeviceToHost));
    if (rc != FC_OK) return rc;
    *n_out = made;
    if (cancelled) return fail(FC_E_CANCELLED, "generation cancelled after %d tokens", made);
    return FC_OK;
}

float fc_llama_last_decode_ms(const fc_llama_cache* s) { return s ? s->last_decode_ms : 0.0f; }

}  // extern "C"

namespace fc {
int llama_create_native(const fc_llama_config* cfg, const fc_llama_weights* w, const RawTensor& tok, const RawTensor& output,
                        const RawLlamaLayer* layers, int device, fc_llama** out) {
    FC_TRY(create_impl(cfg, w, device, false, out));
    fc_llama* m = *out;
    const fc_llama_config& c = m->cfg;
    auto up = [&](const RawTensor& t, int n_out, int n_in, fc_ggml_weight** dst) -> int {
        if (!t.data) return fail(FC_E_FORMAT, "a required tensor is missing");
        return fc_ggml_weight_upload(device, t.type, t.data, t.nbytes, n_out, n_in, dst);
    };
    auto build = [&]() -> int {
        FC_TRY(up(tok, c.vocab, c.d_model, &m->native_tok));
        m->packed.resize(c.n_layer);
        for (int l = 0; l < c.n_layer; ++l) {
            const RawLlamaLayer& h = layers[l];
            fc_llama::PackedLayer& P = m->packed[l];
            FC_TRY(up(h.wq, m->q_dim, c.d_model, &P.wq.gw));
            FC_TRY(up(h.wk, m->kv_dim, c.d_model, &P.wk.gw));
            FC_TRY(up(h.wv, m->kv_dim, c.d_model, &P.wv.gw));
            FC_TRY(up(h.wo, c.d_model, m->q_dim, &P.wo.gw));
            FC_TRY(up(h.gate, c.d_ff, c.d_model, &P.gate.gw));
            FC_TRY(up(h.up, c.d_ff, c.d_model, &P.up.gw));
            FC_TRY(up(h.down, c.d_model, c.d_ff, &P.down.gw));
        }
        // the LM head: output.weight, or the embedding table itself when tied (gguf/llama.rs:304-311)
        FC_TRY(up((c.tied || !output.data) ? tok : output, c.vocab, c.d_model, &m->packed_head.gw));
        m->prec = fc_llama::kNative;
        return FC_OK;
    };
    const int rc = build();
    if (rc != FC_OK) { fc_llama_free(m); *out = nullptr; }
    return rc;
}
}  // namespace fc
