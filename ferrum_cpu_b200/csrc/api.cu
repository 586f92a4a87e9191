// C ABI of libferrum_cuda: model upload, the standalone Q8_0 linear, windowed scoring and
// the KV-cached decode driver. Host logic above the kernels mirrors, in C++, the Rust items
// cited in include/ferrum_cuda.h.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "fc_common.cuh"
#include "mega.cuh"

namespace fc {

// ------------------------------------------------------------------------------- errors
static thread_local char g_err[512] = "";
thread_local int64_t g_launches = 0;
DebugKnobs g_debug;

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}
const char* g_err_text() { return g_err; }
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}
int cuda_fail(cudaError_t e, const char* what, const char* file, int line) {
    snprintf(g_err, sizeof g_err, "CUDA error %d (%s) at %s:%d in %s", (int)e, cudaGetErrorString(e), file, line, what);
    return FC_E_CUDA;
}

// Refuses anything but a Blackwell data-centre part: there is no other code path.
int select_device(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(FC_E_CUDA, "no CUDA device is visible: libferrum_cuda has no CPU fallback");
    }
    if (device < 0 || device >= n) return fail(FC_E_ARG, "device %d out of range (0..%d)", device, n - 1);
    int major = 0;
    FC_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return fail(FC_E_CUDA, "device %d has compute capability %d.x; this library is built for sm_100a only", device, major);
    FC_CUDA(cudaSetDevice(device));
    return FC_OK;
}

int upload_f32(Arena& ar, const float* host, size_t n, float** dev, cudaStream_t st) {
    if (!host) return fail(FC_E_FORMAT, "a required f32 tensor is null");
    FC_TRY(ar.alloc_n(dev, n));
    FC_CUDA(cudaMemcpyAsync(*dev, host, n * sizeof(float), cudaMemcpyHostToDevice, st));
    return FC_OK;
}

// loader/mod.rs:147-154: a matrix is Q8_0 only when its row length is a multiple of 32.
int upload_q8(Arena& ar, const void* host, int N, int K, QMat* out, cudaStream_t st) {
    if (!host) return fail(FC_E_FORMAT, "a required Q8_0 tensor is null");
    if (N <= 0 || K <= 0 || K % 32) return fail(FC_E_FORMAT, "Q8_0 matrix [%d][%d]: row length must be a positive multiple of 32", N, K);
    if (K > 12288) return fail(FC_E_SHAPE, "row length %d exceeds the 12288 supported by the decode GEMV", K);
    const int N_pad = (N + kRowPad - 1) / kRowPad * kRowPad;
    const size_t raw_bytes = (size_t)N * (K / 32) * 34;
    uint8_t* raw = nullptr;
    uint8_t* qu = nullptr;
    __half* d = nullptr;
    FC_CUDA(cudaMalloc((void**)&raw, raw_bytes));
    int rc = ar.alloc_n(&qu, (size_t)N_pad * K);
    if (rc == FC_OK) rc = ar.alloc_n(&d, (size_t)N_pad * (K / 32));
    if (rc == FC_OK && cudaMemcpyAsync(raw, host, raw_bytes, cudaMemcpyHostToDevice, st) != cudaSuccess)
        rc = fail(FC_E_CUDA, "upload of a Q8_0 tensor failed");
    if (rc == FC_OK) rc = launch_repack_q8(raw, N, K, N_pad, qu, d, st);
    if (rc == FC_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(FC_E_CUDA, "repack of a Q8_0 tensor failed");
    cudaFree(raw);
    FC_TRY(rc);
    out->qu = qu; out->d = d; out->N = N; out->K = K; out->N_pad = N_pad;
    return FC_OK;
}

struct LayerDev {
    QMat qkv, out, up, down;
    float *qkv_b, *out_b, *up_b, *down_b, *ln1g, *ln1b, *ln2g, *ln2b;
};

}  // namespace fc

using namespace fc;

struct fc_qweight {
    int device;
    Arena arena;
    QMat w;
    // scratch of the tensor-core path: bf16 hi / lo planes of the activations, status word
    Arena planes;
    uint16_t *xhi = nullptr, *xlo = nullptr;
    int* status = nullptr;
    size_t plane_elems = 0;
};

namespace fc {
const QMat* qweight_matrix(const fc_qweight* w, int* device) {
    *device = w->device;
    return &w->w;
}
}  // namespace fc

// Per-CTA parameter tables of the persistent decode kernel for one grid size.
struct MegaTable {
    int grid = 0;
    int bias_pack = 0;
    fc::MegaLayer* layers = nullptr;
};

// Buffers of the lock-step decode of many streams (fc_decode_batch), for up to `cap` streams.
struct BatchCtx {
    Arena arena;                       // step buffers
    Arena frag_arena;                  // fragment-major weight copies, made on first use
    bool frags = false;
    std::vector<fc::QFrag> qkv, out, up, down;
    fc::QFrag head;
    int cap = 0, out_cap = 0;
    float *x = nullptr, *x2 = nullptr, *qkv_f = nullptr, *logits = nullptr;   // the residual stream alternates between x and x2
    float* part = nullptr;             // K-split partial sums of the out- and down-projections [splits][S][d]
    void *xp = nullptr, *ap = nullptr, *hp = nullptr;      // f16 hi / lo rows of LayerNorm output, attention output, GELU output
    int *cur = nullptr, *done = nullptr, *n_out = nullptr, *out_tok = nullptr, *pos = nullptr;
    float **kcs = nullptr, **vcs = nullptr;
    int** queues = nullptr;
    fc::StepState** states = nullptr;
    // one step, and four steps in a row (no gap between graph launches inside them), captured for
    // (graph_S, graph_eos, out_cap, graph_group)
    cudaGraphExec_t graph = nullptr, graph4 = nullptr;
    int graph_S = 0, graph_eos = 0, graph_cap = 0, graph_nodes = 0, graph4_nodes = 0, graph_group = 0;
    // the step graph runs groups of streams as parallel branches: branch g > 0 is captured on side[g - 1]
    std::vector<cudaStream_t> side;
    std::vector<cudaEvent_t> side_done;
    cudaEvent_t fork = nullptr;
};

struct fc_model {
    fc_config cfg;
    int device;
    cudaStream_t st = nullptr;
    Arena arena;       // weights
    Arena ws_arena;    // prefill workspace
    QMat tok, head;
    float* pos = nullptr;
    float *lnfg = nullptr, *lnfb = nullptr;
    std::vector<LayerDev> layers;
    // prefill workspace for ws_rows rows
    int ws_rows = 0, head_chunk = 0;
    float *x = nullptr, *n = nullptr, *qkv = nullptr, *att = nullptr, *hid = nullptr, *logits = nullptr, *probs_d = nullptr;
    int *ids_d = nullptr, *targets_d = nullptr, *err_d = nullptr;
    double* lp_d = nullptr;
    uint8_t* gr_d = nullptr;
    uint16_t *xhi = nullptr, *xlo = nullptr;   // bf16 planes of the current GEMM input
    // tensor path: bf16 hi / lo planes of LayerNorm output, qkv, attention output, GELU output
    uint16_t *nhi = nullptr, *nlo = nullptr, *qkvhi = nullptr, *qkvlo = nullptr;
    uint16_t *atthi = nullptr, *attlo = nullptr, *hidhi = nullptr, *hidlo = nullptr;
    void* head_stats = nullptr;                // fused head: per (row, 128-column tile) softmax records, 16 B each
    float* head_tlogit = nullptr;              // ... and the logit of each row's target
    int* tc_status = nullptr;                  // raised by a scoring kernel (tensor-core GEMM, attention, row tail) on a timeout
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_score_ms = 0.0f;
    // persistent decode kernel: per-layer parameter table on the device, grid size (0: the
    // model's shape is outside what that kernel supports)
    std::vector<MegaTable> mega_tables;  // [0]: the whole GPU; then halves, quarters, eighths
    float* mega_lnf = nullptr;
    QTile mega_head;                     // tile-major copy of the LM head for the persistent kernel
    int mega_grid = 0;                   // grid of mega_tables[0]
    // streams created by fc_decode_batch, kept for the next call
    std::vector<fc_stream*> pool;
    float last_batch_ms = 0.0f, last_batch_prime_ms = 0.0f;
    // per-layer statistics of the last window forward (fc_model_set_layer_stats)
    int stats_on = 0, stats_n = 0;
    LayerStatsDev* stats_d = nullptr;   // [n_layer + 2]: embedding, every block, final LayerNorm
    void* stats_scratch = nullptr;
    cudaEvent_t ev_prime = nullptr;
    BatchCtx batch;
};

struct fc_stream {
    fc_model* m;
    Arena arena;
    float *kc = nullptr, *vc = nullptr;  // [L][ctx][d]
    float *x = nullptr, *n = nullptr, *q = nullptr, *att = nullptr, *hid = nullptr, *logits = nullptr, *probs = nullptr;
    int* queue = nullptr;
    int queue_cap = 0;
    StepState* state = nullptr;
    int host_pos = 0;
    cudaGraphExec_t graph[3] = {nullptr, nullptr, nullptr};
    int graph_nodes[3] = {0, 0, 0};
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_decode_ms = 0.0f;
    // persistent decode kernel: exchange buffers, grid barrier word, status word
    float *partg = nullptr, *x1g = nullptr, *statg = nullptr;
    unsigned* bar = nullptr;
    int* status = nullptr;
    int attn_splits = 1;
    int use_mega = 0;
    // fc_decode_batch: index of the parameter table (grid size) this stream's launches use, and
    // the CUDA stream they go to (null: the model's)
    int table = 0;
    cudaStream_t cs = nullptr;
    cudaEvent_t cs_done = nullptr;
    unsigned long long* rng_d = nullptr;   // xorshift64* state of a sampled generation
    unsigned long long* trace = nullptr;   // phase timeline of the persistent kernel
    int trace_on = 0;
};
static constexpr int kTraceCap = 256;   // timeline entries per CTA

namespace fc {

// ------------------------------------------------------------------------- decode step
enum StepMode { STEP_NOHEAD = 0, STEP_SELECT = 1, STEP_PROBS = 2 };

// One token through every block: the kernel sequence of CachedTransformer::feed
// (slm/cached.rs:100-125) -> TransformerBlock::forward_with_cache (transformer.rs:221-294).
static int launch_step(fc_stream* s, int mode) {
    fc_model* m = s->m;
    const fc_config& c = m->cfg;
    cudaStream_t st = m->st;
    const int d = c.d_model;
    const size_t layer_stride = (size_t)c.ctx * d;
    FC_TRY(launch_embed_step(m->tok, m->pos, c.ctx, s->queue, s->state, s->x, st));
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerDev& L = m->layers[l];
        float* kc = s->kc + l * layer_stride;
        float* vc = s->vc + l * layer_stride;
        FC_TRY(launch_layernorm(s->x, L.ln1g, L.ln1b, 1, d, s->n, s->state, st));
        GemvOut o;
        o.out[0] = s->q; o.out[1] = kc; o.out[2] = vc; o.seg = d; o.pos_stride = d;
        FC_TRY(launch_gemv_q8(L.qkv, s->n, L.qkv_b, nullptr, EPI_NONE, o, s->state, st));
        FC_TRY(launch_attn_decode(s->q, kc, vc, d, c.n_head, c.ctx, s->state, s->att, st));
        GemvOut ox; ox.out[0] = s->x;
        FC_TRY(launch_gemv_q8(L.out, s->att, L.out_b, s->x, EPI_NONE, ox, s->state, st));
        FC_TRY(launch_layernorm(s->x, L.ln2g, L.ln2b, 1, d, s->n, s->state, st));
        GemvOut oh; oh.out[0] = s->hid;
        FC_TRY(launch_gemv_q8(L.up, s->n, L.up_b, nullptr, EPI_GELU, oh, s->state, st));
        FC_TRY(launch_gemv_q8(L.down, s->hid, L.down_b, s->x, EPI_NONE, ox, s->state, st));
    }
    if (mode == STEP_NOHEAD) return launch_step_advance(s->state, st);
    FC_TRY(launch_layernorm(s->x, m->lnfg, m->lnfb, 1, d, s->n, s->state, st));
    GemvOut ol; ol.out[0] = s->logits;
    FC_TRY(launch_gemv_q8(m->head, s->n, nullptr, nullptr, EPI_NONE, ol, s->state, st));
    return launch_step_tail(s->logits, c.vocab, mode == STEP_PROBS ? s->probs : nullptr, mode == STEP_SELECT ? 1 : 0,
                            s->queue, s->queue_cap, s->state, nullptr, st);
}

// The launch-bound step is captured once per mode into a CUDA graph and replayed; every
// per-step quantity (token, position) is read from device state, so no node is updated.
static int run_step(fc_stream* s, int mode) {
    if (!s->graph[mode]) {
        cudaStream_t st = s->m->st;
        cudaGraph_t g = nullptr;
        const int64_t before = g_launches;
        FC_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        const int rc = launch_step(s, mode);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        s->graph_nodes[mode] = (int)(g_launches - before);
        g_launches = before;
        if (rc != FC_OK) { if (g) cudaGraphDestroy(g); return rc; }
        FC_CUDA(e);
        const cudaError_t ei = cudaGraphInstantiate(&s->graph[mode], g, 0);
        cudaGraphDestroy(g);
        FC_CUDA(ei);
    }
    FC_CUDA(cudaGraphLaunch(s->graph[mode], s->m->st));
    g_launches += s->graph_nodes[mode];
    return FC_OK;
}

// n tokens from the queue through the persistent decode kernel in one launch. Steps before
// head_from skip the LM head; head steps select greedily when `select`, and the last step
// leaves its probabilities in s->probs when `probs`.
static int run_mega(fc_stream* s, int n, int head_from, int select, int probs) {
    fc_model* m = s->m;
    const fc_config& c = m->cfg;
    MegaParams p;
    p.L = c.n_layer; p.d = c.d_model; p.H = c.n_head; p.F = c.d_ff; p.T = c.ctx; p.V = c.vocab;
    p.tok = m->tok; p.head = m->mega_head; p.pos = m->pos; p.lnfpack = m->mega_lnf;
    const MegaTable& tab = m->mega_tables[s->table];
    p.layers = tab.layers;
    p.bias_pack = tab.bias_pack;
    p.kc = s->kc; p.vc = s->vc;
    p.qg = s->q; p.attg = s->att; p.partg = s->partg; p.x1g = s->x1g; p.xg = s->x; p.hidg = s->hid;
    p.logits = s->logits; p.statg = s->statg; p.probs = probs ? s->probs : nullptr;
    p.queue = s->queue; p.queue_cap = s->queue_cap; p.state = s->state;
    p.bar = s->bar; p.status = s->status;
    p.n_steps = n; p.head_from = head_from; p.select = select;
    p.attn_splits = std::max(1, std::min(s->attn_splits, tab.grid / c.n_head));
    p.trace = s->trace_on ? s->trace : nullptr;
    p.trace_cap = kTraceCap;
    p.wait_cycles = g_debug.wait_cycles; p.withhold = g_debug.withhold;
    cudaStream_t st = s->cs ? s->cs : m->st;
    if (p.trace) FC_CUDA(cudaMemsetAsync(s->trace, 0, (size_t)m->mega_grid * kTraceCap * sizeof(unsigned long long), st));
    return launch_decode_mega(p, tab.grid, st);
}

// n steps, the last one in `last_mode`, the ones before it in `mode`.
static int run_steps(fc_stream* s, int n, int mode, int last_mode) {
    if (n <= 0) return FC_OK;
    if (s->use_mega) {
        const int head_from = mode != STEP_NOHEAD ? 0 : (last_mode != STEP_NOHEAD ? n - 1 : n);
        return run_mega(s, n, head_from, last_mode == STEP_SELECT, last_mode == STEP_PROBS);
    }
    for (int i = 0; i < n; ++i) FC_TRY(run_step(s, i + 1 == n ? last_mode : mode));
    return FC_OK;
}

__global__ void set_state_kernel(StepState* st, int pos, int fed, int tail, int done, int eos, int keep_pos) {
    if (!keep_pos) st->pos = pos;
    st->fed = fed; st->tail = tail; st->done = done; st->eos = eos; st->error = 0;
}
static int set_state(fc_stream* s, int pos, int fed, int tail, int eos, int keep_pos) {
    set_state_kernel<<<1, 1, 0, s->m->st>>>(s->state, pos, fed, tail, 0, eos, keep_pos);
    FC_LAUNCHED();
    return FC_OK;
}

static int read_state(fc_stream* s, StepState* out) {
    int status = 0;
    FC_CUDA(cudaMemcpyAsync(out, s->state, sizeof(StepState), cudaMemcpyDeviceToHost, s->m->st));
    if (s->status) FC_CUDA(cudaMemcpyAsync(&status, s->status, sizeof(int), cudaMemcpyDeviceToHost, s->m->st));
    FC_CUDA(cudaStreamSynchronize(s->m->st));
    if (status != 0) {
        cudaMemsetAsync(s->status, 0, sizeof(int), s->m->st);
        return fail(FC_E_TIMEOUT, "a bounded wait inside the persistent decode kernel ran out (status %d)", status);
    }
    return FC_OK;
}

static int check_ids(const fc_model* m, const int32_t* ids, size_t n) {
    for (size_t i = 0; i < n; ++i)
        if (ids[i] < 0 || ids[i] >= m->cfg.vocab)
            return fail(FC_E_DIM, "Token index %d out of bounds for vocab_size %d", ids[i], m->cfg.vocab);
    return FC_OK;
}

// -------------------------------------------------------------------- prefill workspace
static bool tensor_path(const fc_model* m);
static int ensure_workspace(fc_model* m, int rows) {
    if (rows <= m->ws_rows) return FC_OK;
    m->ws_arena.release();
    m->ws_rows = 0;
    const fc_config& c = m->cfg;
    const size_t R = rows, d = c.d_model, F = c.d_ff;
    // fp32 mode: head logits are produced for head_chunk rows at a time (<= 1 GiB of f32). On the tensor-core
    // path the head never writes logits (its epilogue leaves softmax records): one row is kept for predict_next.
    size_t chunk = ((size_t)1 << 28) / (size_t)c.vocab;
    chunk = std::max<size_t>(1, std::min<size_t>(chunk, R));
    if (tensor_path(m)) chunk = 1;
    Arena& a = m->ws_arena;
    FC_TRY(a.alloc_n(&m->x, R * d));
    FC_TRY(a.alloc_n(&m->n, R * d));
    FC_TRY(a.alloc_n(&m->qkv, R * 3 * d));
    FC_TRY(a.alloc_n(&m->att, R * d));
    FC_TRY(a.alloc_n(&m->hid, R * F));
    FC_TRY(a.alloc_n(&m->logits, chunk * (size_t)m->head.N_pad));
    FC_TRY(a.alloc_n(&m->ids_d, R));
    FC_TRY(a.alloc_n(&m->targets_d, R));
    FC_TRY(a.alloc_n(&m->lp_d, R));
    FC_TRY(a.alloc_n(&m->gr_d, R));
    FC_TRY(a.alloc_n(&m->err_d, 1));
    FC_TRY(a.alloc_n(&m->probs_d, (size_t)c.vocab));
    if (c.math_mode == FC_MATH_BF16X3) {
        // bf16 hi / lo planes of the widest GEMM input, and the kernel's status word
        FC_TRY(a.alloc_n(&m->xhi, R * std::max(d, F)));
        FC_TRY(a.alloc_n(&m->xlo, R * std::max(d, F)));
        if (tensor_path(m)) {
            FC_TRY(a.alloc_n(&m->nhi, R * d));       FC_TRY(a.alloc_n(&m->nlo, R * d));
            FC_TRY(a.alloc_n(&m->qkvhi, R * 3 * d)); FC_TRY(a.alloc_n(&m->qkvlo, R * 3 * d));
            FC_TRY(a.alloc_n(&m->atthi, R * d));     FC_TRY(a.alloc_n(&m->attlo, R * d));
            FC_TRY(a.alloc_n(&m->hidhi, R * F));     FC_TRY(a.alloc_n(&m->hidlo, R * F));
            FC_TRY(a.alloc(&m->head_stats, R * (size_t)((c.vocab + 127) / 128) * 16));
            FC_TRY(a.alloc_n(&m->head_tlogit, R));
        }
    }
    FC_TRY(a.alloc_n(&m->tc_status, 1));
    FC_CUDA(cudaMemsetAsync(m->tc_status, 0, sizeof(int), m->st));
    m->ws_rows = rows;
    m->head_chunk = (int)chunk;
    return FC_OK;
}

static int gemm(fc_model* m, const QMat& w, const float* x, const float* bias, const float* res, int epi, float* y, int M, int ldy) {
    // FC_MATH_BF16X3: split the activations into bf16 hi/lo planes, then the tcgen05 kernel
    // (its k-blocks are 64 wide). FC_MATH_FP32, or a K that is not a multiple of 64: the
    // fp32 CUDA-core kernel.
    if (m->cfg.math_mode == FC_MATH_BF16X3 && w.K % 64 == 0) {
        FC_TRY(launch_split_bf16(x, m->xhi, m->xlo, (size_t)M * w.K, m->st));
        return launch_gemm_q8_bf16x3(w, m->xhi, m->xlo, bias, res, epi, y, M, ldy, m->tc_status, m->st);
    }
    return launch_gemm_q8_fp32(w, x, bias, res, epi, y, M, ldy, m->st);
}

// True when the whole window forward runs on tensor cores with bf16-plane activations.
static bool tensor_path(const fc_model* m) {
    const fc_config& c = m->cfg;
    return c.math_mode == FC_MATH_BF16X3 && c.d_model == c.n_head * 64 && c.d_model % 64 == 0 && c.d_ff % 64 == 0;
}

// Sequential::forward (model.rs:51-71) through every block, on B windows of T rows whose ids
// are already in m->ids_d. Leaves the residual stream in m->x.
static int forward_blocks(fc_model* m, int B, int T) {
    const fc_config& c = m->cfg;
    const int R = B * T, d = c.d_model, F = c.d_ff;
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemsetAsync(m->err_d, 0, sizeof(int), st));
    FC_TRY(launch_embed_rows(m->tok, m->pos, m->ids_d, R, T, m->x, m->err_d, st));
    // model.rs:58-68: with the statistics switched on, every layer's output is summarised as it appears
    m->stats_n = 0;
    auto layer_stats = [&]() -> int {
        if (!m->stats_on) return FC_OK;
        return launch_layer_stats(m->x, nullptr, nullptr, (size_t)R * d, m->stats_scratch, m->stats_d + m->stats_n++, st);
    };
    FC_TRY(layer_stats());
    if (tensor_path(m)) {
        // activations between kernels are bf16 hi / lo planes; only the residual stream is f32
        for (int l = 0; l < c.n_layer; ++l) {
            const LayerDev& L = m->layers[l];
            FC_TRY(launch_layernorm_planes(m->x, L.ln1g, L.ln1b, R, d, m->nhi, m->nlo, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.qkv, m->nhi, m->nlo, L.qkv_b, nullptr, EPI_NONE, nullptr, m->qkvhi, m->qkvlo, R, 3 * d, m->tc_status, st));
            FC_TRY(launch_attn_prefill_tc(m->qkvhi, m->qkvlo, B, T, d, c.n_head, m->atthi, m->attlo, m->tc_status, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.out, m->atthi, m->attlo, L.out_b, m->x, EPI_NONE, m->x, nullptr, nullptr, R, d, m->tc_status, st));
            FC_TRY(launch_layernorm_planes(m->x, L.ln2g, L.ln2b, R, d, m->nhi, m->nlo, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.up, m->nhi, m->nlo, L.up_b, nullptr, EPI_GELU, nullptr, m->hidhi, m->hidlo, R, F, m->tc_status, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.down, m->hidhi, m->hidlo, L.down_b, m->x, EPI_NONE, m->x, nullptr, nullptr, R, d, m->tc_status, st));
            FC_TRY(layer_stats());
        }
        return FC_OK;
    }
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerDev& L = m->layers[l];
        FC_TRY(launch_layernorm(m->x, L.ln1g, L.ln1b, R, d, m->n, nullptr, st));
        FC_TRY(gemm(m, L.qkv, m->n, L.qkv_b, nullptr, EPI_NONE, m->qkv, R, 3 * d));
        FC_TRY(launch_attn_prefill(m->qkv, B, T, d, c.n_head, m->att, st));
        FC_TRY(gemm(m, L.out, m->att, L.out_b, m->x, EPI_NONE, m->x, R, d));
        FC_TRY(launch_layernorm(m->x, L.ln2g, L.ln2b, R, d, m->n, nullptr, st));
        FC_TRY(gemm(m, L.up, m->n, L.up_b, nullptr, EPI_GELU, m->hid, R, F));
        FC_TRY(gemm(m, L.down, m->hid, L.down_b, m->x, EPI_NONE, m->x, R, d));
        FC_TRY(layer_stats());
    }
    return FC_OK;
}

// Forward + final LayerNorm + head + scoring tail for ids/targets already on the device.
// lp_d/gr_d filled. Logit rows are ldl floats apart (ldl % 4 == 0 for vector stores).
static int score_device(fc_model* m, int B, int T) {
    const fc_config& c = m->cfg;
    const int R = B * T, d = c.d_model, ldl = m->head.N_pad;
    FC_TRY(forward_blocks(m, B, T));
    if (tensor_path(m)) {
        // the head's epilogue keeps (max, sum of exponentials, first argmax) per row and 128-column tile and the
        // target's logit: [rows][V] logits never reach memory (scoring.rs:175-181 needs one number per row)
        FC_TRY(launch_layernorm_planes(m->x, m->lnfg, m->lnfb, R, d, m->nhi, m->nlo, m->st));
        if (m->stats_on) FC_TRY(launch_layer_stats(nullptr, m->nhi, m->nlo, (size_t)R * d, m->stats_scratch, m->stats_d + m->stats_n++, m->st));
        FC_TRY(launch_gemm_q8_bf16x3_score(m->head, m->nhi, m->nlo, m->targets_d, m->head_stats, m->head_tlogit, R, m->tc_status, m->st));
        return launch_score_combine(m->head_stats, m->head_tlogit, m->targets_d, R, (c.vocab + 127) / 128, c.vocab, m->lp_d, m->gr_d, m->st);
    }
    FC_TRY(launch_layernorm(m->x, m->lnfg, m->lnfb, R, d, m->n, nullptr, m->st));
    if (m->stats_on) FC_TRY(launch_layer_stats(m->n, nullptr, nullptr, (size_t)R * d, m->stats_scratch, m->stats_d + m->stats_n++, m->st));
    for (int r0 = 0; r0 < R; r0 += m->head_chunk) {
        const int rows = std::min(m->head_chunk, R - r0);
        FC_TRY(gemm(m, m->head, m->n + (size_t)r0 * d, nullptr, nullptr, EPI_NONE, m->logits, rows, ldl));
        FC_TRY(launch_score_rows(m->logits, ldl, c.vocab, m->targets_d + r0, rows, m->lp_d + r0, m->gr_d + r0, m->tc_status, m->st));
    }
    return FC_OK;
}

}  // namespace fc

// =====================================================================================
//                                      C ABI
// =====================================================================================
extern "C" {

const char* fc_last_error(void) { return fc::g_err; }

int fc_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    int ok = 0;
    for (int i = 0; i < n; ++i) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ++ok;
    }
    return ok;
}

int64_t fc_take_launch_count(void) {
    const int64_t n = g_launches;
    g_launches = 0;
    return n;
}

// ------------------------------------------------------------------ standalone linear
int fc_qweight_upload(int device, const void* wq, int N, int K, fc_qweight** out) {
    if (!out) return fail(FC_E_ARG, "fc_qweight_upload: out is null");
    *out = nullptr;
    FC_TRY(select_device(device));
    fc_qweight* w = new fc_qweight;
    w->device = device;
    const int rc = upload_q8(w->arena, wq, N, K, &w->w, 0);
    if (rc != FC_OK) { w->arena.release(); delete w; return rc; }
    *out = w;
    return FC_OK;
}

void fc_qweight_free(fc_qweight* w) {
    if (!w) return;
    cudaSetDevice(w->device);
    cudaDeviceSynchronize();
    w->arena.release();
    w->planes.release();
    delete w;
}

int fc_q8_0_linear_dev(const fc_qweight* w, const float* x_dev, const float* bias_dev, float* y_dev,
                       int M, int math_mode, void* cuda_stream) {
    if (!w || !x_dev || !y_dev) return fail(FC_E_ARG, "fc_q8_0_linear_dev: null argument");
    if (!aligned16(x_dev) || !aligned16(y_dev) || !aligned16(bias_dev))
        return fail(FC_E_ARG, "fc_q8_0_linear_dev: x_dev, y_dev and bias_dev must be 16-byte aligned");
    if (M < 0) return fail(FC_E_SHAPE, "fc_q8_0_linear_dev: M = %d", M);
    if (M == 0) return FC_OK;
    if (math_mode != FC_MATH_FP32 && math_mode != FC_MATH_BF16X3) return fail(FC_E_ARG, "unknown math_mode %d", math_mode);
    FC_CUDA(cudaSetDevice(w->device));
    cudaStream_t st = (cudaStream_t)cuda_stream;
    if (M == 1) {
        GemvOut o; o.out[0] = y_dev;
        return launch_gemv_q8(w->w, x_dev, bias_dev, nullptr, EPI_NONE, o, nullptr, st);
    }
    if (math_mode == FC_MATH_BF16X3 && w->w.K % 64 == 0) {
        // the bf16 planes of x and the status word live in the weight handle and grow on demand
        fc_qweight* wm = const_cast<fc_qweight*>(w);
        const size_t need = (size_t)M * w->w.K;
        if (need > wm->plane_elems) {
            FC_CUDA(cudaStreamSynchronize(st));
            wm->planes.release();
            wm->plane_elems = 0;
            FC_TRY(wm->planes.alloc_n(&wm->xhi, need));
            FC_TRY(wm->planes.alloc_n(&wm->xlo, need));
            FC_TRY(wm->planes.alloc_n(&wm->status, 1));
            FC_CUDA(cudaMemsetAsync(wm->status, 0, sizeof(int), st));
            wm->plane_elems = need;
        }
        FC_TRY(launch_split_bf16(x_dev, wm->xhi, wm->xlo, need, st));
        return launch_gemm_q8_bf16x3(w->w, wm->xhi, wm->xlo, bias_dev, nullptr, EPI_NONE, y_dev, M, w->w.N, wm->status, st);
    }
    return launch_gemm_q8_fp32(w->w, x_dev, bias_dev, nullptr, EPI_NONE, y_dev, M, w->w.N, st);
}

int fc_q8_0_linear(int device, const float* x, const void* wq, const float* bias, float* y,
                   int M, int K, int N, int math_mode) {
    if (!x || !wq || !y) return fail(FC_E_ARG, "fc_q8_0_linear: null argument");
    if (M < 0 || N <= 0 || K <= 0) return fail(FC_E_SHAPE, "fc_q8_0_linear: bad shape M=%d K=%d N=%d", M, K, N);
    fc_qweight* w = nullptr;
    FC_TRY(fc_qweight_upload(device, wq, N, K, &w));
    int rc = FC_OK;
    float *xd = nullptr, *bd = nullptr, *yd = nullptr;
    if (M > 0) {
        Arena tmp;
        rc = tmp.alloc_n(&xd, (size_t)M * K);
        if (rc == FC_OK) rc = tmp.alloc_n(&yd, (size_t)M * N);
        if (rc == FC_OK && bias) rc = tmp.alloc_n(&bd, (size_t)N);
        auto copy = [&](void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
            if (rc == FC_OK && cudaMemcpy(dst, src, bytes, kind) != cudaSuccess) rc = fail(FC_E_CUDA, "fc_q8_0_linear: copy failed");
        };
        copy(xd, x, (size_t)M * K * 4, cudaMemcpyHostToDevice);
        if (bias) copy(bd, bias, (size_t)N * 4, cudaMemcpyHostToDevice);
        if (rc == FC_OK) rc = fc_q8_0_linear_dev(w, xd, bd, yd, M, math_mode, nullptr);
        if (rc == FC_OK && cudaDeviceSynchronize() != cudaSuccess) rc = cuda_fail(cudaGetLastError(), "fc_q8_0_linear kernel", __FILE__, __LINE__);
        if (rc == FC_OK && w->status) {
            int status = 0;
            copy(&status, w->status, sizeof(int), cudaMemcpyDeviceToHost);
            if (rc == FC_OK && status != 0) rc = fail(FC_E_TIMEOUT, "a bounded wait inside the tensor-core GEMM ran out (status %d)", status);
        }
        copy(y, yd, (size_t)M * N * 4, cudaMemcpyDeviceToHost);
        tmp.release();
    }
    fc_qweight_free(w);
    return rc;
}

// ------------------------------------------------------------------------------ model
static int model_build(fc_model* m, const fc_weights* w) {
    const fc_config& c = m->cfg;
    const int d = c.d_model, F = c.d_ff, V = c.vocab;
    cudaStream_t st = m->st;
    Arena& a = m->arena;
    FC_TRY(upload_q8(a, w->token_embd_q8, V, d, &m->tok, st));
    if (c.tied) m->head = m->tok;   // loader/gpt2.rs:228-233
    else FC_TRY(upload_q8(a, w->output_q8, V, d, &m->head, st));
    FC_TRY(upload_f32(a, w->position_embd, (size_t)c.ctx * d, &m->pos, st));
    FC_TRY(upload_f32(a, w->out_norm_g, d, &m->lnfg, st));
    FC_TRY(upload_f32(a, w->out_norm_b, d, &m->lnfb, st));
    if (!w->layers) return fail(FC_E_FORMAT, "fc_weights.layers is null");
    m->layers.resize(c.n_layer);
    for (int l = 0; l < c.n_layer; ++l) {
        const fc_layer_weights& s = w->layers[l];
        LayerDev& L = m->layers[l];
        FC_TRY(upload_q8(a, s.attn_qkv_q8, 3 * d, d, &L.qkv, st));
        FC_TRY(upload_q8(a, s.attn_out_q8, d, d, &L.out, st));
        FC_TRY(upload_q8(a, s.ffn_up_q8, F, d, &L.up, st));
        FC_TRY(upload_q8(a, s.ffn_down_q8, d, F, &L.down, st));
        FC_TRY(upload_f32(a, s.attn_qkv_b, 3 * (size_t)d, &L.qkv_b, st));
        FC_TRY(upload_f32(a, s.attn_out_b, d, &L.out_b, st));
        FC_TRY(upload_f32(a, s.ffn_up_b, F, &L.up_b, st));
        FC_TRY(upload_f32(a, s.ffn_down_b, d, &L.down_b, st));
        FC_TRY(upload_f32(a, s.ln1_g, d, &L.ln1g, st));
        FC_TRY(upload_f32(a, s.ln1_b, d, &L.ln1b, st));
        FC_TRY(upload_f32(a, s.ln2_g, d, &L.ln2g, st));
        FC_TRY(upload_f32(a, s.ln2_b, d, &L.ln2b, st));
    }
    if (mega_supported(c)) {
        int full = 0;
        FC_TRY(mega_max_grid(&full));
        // One parameter table per grid size: the full GPU for a single stream, and halves,
        // quarters and eighths of it for streams decoded side by side (fc_decode_batch).
        // Per block: the four LayerNorm vectors back to back, and for every CTA of the
        // persistent kernel the slices of the four bias vectors that belong to its rows.
        std::vector<float*> lnpacks(c.n_layer, nullptr);
        std::vector<float> ln((size_t)4 * d);
        for (int l = 0; l < c.n_layer; ++l) {
            const fc_layer_weights& s = w->layers[l];
            std::copy(s.ln1_g, s.ln1_g + d, ln.begin());
            std::copy(s.ln1_b, s.ln1_b + d, ln.begin() + d);
            std::copy(s.ln2_g, s.ln2_g + d, ln.begin() + 2 * d);
            std::copy(s.ln2_b, s.ln2_b + d, ln.begin() + 3 * d);
            FC_TRY(upload_f32(a, ln.data(), ln.size(), &lnpacks[l], st));
            FC_CUDA(cudaStreamSynchronize(st));   // ln is reused by the next block
        }
        std::fill(ln.begin(), ln.end(), 0.0f);
        std::copy(w->out_norm_g, w->out_norm_g + d, ln.begin());
        std::copy(w->out_norm_b, w->out_norm_b + d, ln.begin() + d);
        FC_TRY(upload_f32(a, ln.data(), ln.size(), &m->mega_lnf, st));
        FC_CUDA(cudaStreamSynchronize(st));
        {   // the persistent kernel reads the LM head from a tile-major copy (integer tensor cores)
            unsigned char* t = nullptr;
            FC_TRY(a.alloc_n(&t, (size_t)(m->head.N_pad / kMegaStripRows) * mega_strip_bytes(m->head.K)));
            FC_TRY(launch_repack_tiles(m->head, t, st));
            m->mega_head.t = t; m->mega_head.N = m->head.N; m->mega_head.K = m->head.K;
        }
        for (int div = 1; div <= 8; div *= 2) {
            const int grid = full / div;
            if (grid < c.n_head) break;
            // the head slice and the bias slices of one CTA must fit its shared-memory buffers
            int pack = 0;
            for (int cta = 0; cta < grid; ++cta) {
                int off[4];
                pack = std::max(pack, mega_bias_offsets(d, F, cta, grid, off));
            }
            pack = (pack + 3) & ~3;
            if ((c.vocab + grid - 1) / grid + 16 > mega_head_rows_max() || pack > kMegaBiasPackMax) break;
            std::vector<MegaLayer> tab(c.n_layer);
            std::vector<float> bp((size_t)grid * pack);
            for (int l = 0; l < c.n_layer; ++l) {
                const fc_layer_weights& s = w->layers[l];
                const LayerDev& L = m->layers[l];
                std::fill(bp.begin(), bp.end(), 0.0f);
                const float* src[4] = {s.attn_qkv_b, s.attn_out_b, s.ffn_up_b, s.ffn_down_b};
                const int N[4] = {3 * d, d, F, d}, K[4] = {d, d, d, F};
                for (int cta = 0; cta < grid; ++cta) {
                    int off[4];
                    mega_bias_offsets(d, F, cta, grid, off);
                    for (int i = 0; i < 4; ++i) {
                        int r0, r1;
                        mega_cta_rows(N[i], K[i], cta, grid, &r0, &r1);
                        std::copy(src[i] + r0, src[i] + r1, bp.begin() + (size_t)cta * pack + off[i]);
                    }
                }
                float* bpd = nullptr;
                FC_TRY(upload_f32(a, bp.data(), bp.size(), &bpd, st));
                FC_CUDA(cudaStreamSynchronize(st));   // bp is reused by the next block
                tab[l] = MegaLayer{L.qkv, L.out, L.up, L.down, lnpacks[l], bpd};
            }
            MegaTable t;
            t.grid = grid;
            t.bias_pack = pack;
            FC_TRY(a.alloc_n(&t.layers, (size_t)c.n_layer));
            FC_CUDA(cudaMemcpyAsync(t.layers, tab.data(), tab.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice, st));
            FC_CUDA(cudaStreamSynchronize(st));
            m->mega_tables.push_back(t);
        }
        if (!m->mega_tables.empty()) m->mega_grid = m->mega_tables[0].grid;
    }
    FC_CUDA(cudaStreamSynchronize(st));
    return FC_OK;
}

int fc_model_create(const fc_config* cfg, const fc_weights* w, int device, fc_model** out) {
    if (!cfg || !w || !out) return fail(FC_E_ARG, "fc_model_create: null argument");
    *out = nullptr;
    const fc_config& c = *cfg;
    if (c.n_layer <= 0 || c.d_model <= 0 || c.n_head <= 0 || c.d_ff <= 0 || c.ctx <= 0 || c.vocab <= 0)
        return fail(FC_E_SHAPE, "fc_model_create: every dimension must be positive");
    if (c.d_model % c.n_head) return fail(FC_E_DIM, "embedding_dim %d is not divisible by num_heads %d", c.d_model, c.n_head);
    if (c.d_model % 32 || c.d_ff % 32) return fail(FC_E_FORMAT, "d_model %d and d_ff %d must be multiples of 32 for Q8_0 storage", c.d_model, c.d_ff);
    const int hd = c.d_model / c.n_head;
    if (hd != 32 && hd != 64) return fail(FC_E_SHAPE, "head_dim %d is not supported (32 or 64)", hd);
    if (c.math_mode != FC_MATH_FP32 && c.math_mode != FC_MATH_BF16X3) return fail(FC_E_ARG, "unknown math_mode %d", c.math_mode);
    if (!c.tied && !w->output_q8) return fail(FC_E_FORMAT, "untied model without output.weight");
    FC_TRY(select_device(device));
    fc_model* m = new fc_model;
    m->cfg = c;
    m->device = device;
    int rc = FC_OK;
    if (cudaStreamCreateWithFlags(&m->st, cudaStreamNonBlocking) != cudaSuccess) rc = fail(FC_E_CUDA, "stream creation failed");
    if (rc == FC_OK && (cudaEventCreate(&m->ev0) != cudaSuccess || cudaEventCreate(&m->ev1) != cudaSuccess)) rc = fail(FC_E_CUDA, "event creation failed");
    if (rc == FC_OK) rc = model_build(m, w);
    if (rc == FC_OK) {
        const char* tr = getenv("FERRUM_CUDA_TRACE");
        if (tr && tr[0] == '1') rc = fc_model_set_layer_stats(m, 1);
    }
    if (rc != FC_OK) { fc_model_free(m); return rc; }
    *out = m;
    return FC_OK;
}

void fc_model_free(fc_model* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    if (m->st) cudaStreamSynchronize(m->st);
    for (fc_stream* s : m->pool) fc_stream_free(s);
    m->pool.clear();
    m->arena.release();
    m->ws_arena.release();
    if (m->batch.graph) cudaGraphExecDestroy(m->batch.graph);
    if (m->batch.graph4) cudaGraphExecDestroy(m->batch.graph4);
    for (cudaStream_t t : m->batch.side) cudaStreamDestroy(t);
    for (cudaEvent_t e : m->batch.side_done) cudaEventDestroy(e);
    if (m->batch.fork) cudaEventDestroy(m->batch.fork);
    m->batch.arena.release();
    m->batch.frag_arena.release();
    if (m->ev0) cudaEventDestroy(m->ev0);
    if (m->ev1) cudaEventDestroy(m->ev1);
    if (m->ev_prime) cudaEventDestroy(m->ev_prime);
    if (m->st) cudaStreamDestroy(m->st);
    delete m;
}

int fc_model_config(const fc_model* m, fc_config* out) {
    if (!m || !out) return fail(FC_E_ARG, "fc_model_config: null argument");
    *out = m->cfg;
    return FC_OK;
}

float fc_last_score_ms(const fc_model* m) { return m ? m->last_score_ms : 0.0f; }

int fc_model_set_layer_stats(fc_model* m, int on) {
    if (!m) return fail(FC_E_ARG, "fc_model_set_layer_stats: null model");
    FC_CUDA(cudaSetDevice(m->device));
    if (on && !m->stats_d) {
        FC_TRY(m->arena.alloc_n(&m->stats_d, (size_t)m->cfg.n_layer + 2));
        FC_TRY(m->arena.alloc(&m->stats_scratch, layer_stats_scratch_bytes()));
    }
    m->stats_on = on != 0;
    m->stats_n = 0;
    return FC_OK;
}

int fc_model_read_layer_stats(fc_model* m, fc_layer_stats* out, int cap) {
    if (!m || (cap > 0 && !out) || cap < 0) return fail(FC_E_ARG, "fc_model_read_layer_stats: bad argument");
    if (!m->stats_d || m->stats_n == 0) return 0;
    FC_CUDA(cudaSetDevice(m->device));
    FC_CUDA(cudaStreamSynchronize(m->st));
    std::vector<LayerStatsDev> h(m->stats_n);
    FC_CUDA(cudaMemcpy(h.data(), m->stats_d, h.size() * sizeof(LayerStatsDev), cudaMemcpyDeviceToHost));
    const int n = std::min(cap, m->stats_n);
    for (int i = 0; i < n; ++i) {
        out[i].min = h[i].min; out[i].max = h[i].max; out[i].mean = h[i].mean;
        out[i].nan_count = h[i].nan_count; out[i].inf_count = h[i].inf_count; out[i].n_elements = h[i].n;
    }
    return n;
}

// ---------------------------------------------------------------------------- scoring
// Runs B windows x T rows through the model; double log-probs / flags stay on the device
// until copied into the caller's arrays.
static int score_windows_impl(fc_model* m, const int32_t* ids, const int32_t* targets, int B, int T,
                              double* lp_host, uint8_t* gr_host) {
    const fc_config& c = m->cfg;
    if (B <= 0 || T <= 0) return fail(FC_E_SHAPE, "scoring needs B > 0 and T > 0 (got %d, %d)", B, T);
    if (T > c.ctx) return fail(FC_E_DIM, "Sequence length %d exceeds max_seq_len %d", T, c.ctx);
    if ((int64_t)B * T > (int64_t)1 << 24) return fail(FC_E_SHAPE, "too many rows in one forward: %lld", (long long)B * T);
    const int R = B * T;
    FC_TRY(check_ids(m, ids, (size_t)R));
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(ensure_workspace(m, R));
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemcpyAsync(m->ids_d, ids, (size_t)R * 4, cudaMemcpyHostToDevice, st));
    FC_CUDA(cudaMemcpyAsync(m->targets_d, targets, (size_t)R * 4, cudaMemcpyHostToDevice, st));
    FC_CUDA(cudaEventRecord(m->ev0, st));
    FC_TRY(score_device(m, B, T));
    FC_CUDA(cudaEventRecord(m->ev1, st));
    FC_CUDA(cudaMemcpyAsync(lp_host, m->lp_d, (size_t)R * 8, cudaMemcpyDeviceToHost, st));
    FC_CUDA(cudaMemcpyAsync(gr_host, m->gr_d, (size_t)R, cudaMemcpyDeviceToHost, st));
    int tc_status = 0;
    if (m->tc_status) FC_CUDA(cudaMemcpyAsync(&tc_status, m->tc_status, sizeof(int), cudaMemcpyDeviceToHost, st));
    FC_CUDA(cudaStreamSynchronize(st));
    if (tc_status != 0) {
        cudaMemsetAsync(m->tc_status, 0, sizeof(int), st);
        return fail(FC_E_TIMEOUT, "a bounded wait inside a scoring kernel ran out (status %d)", tc_status);
    }
    float ms = 0.0f;
    FC_CUDA(cudaEventElapsedTime(&ms, m->ev0, m->ev1));
    m->last_score_ms += ms;
    return FC_OK;
}

int fc_score_windows(fc_model* m, const int32_t* ids, const int32_t* targets, int B, int T,
                     float* logprob, uint8_t* is_greedy) {
    if (!m || !ids || !targets || !logprob || !is_greedy) return fail(FC_E_ARG, "fc_score_windows: null argument");
    m->last_score_ms = 0.0f;
    std::vector<double> lp((size_t)std::max(0, B) * std::max(0, T));
    FC_TRY(score_windows_impl(m, ids, targets, B, T, lp.data(), is_greedy));
    for (size_t i = 0; i < lp.size(); ++i) logprob[i] = (float)lp[i];
    return FC_OK;
}

}  // extern "C"

namespace {
// One window of the plan of scoring.rs:164-172.
struct Window { int seq, start, first, end; };

// (start, first target, end target exclusive) for targets from..n of one sequence.
void plan_windows(int seq, int n, int from, int T, std::vector<Window>* out) {
    const int half = std::max(1, T / 2);
    int next = std::max(from, 1);
    while (next < n) {
        const int start = next <= T ? 0 : next - half;
        const int end = std::min(start + T + 1, n);
        out->push_back(Window{seq, start, next, end});
        next = end;
    }
}

// Scores every window of `plan` in batches; seq_ids(s) gives the ids of sequence s, seq_len(s)
// its length. For each scored target calls add(seq, target, logprob, greedy).
template <class Ids, class Len, class Add>
int run_plan_ragged(fc_model* m, const std::vector<Window>& plan, int batch, Ids seq_ids, Len seq_len, Add add) {
    const int T = m->cfg.ctx;
    std::vector<int32_t> ids, targets;
    std::vector<double> lp;
    std::vector<uint8_t> gr;
    for (size_t w0 = 0; w0 < plan.size(); w0 += batch) {
        const int B = (int)std::min<size_t>(batch, plan.size() - w0);
        // rows past the longest window of the batch are never read under the causal mask
        int Tb = 1;
        for (int b = 0; b < B; ++b) Tb = std::max(Tb, std::min(plan[w0 + b].start + T, seq_len(plan[w0 + b].seq)) - plan[w0 + b].start);
        ids.assign((size_t)B * Tb, 0);          // right padding with id 0 (scoring.rs:188-190)
        targets.assign((size_t)B * Tb, -1);
        for (int b = 0; b < B; ++b) {
            const Window& w = plan[w0 + b];
            const int32_t* src = seq_ids(w.seq);
            const int wl = std::min(w.start + T, seq_len(w.seq)) - w.start;
            std::copy(src + w.start, src + w.start + wl, ids.begin() + (size_t)b * Tb);
            for (int t = w.first; t < w.end; ++t) targets[(size_t)b * Tb + (t - 1 - w.start)] = src[t];
        }
        lp.resize((size_t)B * Tb);
        gr.resize((size_t)B * Tb);
        FC_TRY(score_windows_impl(m, ids.data(), targets.data(), B, Tb, lp.data(), gr.data()));
        for (int b = 0; b < B; ++b) {
            const Window& w = plan[w0 + b];
            for (int t = w.first; t < w.end; ++t) {
                const size_t r = (size_t)b * Tb + (t - 1 - w.start);
                add(w.seq, t, lp[r], gr[r]);
            }
        }
    }
    return FC_OK;
}
template <class Ids, class Add>
int run_plan(fc_model* m, const std::vector<Window>& plan, int batch, Ids seq_ids, int n, Add add) {
    return run_plan_ragged(m, plan, batch, seq_ids, [n](int) { return n; }, add);
}
}  // namespace

extern "C" {

int fc_score_requests(fc_model* m, const int32_t* ids, const int64_t* offsets, const int32_t* from, int n_req, int batch_windows,
                      fc_score* scores) {
    if (!m || !scores || (n_req > 0 && (!ids || !offsets || !from))) return fail(FC_E_ARG, "fc_score_requests: null argument");
    if (n_req < 0) return fail(FC_E_SHAPE, "fc_score_requests: n_req = %d", n_req);
    m->last_score_ms = 0.0f;
    std::vector<Window> plan;
    for (int r = 0; r < n_req; ++r) {
        scores[r].logprob = 0.0; scores[r].n_tokens = 0; scores[r].greedy = 1;
        const int64_t n = offsets[r + 1] - offsets[r];
        if (n < 0 || n > (1 << 30) || from[r] < 0) return fail(FC_E_SHAPE, "fc_score_requests: request %d has length %lld, from %d", r, (long long)n, from[r]);
        FC_TRY(check_ids(m, ids + offsets[r], (size_t)n));
        plan_windows(r, (int)n, from[r], m->cfg.ctx, &plan);
    }
    if (plan.empty()) return FC_OK;
    // windows of similar length share a forward: the rows a batch pads are wasted work
    auto wlen = [&](const Window& w) { return std::min<int64_t>(w.start + m->cfg.ctx, offsets[w.seq + 1] - offsets[w.seq]) - w.start; };
    std::stable_sort(plan.begin(), plan.end(), [&](const Window& a, const Window& b) { return wlen(a) > wlen(b); });
    if (batch_windows <= 0) batch_windows = 32;
    return run_plan_ragged(m, plan, batch_windows, [&](int r) { return ids + offsets[r]; },
                           [&](int r) { return (int)(offsets[r + 1] - offsets[r]); },
                           [&](int r, int, double l, uint8_t g) { scores[r].logprob += l; scores[r].n_tokens += 1; scores[r].greedy &= (int32_t)g; });
}

int fc_token_logprobs(fc_model* m, const int32_t* ids, int n, int from, fc_score* score, float* lp, uint8_t* is_greedy) {
    if (!m || !score || (n > 0 && !ids)) return fail(FC_E_ARG, "fc_token_logprobs: null argument");
    score->logprob = 0.0; score->n_tokens = 0; score->greedy = 1;
    m->last_score_ms = 0.0f;
    if (n <= 0) return FC_OK;
    FC_TRY(check_ids(m, ids, (size_t)n));
    std::vector<Window> plan;
    plan_windows(0, n, from, m->cfg.ctx, &plan);
    // SCORE_BATCH = 32 windows per forward (scoring.rs:45)
    return run_plan(m, plan, 32, [&](int) { return ids; }, n, [&](int, int t, double l, uint8_t g) {
        score->logprob += l; score->n_tokens += 1; score->greedy &= (int32_t)g;
        if (lp) lp[t] = (float)l;
        if (is_greedy) is_greedy[t] = g;
    });
}

int fc_score_sequences(fc_model* m, const int32_t* ids, int n_seq, int seq_len, int batch_windows,
                       fc_score* scores, float* lp) {
    if (!m || !ids || !scores) return fail(FC_E_ARG, "fc_score_sequences: null argument");
    if (n_seq < 0 || seq_len < 0) return fail(FC_E_SHAPE, "fc_score_sequences: negative size");
    m->last_score_ms = 0.0f;
    for (int s = 0; s < n_seq; ++s) { scores[s].logprob = 0.0; scores[s].n_tokens = 0; scores[s].greedy = 1; }
    if (n_seq == 0 || seq_len == 0) return FC_OK;
    FC_TRY(check_ids(m, ids, (size_t)n_seq * seq_len));
    std::vector<Window> plan;
    for (int s = 0; s < n_seq; ++s) plan_windows(s, seq_len, 1, m->cfg.ctx, &plan);
    if (batch_windows <= 0) batch_windows = 32;
    if (lp) for (int s = 0; s < n_seq; ++s) lp[(size_t)s * seq_len] = 0.0f;
    return run_plan(m, plan, batch_windows, [&](int s) { return ids + (size_t)s * seq_len; }, seq_len,
                    [&](int s, int t, double l, uint8_t g) {
                        scores[s].logprob += l; scores[s].n_tokens += 1; scores[s].greedy &= (int32_t)g;
                        if (lp) lp[(size_t)s * seq_len + t] = (float)l;
                    });
}

int fc_predict_next(fc_model* m, const int32_t* ids, int n, float* probs) {
    if (!m || !ids || !probs) return fail(FC_E_ARG, "fc_predict_next: null argument");
    const fc_config& c = m->cfg;
    if (n <= 0) return fail(FC_E_SHAPE, "fc_predict_next: empty input");
    if (n > c.ctx) return fail(FC_E_DIM, "Sequence length %d exceeds max_seq_len %d", n, c.ctx);
    FC_TRY(check_ids(m, ids, (size_t)n));
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(ensure_workspace(m, n));
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemcpyAsync(m->ids_d, ids, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    FC_TRY(forward_blocks(m, 1, n));
    FC_TRY(launch_layernorm(m->x + (size_t)(n - 1) * c.d_model, m->lnfg, m->lnfb, 1, c.d_model,
                            m->n + (size_t)(n - 1) * c.d_model, nullptr, st));
    GemvOut o; o.out[0] = m->logits;
    FC_TRY(launch_gemv_q8(m->head, m->n + (size_t)(n - 1) * c.d_model, nullptr, nullptr, EPI_NONE, o, nullptr, st));
    FC_TRY(launch_softmax_row(m->logits, c.vocab, m->probs_d, st));
    FC_CUDA(cudaMemcpyAsync(probs, m->probs_d, (size_t)c.vocab * 4, cudaMemcpyDeviceToHost, st));
    FC_CUDA(cudaStreamSynchronize(st));
    return FC_OK;
}

// ----------------------------------------------------------------------------- streams
int fc_stream_create(fc_model* m, fc_stream** out) {
    if (!m || !out) return fail(FC_E_ARG, "fc_stream_create: null argument");
    *out = nullptr;
    FC_CUDA(cudaSetDevice(m->device));
    const fc_config& c = m->cfg;
    fc_stream* s = new fc_stream;
    s->m = m;
    Arena& a = s->arena;
    const size_t cache = (size_t)c.n_layer * c.ctx * c.d_model;
    s->queue_cap = c.ctx + 8;
    int rc = a.alloc_n(&s->kc, cache);
    if (rc == FC_OK) rc = a.alloc_n(&s->vc, cache);
    if (rc == FC_OK) rc = a.alloc_n(&s->x, (size_t)c.d_model);
    if (rc == FC_OK) rc = a.alloc_n(&s->n, (size_t)c.d_model);
    if (rc == FC_OK) rc = a.alloc_n(&s->q, (size_t)c.d_model);
    if (rc == FC_OK) rc = a.alloc_n(&s->att, (size_t)c.d_model);
    if (rc == FC_OK) rc = a.alloc_n(&s->hid, (size_t)c.d_ff);
    if (rc == FC_OK) rc = a.alloc_n(&s->logits, (size_t)c.vocab);
    if (rc == FC_OK) rc = a.alloc_n(&s->probs, (size_t)c.vocab);
    if (rc == FC_OK) rc = a.alloc_n(&s->queue, (size_t)s->queue_cap);
    if (rc == FC_OK) rc = a.alloc_n(&s->state, 1);
    if (rc == FC_OK && m->mega_grid > 0) {
        const int hd = c.d_model / c.n_head;
        s->attn_splits = std::max(1, std::min(8, m->mega_grid / c.n_head));
        rc = a.alloc_n(&s->partg, (size_t)c.n_head * s->attn_splits * (hd + 2));
        if (rc == FC_OK) rc = a.alloc_n(&s->x1g, (size_t)c.d_model);
        if (rc == FC_OK) rc = a.alloc_n(&s->statg, (size_t)m->mega_grid * 4);
        if (rc == FC_OK) rc = a.alloc_n(&s->bar, 1);
        if (rc == FC_OK) rc = a.alloc_n(&s->status, 1);
        if (rc == FC_OK && cudaMemsetAsync(s->status, 0, sizeof(int), m->st) != cudaSuccess) rc = fail(FC_E_CUDA, "status word initialisation failed");
        if (rc == FC_OK) rc = a.alloc_n(&s->trace, (size_t)m->mega_grid * kTraceCap);
        s->use_mega = 1;
    }
    if (rc == FC_OK && (cudaEventCreate(&s->ev0) != cudaSuccess || cudaEventCreate(&s->ev1) != cudaSuccess)) rc = fail(FC_E_CUDA, "event creation failed");
    if (rc == FC_OK) rc = set_state(s, 0, 0, 0, -1, 0);
    if (rc == FC_OK && cudaStreamSynchronize(m->st) != cudaSuccess) rc = fail(FC_E_CUDA, "stream initialisation failed");
    if (rc != FC_OK) { fc_stream_free(s); return rc; }
    *out = s;
    return FC_OK;
}

void fc_stream_free(fc_stream* s) {
    if (!s) return;
    cudaSetDevice(s->m->device);
    cudaStreamSynchronize(s->m->st);
    if (s->cs) { cudaStreamSynchronize(s->cs); cudaStreamDestroy(s->cs); }
    if (s->cs_done) cudaEventDestroy(s->cs_done);
    for (int i = 0; i < 3; ++i) if (s->graph[i]) cudaGraphExecDestroy(s->graph[i]);
    if (s->ev0) cudaEventDestroy(s->ev0);
    if (s->ev1) cudaEventDestroy(s->ev1);
    s->arena.release();
    delete s;
}

int fc_stream_reset(fc_stream* s) {
    if (!s) return fail(FC_E_ARG, "fc_stream_reset: null stream");
    FC_CUDA(cudaSetDevice(s->m->device));
    s->host_pos = 0;
    return set_state(s, 0, 0, 0, -1, 0);
}

int fc_cached_len(const fc_stream* s) { return s ? s->host_pos : 0; }

int fc_stream_set_trace(fc_stream* s, int on) {
    if (!s) return fail(FC_E_ARG, "fc_stream_set_trace: null stream");
    if (on && !s->trace) return fail(FC_E_SHAPE, "tracing needs the persistent decode kernel");
    s->trace_on = on != 0;
    return FC_OK;
}

int fc_stream_read_trace(fc_stream* s, uint64_t* out, int cap) { return fc_stream_read_trace_cta(s, 0, out, cap); }

int fc_stream_read_trace_cta(fc_stream* s, int cta, uint64_t* out, int cap) {
    if (!s || !out || cap < 0) return fail(FC_E_ARG, "fc_stream_read_trace: bad argument");
    if (!s->trace) return 0;
    if (cta < 0 || cta >= s->m->mega_grid) return fail(FC_E_ARG, "fc_stream_read_trace: the kernel runs %d CTAs", s->m->mega_grid);
    FC_CUDA(cudaSetDevice(s->m->device));
    FC_CUDA(cudaStreamSynchronize(s->m->st));
    std::vector<unsigned long long> h(kTraceCap);
    FC_CUDA(cudaMemcpy(h.data(), s->trace + (size_t)cta * kTraceCap, kTraceCap * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    int n = 0;
    while (n < kTraceCap && n < cap && h[n] != 0) { out[n] = h[n]; ++n; }
    return n;
}

int fc_stream_set_mode(fc_stream* s, int mode) {
    if (!s) return fail(FC_E_ARG, "fc_stream_set_mode: null stream");
    if (mode == FC_DECODE_PERSISTENT && s->m->mega_grid <= 0)
        return fail(FC_E_SHAPE, "the persistent decode kernel does not support this model shape");
    if (mode != FC_DECODE_PERSISTENT && mode != FC_DECODE_PER_KERNEL) return fail(FC_E_ARG, "unknown decode mode %d", mode);
    s->use_mega = mode == FC_DECODE_PERSISTENT;
    return FC_OK;
}
float fc_last_decode_ms(const fc_stream* s) { return s ? s->last_decode_ms : 0.0f; }

__global__ void bump_state_kernel(StepState* st, int by) {
    if (st->done | st->error) return;
    st->pos += by;
    st->fed += by;
}

// CachedTransformer::prime (slm/cached.rs:129-136) feeds the ids one at a time; on an empty
// cache the same rows come out of ONE window forward (TransformerBlock::forward,
// layer/transformer.rs:314-534, equals forward_with_cache row by row: transformer.rs:669-716),
// so the n ids in queue[0..n) of each of the S streams go through every block as S windows of
// n rows in fp32, each block's K and V rows are copied into the streams' caches, and only the
// last row of a window meets the head.
// Very short prompts stay on the token-by-token path (one persistent-kernel launch); up to 64
// rows the GEMMs run on small tiles so that every SM gets one.
// Returns FC_OK with *used = 0 when the shape is not covered (the caller feeds token by token).
constexpr int kPrimeBatchMin = 8;
static int prime_batched(fc_stream* const* ss, int S, int n, int last_mode, int* used, float* const* kcs_dev = nullptr,
                         float* const* vcs_dev = nullptr) {
    fc_model* m = ss[0]->m;
    const fc_config& c = m->cfg;
    const int d = c.d_model, F = c.d_ff, hd = d / c.n_head, R = S * n;
    *used = 0;
    if (R < kPrimeBatchMin || n < 2 || (hd != 32 && hd != 64)) return FC_OK;
    for (int i = 0; i < S; ++i)
        if (ss[i]->host_pos != 0) return FC_OK;
    cudaStream_t st = m->st;
    FC_TRY(ensure_workspace(m, R));
    for (int i = 0; i < S; ++i)
        FC_CUDA(cudaMemcpyAsync(m->ids_d + (size_t)i * n, ss[i]->queue, (size_t)n * sizeof(int), cudaMemcpyDeviceToDevice, st));
    FC_CUDA(cudaMemsetAsync(m->err_d, 0, sizeof(int), st));
    FC_TRY(launch_embed_rows(m->tok, m->pos, m->ids_d, R, n, m->x, m->err_d, st));
    const size_t layer_stride = (size_t)c.ctx * d;
    // rows [q | k | v] of window i -> cache positions 0..n-1 of stream i
    auto to_caches = [&](int l) -> int {
        if (kcs_dev && vcs_dev) return launch_scatter_kv(m->qkv, kcs_dev, vcs_dev, l * layer_stride, S, n, d, st);
        for (int i = 0; i < S; ++i) {
            const float* rows = m->qkv + (size_t)i * n * 3 * d;
            FC_CUDA(cudaMemcpy2DAsync(ss[i]->kc + l * layer_stride, (size_t)d * 4, rows + d, (size_t)3 * d * 4, (size_t)d * 4, n,
                                      cudaMemcpyDeviceToDevice, st));
            FC_CUDA(cudaMemcpy2DAsync(ss[i]->vc + l * layer_stride, (size_t)d * 4, rows + 2 * d, (size_t)3 * d * 4, (size_t)d * 4, n,
                                      cudaMemcpyDeviceToDevice, st));
        }
        return FC_OK;
    };
    if (tensor_path(m) && R >= 256) {
        // many rows: the window forward of the scoring path (tcgen05 GEMMs and attention on bf16 hi / lo
        // planes); the QKV product also leaves f32 rows, which feed the caches
        for (int l = 0; l < c.n_layer; ++l) {
            const LayerDev& L = m->layers[l];
            FC_TRY(launch_layernorm_planes(m->x, L.ln1g, L.ln1b, R, d, m->nhi, m->nlo, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.qkv, m->nhi, m->nlo, L.qkv_b, nullptr, EPI_NONE, m->qkv, nullptr, nullptr, R, 3 * d, m->tc_status, st));
            FC_TRY(to_caches(l));
            FC_TRY(launch_split_bf16(m->qkv, m->qkvhi, m->qkvlo, (size_t)R * 3 * d, st));
            FC_TRY(launch_attn_prefill_tc(m->qkvhi, m->qkvlo, S, n, d, c.n_head, m->atthi, m->attlo, m->tc_status, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.out, m->atthi, m->attlo, L.out_b, m->x, EPI_NONE, m->x, nullptr, nullptr, R, d, m->tc_status, st));
            FC_TRY(launch_layernorm_planes(m->x, L.ln2g, L.ln2b, R, d, m->nhi, m->nlo, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.up, m->nhi, m->nlo, L.up_b, nullptr, EPI_GELU, nullptr, m->hidhi, m->hidlo, R, F, m->tc_status, st));
            FC_TRY(launch_gemm_q8_bf16x3_ex(L.down, m->hidhi, m->hidlo, L.down_b, m->x, EPI_NONE, m->x, nullptr, nullptr, R, d, m->tc_status, st));
        }
    } else {
        for (int l = 0; l < c.n_layer; ++l) {
            const LayerDev& L = m->layers[l];
            FC_TRY(launch_layernorm(m->x, L.ln1g, L.ln1b, R, d, m->n, nullptr, st));
            FC_TRY(launch_gemm_q8_fp32(L.qkv, m->n, L.qkv_b, nullptr, EPI_NONE, m->qkv, R, 3 * d, st));
            FC_TRY(to_caches(l));
            FC_TRY(launch_attn_prefill(m->qkv, S, n, d, c.n_head, m->att, st));
            FC_TRY(launch_gemm_q8_fp32(L.out, m->att, L.out_b, m->x, EPI_NONE, m->x, R, d, st));
            FC_TRY(launch_layernorm(m->x, L.ln2g, L.ln2b, R, d, m->n, nullptr, st));
            FC_TRY(launch_gemm_q8_fp32(L.up, m->n, L.up_b, nullptr, EPI_GELU, m->hid, R, F, st));
            FC_TRY(launch_gemm_q8_fp32(L.down, m->hid, L.down_b, m->x, EPI_NONE, m->x, R, d, st));
        }
    }
    *used = 1;
    for (int i = 0; i < S; ++i) {
        fc_stream* s = ss[i];
        if (last_mode == STEP_NOHEAD) {
            bump_state_kernel<<<1, 1, 0, st>>>(s->state, n);
            FC_LAUNCHED();
            continue;
        }
        // the head sees the last row only; its tail advances the position by one
        bump_state_kernel<<<1, 1, 0, st>>>(s->state, n - 1);
        FC_LAUNCHED();
        FC_TRY(launch_layernorm(m->x + ((size_t)i * n + n - 1) * d, m->lnfg, m->lnfb, 1, d, s->n, s->state, st));
        GemvOut ol; ol.out[0] = s->logits;
        FC_TRY(launch_gemv_q8(m->head, s->n, nullptr, nullptr, EPI_NONE, ol, s->state, st));
        FC_TRY(launch_step_tail(s->logits, c.vocab, last_mode == STEP_PROBS ? s->probs : nullptr, last_mode == STEP_SELECT ? 1 : 0,
                                s->queue, s->queue_cap, s->state, nullptr, st));
    }
    return FC_OK;
}

// Feeds queue[0..n) (already uploaded) from the current position; the last step runs in
// `last_mode`, the ones before it skip the head (its output would be discarded).
static int feed_queued(fc_stream* s, int n, int last_mode) {
    int used = 0;
    FC_TRY(prime_batched(&s, 1, n, last_mode, &used));
    if (used) return FC_OK;
    return run_steps(s, n, STEP_NOHEAD, last_mode);
}

static int feed_ids(fc_stream* s, const int32_t* ids, int n, float* probs) {
    fc_model* m = s->m;
    const fc_config& c = m->cfg;
    FC_TRY(check_ids(m, ids, (size_t)n));
    if (s->host_pos + n > c.ctx)
        return fail(FC_E_DIM, "KvCache full (%d positions): clear and re-prime to continue", c.ctx);
    if (n == 0) return FC_OK;
    cudaStream_t st = m->st;
    FC_CUDA(cudaMemcpyAsync(s->queue, ids, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    FC_TRY(set_state(s, 0, 0, n, -1, /*keep_pos=*/1));
    FC_TRY(feed_queued(s, n, probs ? STEP_PROBS : STEP_NOHEAD));
    if (probs) FC_CUDA(cudaMemcpyAsync(probs, s->probs, (size_t)c.vocab * 4, cudaMemcpyDeviceToHost, st));
    StepState hs;
    FC_TRY(read_state(s, &hs));
    if (hs.error) return fail(hs.error, "decode step rejected a token or position on the device");
    s->host_pos = hs.pos;
    return FC_OK;
}

int fc_feed(fc_stream* s, int32_t token, float* probs) {
    if (!s) return fail(FC_E_ARG, "fc_feed: null stream");
    FC_CUDA(cudaSetDevice(s->m->device));
    return feed_ids(s, &token, 1, probs);
}

int fc_prime(fc_stream* s, const int32_t* ids, int n, float* probs) {
    if (!s || (n > 0 && !ids)) return fail(FC_E_ARG, "fc_prime: null argument");
    if (n < 0) return fail(FC_E_SHAPE, "fc_prime: n = %d", n);
    FC_TRY(fc_stream_reset(s));
    return feed_ids(s, ids, n, probs);
}

int fc_generate_greedy(fc_stream* s, const int32_t* prompt, int n, int max_new, int32_t eos,
                       const volatile int32_t* cancel, int32_t* out, int* n_out) {
    if (!s || !prompt || !n_out || (max_new > 0 && !out)) return fail(FC_E_ARG, "fc_generate_greedy: null argument");
    *n_out = 0;
    if (n <= 0) return fail(FC_E_SHAPE, "fc_generate_greedy: empty prompt (pass the BOS id, token_stream.rs:84-86)");
    if (max_new < 0) return fail(FC_E_SHAPE, "fc_generate_greedy: max_new = %d", max_new);
    fc_model* m = s->m;
    const fc_config& c = m->cfg;
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, prompt, (size_t)n));
    cudaStream_t st = m->st;
    const int cap = std::max(1, (int)c.ctx), keep = std::max(1, cap / 2);
    s->last_decode_ms = 0.0f;

    // window = the last `cap` prompt ids (token_stream.rs:87-89)
    std::vector<int32_t> window(prompt + std::max(0, n - cap), prompt + n);
    int made = 0;          // tokens already copied to `out` (earlier windows)
    bool done = false, cancelled = false;
    // Starts a window: reset, upload, prime. The last prime step selects the next token when
    // one is still wanted.
    auto start_window = [&](bool select) -> int {
        FC_TRY(fc_stream_reset(s));
        FC_CUDA(cudaMemcpyAsync(s->queue, window.data(), window.size() * 4, cudaMemcpyHostToDevice, st));
        FC_TRY(set_state(s, 0, 0, (int)window.size(), eos, 0));
        return feed_queued(s, (int)window.size(), select ? STEP_SELECT : STEP_PROBS);
    };
    // Reads back what the device appended to the current window; sets `done` on eos.
    auto harvest = [&]() -> int {
        StepState hs;
        FC_TRY(read_state(s, &hs));
        if (hs.error) return fail(hs.error, "decode step rejected a token or position on the device");
        const int have = hs.tail - (int)window.size();
        if (have > 0) {
            window.resize(hs.tail);
            FC_CUDA(cudaMemcpy(window.data() + hs.tail - have, s->queue + hs.tail - have, (size_t)have * 4, cudaMemcpyDeviceToHost));
            for (int i = 0; i < have && made < max_new; ++i) out[made++] = window[hs.tail - have + i];
        }
        s->host_pos = hs.pos;
        done = hs.done != 0;
        return FC_OK;
    };

    FC_TRY(start_window(max_new > 0));
    FC_CUDA(cudaEventRecord(s->ev0, st));
    int win_start_len = (int)window.size();  // ids in the window when it was primed
    int gen_win = max_new > 0 ? 1 : 0;       // tokens selected inside this window (issued)
    // feed i (1-based) pushes generated token i; it selects token i+1 unless it is the last.
    // Consecutive selecting feeds are issued as one batch of at most 32 steps.
    int i = 1;
    while (i <= max_new && !done) {
        if (cancel && *cancel) { cancelled = true; break; }
        if (win_start_len + gen_win > cap) {
            // the window outgrew the context: keep the last cap/2 ids and re-prime
            // (token_stream.rs:162-165)
            const bool select = i < max_new;
            FC_TRY(harvest());
            if (done) break;
            window.erase(window.begin(), window.end() - keep);
            FC_TRY(start_window(select));
            win_start_len = (int)window.size();
            gen_win = select ? 1 : 0;
            i += 1;
        } else {
            // selecting feeds i..max_new-1, as many as stay inside the context
            const int k = std::min(std::min(max_new - i, 32), cap - win_start_len - gen_win + 1);
            if (k >= 1) {
                FC_TRY(run_steps(s, k, STEP_SELECT, STEP_SELECT));
                gen_win += k;
                i += k;
            } else {
                FC_TRY(run_steps(s, 1, STEP_PROBS, STEP_PROBS));   // the last feed selects nothing
                i += 1;
            }
        }
        // eos can only be noticed on the host at a synchronisation point
        if (eos >= 0) FC_TRY(harvest());
    }
    FC_CUDA(cudaEventRecord(s->ev1, st));
    FC_TRY(harvest());
    FC_CUDA(cudaEventElapsedTime(&s->last_decode_ms, s->ev0, s->ev1));
    *n_out = made;
    if (cancelled) return fail(FC_E_CANCELLED, "generation cancelled after %d tokens", made);
    return FC_OK;
}

int fc_sample_logits(int device, const float* logits, int n, const fc_sampling* params, const int32_t* recent, int n_recent,
                     uint64_t* rng_state, int32_t* token) {
    if (!logits || !params || !rng_state || !token || (n_recent > 0 && !recent)) return fail(FC_E_ARG, "fc_sample_logits: null argument");
    if (n <= 0 || n_recent < 0) return fail(FC_E_SHAPE, "fc_sample_logits: n = %d, n_recent = %d", n, n_recent);
    FC_TRY(select_device(device));
    Arena a;
    float* d_logits = nullptr;
    int* d_recent = nullptr;
    unsigned long long* d_rng = nullptr;
    int* d_tok = nullptr;
    int rc = a.alloc_n(&d_logits, (size_t)n);
    if (rc == FC_OK) rc = a.alloc_n(&d_recent, (size_t)std::max(n_recent, 1));
    if (rc == FC_OK) rc = a.alloc_n(&d_rng, 1);
    if (rc == FC_OK) rc = a.alloc_n(&d_tok, 1);
    auto copy = [&](void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
        if (rc == FC_OK && bytes && cudaMemcpy(dst, src, bytes, kind) != cudaSuccess) rc = fail(FC_E_CUDA, "fc_sample_logits: copy failed");
    };
    copy(d_logits, logits, (size_t)n * 4, cudaMemcpyHostToDevice);
    copy(d_recent, recent, (size_t)n_recent * 4, cudaMemcpyHostToDevice);
    copy(d_rng, rng_state, 8, cudaMemcpyHostToDevice);
    if (rc == FC_OK) rc = launch_sample(d_logits, n, 0, *params, d_recent, n_recent, d_rng, nullptr, 0, nullptr, d_tok, nullptr);
    if (rc == FC_OK && cudaDeviceSynchronize() != cudaSuccess) rc = fail(FC_E_CUDA, "fc_sample_logits: the sampler failed");
    copy(token, d_tok, 4, cudaMemcpyDeviceToHost);
    copy(rng_state, d_rng, 8, cudaMemcpyDeviceToHost);
    a.release();
    return rc;
}

int fc_generate_sampled(fc_stream* s, const int32_t* prompt, int n, int max_new, int32_t eos, const fc_sampling* params,
                        uint64_t* rng_state, const volatile int32_t* cancel, int32_t* out, int* n_out) {
    if (!s || !prompt || !n_out || !params || !rng_state || (max_new > 0 && !out)) return fail(FC_E_ARG, "fc_generate_sampled: null argument");
    *n_out = 0;
    if (n <= 0) return fail(FC_E_SHAPE, "fc_generate_sampled: empty prompt (pass the BOS id, token_stream.rs:84-86)");
    if (max_new < 0) return fail(FC_E_SHAPE, "fc_generate_sampled: max_new = %d", max_new);
    fc_model* m = s->m;
    const fc_config& c = m->cfg;
    FC_CUDA(cudaSetDevice(m->device));
    FC_TRY(check_ids(m, prompt, (size_t)n));
    cudaStream_t st = m->st;
    const int cap = std::max(1, (int)c.ctx), keep = std::max(1, cap / 2);
    if (!s->rng_d) FC_TRY(s->arena.alloc_n(&s->rng_d, 1));
    FC_CUDA(cudaMemcpyAsync(s->rng_d, rng_state, 8, cudaMemcpyHostToDevice, st));
    s->last_decode_ms = 0.0f;
    // window = the last `cap` prompt ids (token_stream.rs:87-89); priming leaves the distribution
    // of the next token in s->probs
    std::vector<int32_t> window(prompt + std::max(0, n - cap), prompt + n);
    auto start_window = [&]() -> int {
        FC_TRY(fc_stream_reset(s));
        FC_CUDA(cudaMemcpyAsync(s->queue, window.data(), window.size() * 4, cudaMemcpyHostToDevice, st));
        FC_TRY(set_state(s, 0, 0, (int)window.size(), eos, 0));
        return feed_queued(s, (int)window.size(), STEP_PROBS);
    };
    FC_TRY(start_window());
    FC_CUDA(cudaEventRecord(s->ev0, st));
    int made = 0;
    bool cancelled = false, timed = false;
    int rc = FC_OK;
    while (made < max_new) {
        if (cancel && *cancel) { cancelled = true; break; }
        // draw from the current distribution with the window as `recent`; the token is appended
        // to the queue on the device, or `done` is raised on eos
        rc = launch_sample(s->probs, c.vocab, 1, *params, s->queue, 0, s->rng_d, s->queue, s->queue_cap, s->state, nullptr, st);
        if (rc != FC_OK) break;
        StepState hs;
        rc = read_state(s, &hs);
        if (rc != FC_OK) break;
        if (hs.error) { rc = fail(hs.error, "decode step rejected a token or position on the device"); break; }
        if (hs.done) break;                                   // eos: nothing was appended
        int32_t tok = 0;
        if (cudaMemcpy(&tok, s->queue + hs.tail - 1, 4, cudaMemcpyDeviceToHost) != cudaSuccess) { rc = fail(FC_E_CUDA, "token download failed"); break; }
        out[made++] = tok;
        // the feed (or re-prime) after the last requested token keeps the stream continuable, as the reference's call
        // order does, but its distribution is not used here: it stays outside the timed region
        if (made == max_new) { FC_CUDA(cudaEventRecord(s->ev1, st)); timed = true; }
        window.push_back(tok);
        if ((int)window.size() > cap) {
            // the window outgrew the context: keep the last cap/2 ids and re-prime (token_stream.rs:162-165)
            window.erase(window.begin(), window.end() - keep);
            rc = start_window();
        } else {
            rc = run_steps(s, 1, STEP_PROBS, STEP_PROBS);     // feed(next): the distribution of the token after it
        }
        if (rc != FC_OK) break;
    }
    if (rc == FC_OK) {
        if (!timed) FC_CUDA(cudaEventRecord(s->ev1, st));
        StepState hs;
        rc = read_state(s, &hs);
        if (rc == FC_OK && hs.error) rc = fail(hs.error, "decode step rejected a token or position on the device");
        if (rc == FC_OK) {
            s->host_pos = hs.pos;
            FC_CUDA(cudaEventElapsedTime(&s->last_decode_ms, s->ev0, s->ev1));
        }
    }
    FC_CUDA(cudaMemcpy(rng_state, s->rng_d, 8, cudaMemcpyDeviceToHost));
    if (rc != FC_OK) return rc;
    *n_out = made;
    if (cancelled) return fail(FC_E_CANCELLED, "generation cancelled after %d tokens", made);
    return FC_OK;
}

// ------------------------------------------------------------------- lock-step decode
// Fragment-major copies of every matrix, made once per model on the first batched decode.
static int batch_make_frags(fc_model* m) {
    BatchCtx& b = m->batch;
    if (b.frags) return FC_OK;
    cudaStream_t st = m->st;
    auto make = [&](const QMat& w, QFrag* out) -> int {
        void *q = nullptr, *d = nullptr;
        FC_TRY(b.frag_arena.alloc(&q, frag_quant_bytes(w)));
        FC_TRY(b.frag_arena.alloc(&d, frag_scale_bytes(w)));
        FC_TRY(launch_repack_frag(w, q, d, st));
        out->q = q; out->d = d; out->N = w.N; out->K = w.K; out->N_pad = w.N_pad;
        return FC_OK;
    };
    const int L = m->cfg.n_layer;
    b.qkv.resize(L); b.out.resize(L); b.up.resize(L); b.down.resize(L);
    int rc = FC_OK;
    for (int l = 0; l < L && rc == FC_OK; ++l) {
        rc = make(m->layers[l].qkv, &b.qkv[l]);
        if (rc == FC_OK) rc = make(m->layers[l].out, &b.out[l]);
        if (rc == FC_OK) rc = make(m->layers[l].up, &b.up[l]);
        if (rc == FC_OK) rc = make(m->layers[l].down, &b.down[l]);
    }
    if (rc == FC_OK) rc = make(m->head, &b.head);
    if (rc == FC_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(FC_E_CUDA, "fragment-major weight copy failed");
    if (rc != FC_OK) { b.frag_arena.release(); return rc; }
    b.frags = true;
    return FC_OK;
}

static int batch_ensure(fc_model* m, int S, int out_cap) {
    BatchCtx& b = m->batch;
    if (S <= b.cap && out_cap <= b.out_cap) return FC_OK;
    FC_CUDA(cudaStreamSynchronize(m->st));
    if (b.graph) { cudaGraphExecDestroy(b.graph); b.graph = nullptr; }
    if (b.graph4) { cudaGraphExecDestroy(b.graph4); b.graph4 = nullptr; }
    b.graph_S = 0;
    b.arena.release();
    b.cap = b.out_cap = 0;
    const fc_config& c = m->cfg;
    // two f16 columns per stream; a ragged last group reads (never uses) up to 128 columns past its own
    const size_t cap = std::max(S, b.cap), oc = std::max(out_cap, b.out_cap), C = kBatchMaxStreams * 2 + 128;
    const size_t d = c.d_model, F = c.d_ff;
    Arena& a = b.arena;
    FC_TRY(a.alloc_n(&b.x, cap * d));
    FC_TRY(a.alloc_n(&b.x2, cap * d));
    FC_TRY(a.alloc_n(&b.part, (size_t)skinny_max_splits() * cap * d));
    FC_TRY(a.alloc_n(&b.qkv_f, cap * 3 * d));
    FC_TRY(a.alloc_n(&b.logits, cap * (size_t)m->head.N_pad));
    FC_TRY(a.alloc(&b.xp, C * d * 2));
    FC_TRY(a.alloc(&b.ap, C * d * 2));
    FC_TRY(a.alloc(&b.hp, C * F * 2));
    // rows past the live streams are read by the MMA tiles: they stay zero
    FC_CUDA(cudaMemsetAsync(b.xp, 0, C * d * 2, m->st));
    FC_CUDA(cudaMemsetAsync(b.ap, 0, C * d * 2, m->st));
    FC_CUDA(cudaMemsetAsync(b.hp, 0, C * F * 2, m->st));
    FC_TRY(a.alloc_n(&b.cur, cap));
    FC_TRY(a.alloc_n(&b.done, cap));
    FC_TRY(a.alloc_n(&b.n_out, cap));
    FC_TRY(a.alloc_n(&b.out_tok, cap * std::max<size_t>(oc, 1)));
    FC_TRY(a.alloc_n(&b.pos, kBatchMaxStreams));   // one position word per group of the step graph, all equal
    FC_TRY(a.alloc_n(&b.kcs, cap));
    FC_TRY(a.alloc_n(&b.vcs, cap));
    FC_TRY(a.alloc_n(&b.queues, cap));
    FC_TRY(a.alloc_n(&b.states, cap));
    b.cap = (int)cap;
    b.out_cap = (int)oc;
    return FC_OK;
}

// The buffers of one group of streams (streams s0 .. s0 + S of a wave). Every per-stream array is indexed by the
// stream, so a group is a set of offsets into the wave's buffers, its own position word and the CUDA stream its
// kernels are issued on.
struct BatchView {
    int S;
    float *x, *x2, *part, *qkv_f, *logits;
    void *xp, *ap, *hp;
    int *cur, *done, *n_out, *out_tok, *pos;
    float **kcs, **vcs;
    cudaStream_t st;
    int max_warps;                     // per CTA of the products: fewer when several groups run side by side
    bool long_k_block;                 // the 32-warp tile of the long-K products: up to two groups
};

static BatchView batch_view(fc_model* m, int s0, int S, int group_index, cudaStream_t st, int n_groups = 1) {
    const fc_config& c = m->cfg;
    BatchCtx& b = m->batch;
    const size_t d = c.d_model, F = c.d_ff, o = (size_t)s0;
    BatchView v;
    v.S = S;
    v.x = b.x + o * d;
    v.x2 = b.x2 + o * d;
    v.part = b.part + (size_t)skinny_max_splits() * o * d;        // [splits][S][d] of the group
    v.qkv_f = b.qkv_f + o * 3 * d;
    v.logits = b.logits + o * (size_t)m->head.N_pad;
    v.xp = (char*)b.xp + 2 * o * d * 2;                           // two f16 columns per stream
    v.ap = (char*)b.ap + 2 * o * d * 2;
    v.hp = (char*)b.hp + 2 * o * F * 2;
    v.cur = b.cur + o; v.done = b.done + o; v.n_out = b.n_out + o;
    v.out_tok = b.out_tok + o * (size_t)b.out_cap;
    v.pos = b.pos + group_index;
    v.kcs = b.kcs + o; v.vcs = b.vcs + o;
    v.st = st;
    v.max_warps = n_groups > 1 ? 8 : 16;
    v.long_k_block = n_groups <= 2;
    return v;
}

// The tail of a step: final LayerNorm (model.rs:51-71 layer list: ..., LayerNorm, Linear, Softmax), head,
// greedy pick. With `part` the last down-projection is still in partial sums, which the LayerNorm adds.
static int batch_head_and_pick(fc_model* m, const BatchView& v, int eos, const float* x, const float* part, int n_part,
                               const float* part_bias, float* x_other, int advance) {
    const fc_config& c = m->cfg;
    BatchCtx& b = m->batch;
    FC_TRY(launch_ln_rows_f16(x, part, n_part, part_bias, x_other, m->lnfg, m->lnfb, v.S, c.d_model, v.xp, v.st));
    SkinnyOut out;
    out.max_warps = v.max_warps; out.long_k_block = v.long_k_block;
    out.y = v.logits; out.ldy = m->head.N_pad;
    FC_TRY(launch_skinny_q8(b.head, v.S, v.xp, nullptr, EPI_NONE, out, nullptr, v.st));
    return launch_pick_batch(v.logits, m->head.N_pad, c.vocab, v.S, eos, v.cur, v.done, v.n_out, v.out_tok, b.out_cap, v.pos, advance, v.st);
}

// One step for the S streams of a group: CachedTransformer::feed (cached.rs:100-125) on every stream's current
// token at the shared position, then the greedy pick per stream. Seven kernels per block.
//  * Up to 16 streams every kernel is a chain of a few memory round trips and nothing else: the
//    out- and down-projections add bias and residual in their own epilogue (in place).
//  * Beyond that the out- and down-projections split K over CTAs (their 1024-odd output rows
//    alone would leave most SMs idle) and leave partial sums; the LayerNorm kernel that reads the
//    residual stream next adds them, the bias and the residual in a fixed order
//    (transformer.rs:272,293).
static int batch_launch_step(fc_model* m, const BatchView& v, int eos) {
    const fc_config& c = m->cfg;
    BatchCtx& b = m->batch;
    cudaStream_t st = v.st;
    const int S = v.S, d = c.d_model, F = c.d_ff;
    const size_t layer_stride = (size_t)c.ctx * d;
    const bool split_k = S > 16;
    FC_TRY(launch_embed_batch(m->tok, m->pos, v.cur, v.pos, S, v.x, st));
    float *x = v.x, *x_other = v.x2;       // the stream as of the last completed residual add, and the other buffer
    const float* part_bias = nullptr;      // bias of the product whose partial sums are pending
    int n_part = 0;
    // LayerNorm of the residual stream, completed first when partial sums are pending
    auto normed = [&](const float* g, const float* be) -> int {
        FC_TRY(launch_ln_rows_f16(x, n_part > 0 ? v.part : nullptr, n_part, part_bias, x_other, g, be, S, d, v.xp, st));
        if (n_part > 0) std::swap(x, x_other);   // the completed stream now lives in the other buffer
        n_part = 0;
        part_bias = nullptr;
        return FC_OK;
    };
    // x <- x + (W in + bias): as partial sums for the next LayerNorm, or finished in the epilogue
    auto project_add = [&](const QFrag& w, const void* in, const float* bias) -> int {
        SkinnyOut o;
        o.max_warps = v.max_warps; o.long_k_block = v.long_k_block;
        if (split_k) {
            o.part = v.part;
            FC_TRY(launch_skinny_q8(w, S, in, nullptr, EPI_NONE, o, &n_part, st));
            part_bias = bias;
            return FC_OK;
        }
        o.y = x; o.ldy = d; o.residual = x;
        return launch_skinny_q8(w, S, in, bias, EPI_NONE, o, nullptr, st);
    };
    SkinnyOut oq, oh;
    oq.max_warps = oh.max_warps = v.max_warps;
    oq.long_k_block = oh.long_k_block = v.long_k_block;
    oq.y = v.qkv_f; oq.ldy = 3 * d;
    oh.planes = v.hp; oh.ldp = F;
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerDev& L = m->layers[l];
        FC_TRY(normed(L.ln1g, L.ln1b));
        FC_TRY(launch_skinny_q8(b.qkv[l], S, v.xp, L.qkv_b, EPI_NONE, oq, nullptr, st));
        FC_TRY(launch_attn_decode_batch(v.qkv_f, v.kcs, v.vcs, l * layer_stride, d, c.n_head, c.ctx, v.pos, S, v.ap, st));
        FC_TRY(project_add(b.out[l], v.ap, L.out_b));
        FC_TRY(normed(L.ln2g, L.ln2b));
        FC_TRY(launch_skinny_q8(b.up[l], S, v.xp, L.up_b, EPI_GELU, oh, nullptr, st));
        FC_TRY(project_add(b.down[l], v.hp, L.down_b));
    }
    return batch_head_and_pick(m, v, eos, x, v.part, n_part, part_bias, x_other, 1);
}

// Streams per group of the step graph. Every step kernel is a chain of memory round trips that leaves most of the
// GPU idle, and its duration hardly falls with fewer streams, so groups run as parallel branches of the graph and
// their chains overlap. The weights are then read once per group, the re-reads coming from L2 (a block's matrices
// are a few MB and the branches stay within a block or two of each other). Measured on the 24-block, 1024-wide
// shape with 64 streams: one group 1.63 ms per step, groups of 32 1.47 ms, of 16 1.37 ms, of 8 1.55 ms.
// FERRUM_LOCKSTEP_GROUP=<n> overrides the choice (a tuning aid; results do not depend on it beyond the
// summation order of the kernels that n selects).
static int batch_group_size(int S) {
    if (const char* e = getenv("FERRUM_LOCKSTEP_GROUP")) {
        const int forced = atoi(e);
        if (forced > 0) return std::min(forced, kBatchMaxStreams);
    }
    return S > 16 ? 16 : S;
}

// All groups of one step on the capture: group 0 on the model's stream, the others on side streams forked from
// it and joined back.
static int batch_launch_groups(fc_model* m, int S, int eos, int group) {
    BatchCtx& b = m->batch;
    const int n_groups = (S + group - 1) / group;
    while ((int)b.side.size() < n_groups - 1) {
        cudaStream_t s = nullptr;
        cudaEvent_t e = nullptr;
        FC_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        b.side.push_back(s);
        FC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        b.side_done.push_back(e);
    }
    if (!b.fork) FC_CUDA(cudaEventCreateWithFlags(&b.fork, cudaEventDisableTiming));
    if (n_groups > 1) FC_CUDA(cudaEventRecord(b.fork, m->st));
    for (int g = 1; g < n_groups; ++g) {
        FC_CUDA(cudaStreamWaitEvent(b.side[g - 1], b.fork, 0));
        FC_TRY(batch_launch_step(m, batch_view(m, g * group, std::min(group, S - g * group), g, b.side[g - 1], n_groups), eos));
        FC_CUDA(cudaEventRecord(b.side_done[g - 1], b.side[g - 1]));
    }
    FC_TRY(batch_launch_step(m, batch_view(m, 0, std::min(group, S), 0, m->st, n_groups), eos));
    for (int g = 1; g < n_groups; ++g) FC_CUDA(cudaStreamWaitEvent(m->st, b.side_done[g - 1], 0));
    return FC_OK;
}

// The step is launch-bound (7 small kernels per block): it is captured once into a CUDA graph and
// replayed; position and tokens are read from device memory, so no node changes between steps.
// n_steps: 1 or 4 consecutive steps in one launch.
static int batch_run_steps(fc_model* m, int S, int eos, int n_steps) {
    BatchCtx& b = m->batch;
    const int group = batch_group_size(S);
    if (b.graph_S != S || b.graph_eos != eos || b.graph_cap != b.out_cap || b.graph_group != group) {
        if (b.graph) { cudaGraphExecDestroy(b.graph); b.graph = nullptr; }
        if (b.graph4) { cudaGraphExecDestroy(b.graph4); b.graph4 = nullptr; }
        b.graph_S = S; b.graph_eos = eos; b.graph_cap = b.out_cap; b.graph_group = group;
    }
    cudaGraphExec_t& exec = n_steps == 4 ? b.graph4 : b.graph;
    int& nodes = n_steps == 4 ? b.graph4_nodes : b.graph_nodes;
    if (!exec) {
        cudaGraph_t g = nullptr;
        const int64_t before = g_launches;
        FC_CUDA(cudaStreamBeginCapture(m->st, cudaStreamCaptureModeThreadLocal));
        int rc = FC_OK;
        for (int k = 0; k < n_steps && rc == FC_OK; ++k) rc = batch_launch_groups(m, S, eos, group);
        const cudaError_t e = cudaStreamEndCapture(m->st, &g);
        nodes = (int)(g_launches - before);
        g_launches = before;
        if (rc != FC_OK) { if (g) cudaGraphDestroy(g); return rc; }
        FC_CUDA(e);
        const cudaError_t ei = cudaGraphInstantiate(&exec, g, 0);
        cudaGraphDestroy(g);
        FC_CUDA(ei);
    }
    FC_CUDA(cudaGraphLaunch(exec, m->st));
    g_launches += nodes;
    return FC_OK;
}

// Independent greedy streams on one GPU (the 64-stream workload is split over GPUs above the
// ABI). Each stream is a CachedTransformer of its own (its own KV caches and window); the
// streams advance in lock step, up to 64 at a time: the prompts are primed as one batch of
// windows, then every step runs all streams through each Q8_0 matrix at once, so the weights
// are read once per step whatever the number of streams. A stream that picks `eos` stops
// emitting; the others go on. The reference's extra feed after the last sampled token
// (token_stream.rs:181-186) is not run: its distribution is never used.
// Streams that would outgrow the context (they need the re-prime of token_stream.rs:162-165)
// and single streams run one after the other through fc_generate_greedy.
int fc_decode_batch(fc_model* m, int n_streams, const int32_t* prompts, int prompt_len, int max_new, int32_t eos,
                    int32_t* out, int* n_out) {
    if (!m || !prompts || !n_out || (max_new > 0 && !out)) return fail(FC_E_ARG, "fc_decode_batch: null argument");
    if (n_streams < 0 || prompt_len <= 0 || max_new < 0) return fail(FC_E_SHAPE, "fc_decode_batch: bad sizes");
    FC_CUDA(cudaSetDevice(m->device));
    const fc_config& c = m->cfg;
    while ((int)m->pool.size() < n_streams) {
        fc_stream* s = nullptr;
        FC_TRY(fc_stream_create(m, &s));
        m->pool.push_back(s);
    }
    m->last_batch_ms = 0.0f;
    m->last_batch_prime_ms = 0.0f;
    if (!m->ev_prime) FC_CUDA(cudaEventCreate(&m->ev_prime));
    const int hd = c.d_model / c.n_head;
    const bool lock_step = n_streams >= 2 && max_new > 0 && prompt_len + max_new <= c.ctx && hd <= 64 && hd % 4 == 0 &&
                           (size_t)(c.ctx + 4 + 64 + 1024) * sizeof(float) <= 48 * 1024;
    if (!lock_step) {
        for (int i = 0; i < n_streams; ++i) {
            FC_TRY(fc_generate_greedy(m->pool[i], prompts + (size_t)i * prompt_len, prompt_len, max_new, eos, nullptr,
                                      out + (size_t)i * max_new, n_out + i));
            m->last_batch_ms += m->pool[i]->last_decode_ms;
        }
        return FC_OK;
    }
    FC_TRY(check_ids(m, prompts, (size_t)n_streams * prompt_len));
    FC_TRY(batch_make_frags(m));
    FC_TRY(batch_ensure(m, std::min(n_streams, kBatchMaxStreams), max_new));
    BatchCtx& b = m->batch;
    cudaStream_t st = m->st;
    FC_CUDA(cudaEventRecord(m->ev0, st));
    for (int w0 = 0; w0 < n_streams; w0 += kBatchMaxStreams) {
        const int S = std::min(kBatchMaxStreams, n_streams - w0);
        if (w0 > 0) FC_CUDA(cudaEventRecord(m->ev1, st));   // start of this wave's prime (the first wave starts at ev0)
        // prime: all prompts of the wave as one batch of windows; the last row of each selects token 1
        std::vector<fc_stream*> wv;
        for (int i = 0; i < S; ++i) {
            fc_stream* s = m->pool[w0 + i];
            s->table = 0;
            FC_TRY(fc_stream_reset(s));
            FC_CUDA(cudaMemcpyAsync(s->queue, prompts + (size_t)(w0 + i) * prompt_len, (size_t)prompt_len * 4, cudaMemcpyHostToDevice, st));
            FC_TRY(set_state(s, 0, 0, prompt_len, eos, 0));
            wv.push_back(s);
        }
        // per-stream pointers for the step kernels
        std::vector<float*> kcs(S), vcs(S);
        std::vector<int*> queues(S);
        std::vector<StepState*> states(S);
        for (int i = 0; i < S; ++i) { kcs[i] = wv[i]->kc; vcs[i] = wv[i]->vc; queues[i] = wv[i]->queue; states[i] = wv[i]->state; }
        FC_CUDA(cudaMemcpyAsync(b.kcs, kcs.data(), S * sizeof(float*), cudaMemcpyHostToDevice, st));
        FC_CUDA(cudaMemcpyAsync(b.vcs, vcs.data(), S * sizeof(float*), cudaMemcpyHostToDevice, st));
        FC_CUDA(cudaMemcpyAsync(b.queues, queues.data(), S * sizeof(int*), cudaMemcpyHostToDevice, st));
        FC_CUDA(cudaMemcpyAsync(b.states, states.data(), S * sizeof(StepState*), cudaMemcpyHostToDevice, st));
        FC_CUDA(cudaStreamSynchronize(st));   // the host vectors above go out of use
        int used = 0;
        FC_TRY(prime_batched(wv.data(), S, prompt_len, STEP_NOHEAD, &used, b.kcs, b.vcs));
        if (used) {
            // the head sees the last row of every window: final LayerNorm, one product for all streams, pick of token 1
            const int d = c.d_model;
            FC_TRY(launch_gather_last_rows(m->x, S, prompt_len, d, b.x, st));
            FC_TRY(launch_batch_init(S, prompt_len, b.done, b.n_out, b.cur, b.pos, st));
            FC_TRY(batch_head_and_pick(m, batch_view(m, 0, S, 0, st), eos, b.x, nullptr, 0, nullptr, nullptr, 0));
        } else {
            // prompts too short for a window forward: token by token per stream; the last step selects token 1
            for (int i = 0; i < S; ++i) FC_TRY(run_steps(wv[i], prompt_len, STEP_NOHEAD, STEP_SELECT));
            FC_TRY(launch_gather_first(b.queues, b.states, prompt_len, S, b.cur, b.done, b.n_out, b.out_tok, b.out_cap, b.pos, st));
        }
        FC_CUDA(cudaEventRecord(m->ev_prime, st));
        std::vector<int> done(S, 0);
        for (int i = 1; i < max_new; ++i) {        // step i feeds token i and picks token i + 1
            // four steps per launch while they fit (steps 1-4, 5-8, ...: a chunk ends where the eos check falls)
            const int n_steps = (i % 4 == 1 && i + 3 < max_new) ? 4 : 1;
            FC_TRY(batch_run_steps(m, S, eos, n_steps));
            i += n_steps - 1;
            if (eos >= 0 && (i % 16 == 0)) {          // eos can only be noticed on the host at a synchronisation point
                FC_CUDA(cudaMemcpyAsync(done.data(), b.done, S * sizeof(int), cudaMemcpyDeviceToHost, st));
                FC_CUDA(cudaStreamSynchronize(st));
                if (std::all_of(done.begin(), done.end(), [](int v) { return v != 0; })) break;
            }
        }
        std::vector<int> cnt(S);
        FC_CUDA(cudaMemcpyAsync(done.data(), b.done, S * sizeof(int), cudaMemcpyDeviceToHost, st));
        std::vector<int32_t> toks((size_t)S * b.out_cap);
        int pos_h = 0;
        FC_CUDA(cudaMemcpyAsync(cnt.data(), b.n_out, S * sizeof(int), cudaMemcpyDeviceToHost, st));
        FC_CUDA(cudaMemcpyAsync(toks.data(), b.out_tok, toks.size() * 4, cudaMemcpyDeviceToHost, st));
        FC_CUDA(cudaMemcpyAsync(&pos_h, b.pos, sizeof(int), cudaMemcpyDeviceToHost, st));
        FC_CUDA(cudaStreamSynchronize(st));
        {
            float pm = 0.0f;
            FC_CUDA(cudaEventElapsedTime(&pm, w0 > 0 ? m->ev1 : m->ev0, m->ev_prime));
            m->last_batch_prime_ms += pm;
        }
        for (int i = 0; i < S; ++i)
            if (done[i] == 2) return fail(FC_E_CUDA, "fc_decode_batch: stream %d produced no finite logit", w0 + i);
        for (int i = 0; i < S; ++i) {
            const int have = std::min(cnt[i], max_new);
            std::copy(toks.begin() + (size_t)i * b.out_cap, toks.begin() + (size_t)i * b.out_cap + have, out + (size_t)(w0 + i) * max_new);
            n_out[w0 + i] = have;
            wv[i]->host_pos = pos_h;
        }
    }
    FC_CUDA(cudaEventRecord(m->ev1, st));
    FC_CUDA(cudaStreamSynchronize(st));
    FC_CUDA(cudaEventElapsedTime(&m->last_batch_ms, m->ev0, m->ev1));
    return FC_OK;
}

float fc_last_batch_ms(const fc_model* m) { return m ? m->last_batch_ms : 0.0f; }
float fc_last_batch_prime_ms(const fc_model* m) { return m ? m->last_batch_prime_ms : 0.0f; }

}  // extern "C"

// ---------------------------------------------------------------- several devices, one call
namespace {
// Runs fn(i, first, last) for every model on a host thread of its own (one handle = one GPU = one host thread
// at a time, as everywhere in this ABI), item i * n / n_models .. (i + 1) * n / n_models each. The first
// failure (in model order) is returned with its message; kernel launches are credited to the caller.
template <class Fn>
int run_on_models(int n_models, int n_items, Fn fn) {
    std::vector<int> rc(n_models, FC_OK);
    std::vector<std::string> msg(n_models);
    std::vector<int64_t> launches(n_models, 0);
    std::vector<std::thread> workers;
    for (int i = 0; i < n_models; ++i) {
        const int first = (int)((long long)i * n_items / n_models), last = (int)((long long)(i + 1) * n_items / n_models);
        workers.emplace_back([&, i, first, last] {
            if (last > first) rc[i] = fn(i, first, last);
            if (rc[i] != FC_OK) msg[i] = fc::g_err_text();
            launches[i] = fc::g_launches;
        });
    }
    for (auto& w : workers) w.join();
    for (int i = 0; i < n_models; ++i) fc::g_launches += launches[i];
    for (int i = 0; i < n_models; ++i)
        if (rc[i] != FC_OK) return fail(rc[i], "model %d of %d: %s", i, n_models, msg[i].c_str());
    return FC_OK;
}
}  // namespace

extern "C" {

int fc_score_sequences_multi(fc_model* const* models, int n_models, const int32_t* ids, int n_seq, int seq_len, int batch_windows,
                             fc_score* scores, float* lp) {
    if (!models || n_models <= 0 || !ids || !scores) return fail(FC_E_ARG, "fc_score_sequences_multi: null argument");
    for (int i = 0; i < n_models; ++i)
        if (!models[i]) return fail(FC_E_ARG, "fc_score_sequences_multi: model %d is null", i);
    if (n_seq < 0 || seq_len < 0) return fail(FC_E_SHAPE, "fc_score_sequences_multi: negative size");
    return run_on_models(n_models, n_seq, [&](int i, int a, int b) {
        return fc_score_sequences(models[i], ids + (size_t)a * seq_len, b - a, seq_len, batch_windows, scores + a,
                                  lp ? lp + (size_t)a * seq_len : nullptr);
    });
}

int fc_decode_batch_multi(fc_model* const* models, int n_models, int n_streams, const int32_t* prompts, int prompt_len, int max_new,
                          int32_t eos, int32_t* out, int* n_out) {
    if (!models || n_models <= 0 || !prompts || !n_out || (max_new > 0 && !out)) return fail(FC_E_ARG, "fc_decode_batch_multi: null argument");
    for (int i = 0; i < n_models; ++i)
        if (!models[i]) return fail(FC_E_ARG, "fc_decode_batch_multi: model %d is null", i);
    if (n_streams < 0 || prompt_len <= 0 || max_new < 0) return fail(FC_E_SHAPE, "fc_decode_batch_multi: bad sizes");
    return run_on_models(n_models, n_streams, [&](int i, int a, int b) {
        return fc_decode_batch(models[i], b - a, prompts + (size_t)a * prompt_len, prompt_len, max_new, eos, out + (size_t)a * max_new, n_out + a);
    });
}

int fc_debug_set_wait_budget(long long cycles, int withhold_producers) {
    if (cycles <= 0) return fail(FC_E_ARG, "fc_debug_set_wait_budget: cycles = %lld", cycles);
    g_debug.wait_cycles = cycles;
    g_debug.withhold = withhold_producers != 0;
    return FC_OK;
}

}  // extern "C"
