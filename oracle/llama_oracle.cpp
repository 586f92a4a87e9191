// llama_oracle — CPU restatement of Ferrum's imported Llama / Qwen decoder
// (ferrum_core/src/llm.rs, llm_score.rs), linked into libferrum_oracle.so.
//
// TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against. Nothing in the
// shipped library links, loads or calls it.
//
// Parity status: the Rust reference cannot be compiled in this environment, so the restatement
// is pinned against the known-answer values of the reference's own unit tests — RMSNorm
// formula and unit RMS (llm.rs:791-812), RoPE identity at position 0, norm preservation,
// NORM/NEOX difference, unit factors, the hand-computed frequency-factor rotations and the
// linear factor (llm.rs:817-933), the window plans and log-softmax of llm_score.rs:104-138 —
// and at cross-path level (KV-cached == full forward, llm.rs:974-1160). Absolute logits of a
// real checkpoint are "parity unpinned": the reference holds none.
//
// Arithmetic rules: f32 everywhere except where the reference uses f64 (the RoPE frequency,
// the scorer's log-softmax), products added in ascending k, bias added last, no FMA contraction
// (-ffp-contract=off), glibc sinf/cosf/expf/sqrtf/exp/log.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {
// ferrum_oracle.cpp
void fo_linear(const float* x, const float* w_kn, const float* bias, int m, int k, int n, float* y, int threads);
void fo_q8_0_expand_kn(const void* wq, int n, int k, float* w_kn);
void fo_q8_0_decode(const uint8_t* raw, size_t n, float* out);
int fo_argmax_first(const float* x, int n);
size_t fo_rowq_packed_len(int rows, int cols, int kind);
void fo_rowq_from_f32(const float* data, int rows, int cols, int kind, float* scales, uint8_t* q);
void fo_rowq_linear(const float* x, const uint8_t* q, const float* scales, int kind, const float* bias, int m, int k, int n, float* y);
int fo_sample_with_params(const float* logits, int n, float temperature, int top_k, float top_p, float rep_penalty,
                          const int32_t* recent, int n_recent, uint64_t* state);
}

namespace {

// Mirrors of the C ABI structs (include/ferrum_cuda.h).
struct Cfg {
    int32_t vocab, d, n_layer, n_head, n_kv, hd, ff, rope_dim;
    float rope_base;
    int32_t rope_type;
    float linear;
    float eps;
    int32_t ctx, tied, math_mode;
};
struct LayerW {
    const float* attn_norm;
    const void *wq, *wk, *wv, *wo;
    const float *bq, *bk, *bv;
    const float* ffn_norm;
    const void *gate, *up, *down;
};
struct Weights {
    const void* token_embd;
    const LayerW* layers;
    const float* output_norm;
    const void* output;
    const float* rope_freqs;
};

struct Lin {                     // Linear (layer/linear.rs): weight [in][out], bias [out]
    std::vector<float> w, b;
    int in = 0, out = 0;
    void load(const void* q8, const float* bias, int out_f, int in_f) {
        in = in_f; out = out_f;
        w.resize((size_t)in * out);
        fo_q8_0_expand_kn(q8, out, in, w.data());
        b.assign(out, 0.0f);
        if (bias) std::memcpy(b.data(), bias, (size_t)out * 4);
    }
    // Linear::quantized (layer/linear.rs:98-130) as gguf/llama.rs:13-27 builds it: the weight packed by
    // QWeight::from_f32 (quant.rs:164-212), forward = ops::qlinear (layer/linear.rs:191-194, ops.rs:316-377)
    int kind = -1;
    std::vector<uint8_t> q;
    std::vector<float> scales;
    void pack(int k) {
        kind = k;
        q.assign(fo_rowq_packed_len(in, out, k), 0);
        scales.assign(in, 0.0f);
        fo_rowq_from_f32(w.data(), in, out, k, scales.data(), q.data());
    }
    void forward(const float* x, int rows, float* y, int threads) const {
        if (kind >= 0) fo_rowq_linear(x, q.data(), scales.data(), kind, b.data(), rows, in, out, y);
        else fo_linear(x, w.data(), b.data(), rows, in, out, y, threads);
    }
};

// llm.rs:57-64 RmsNorm::forward_row.
void rmsnorm_row(const float* x, const float* w, float eps, int dim, float* out) {
    float ss = 0.0f;
    for (int i = 0; i < dim; ++i) ss += x[i] * x[i];
    const float ms = ss / (float)dim;
    const float inv = 1.0f / std::sqrt(ms + eps);
    for (int i = 0; i < dim; ++i) out[i] = x[i] * inv * w[i];
}

// llm.rs:129-132 RopeScaling::angle and llm.rs:158-185 apply_rope.
void apply_rope(float* x, int n_heads, int hd, int rope_dim, int pos, float base, int neox, const float* ff, int n_ff, float linear) {
    const int half = rope_dim / 2;
    for (int h = 0; h < n_heads; ++h) {
        const int off = h * hd;
        for (int i = 0; i < half; ++i) {
            const float freq = (float)std::pow((double)base, -2.0 * (double)i / (double)rope_dim);
            const float f = i < n_ff ? ff[i] : 1.0f;
            const float theta = (float)pos * freq / f * (1.0f / linear);
            const float s = sinf(theta), c = cosf(theta);
            const int ia = neox ? off + i : off + 2 * i, ib = neox ? off + i + half : off + 2 * i + 1;
            const float a = x[ia], b = x[ib];
            x[ia] = a * c - b * s;
            x[ib] = a * s + b * c;
        }
    }
}

struct Layer {
    std::vector<float> attn_norm, ffn_norm;
    Lin wq, wk, wv, wo, gate, up, down;
};

struct Model {
    Cfg c;
    std::vector<float> tok;      // [V][d] f32 (llm.rs:552-553)
    std::vector<Layer> layers;
    std::vector<float> out_norm, ff;
    Lin head;
    int threads = 1;
    int q_dim() const { return c.n_head * c.hd; }
    int kv_dim() const { return c.n_kv * c.hd; }
};

struct Cache {
    Model* m;
    std::vector<std::vector<float>> k, v;   // per layer [len * kv_dim]
    int pos = 0;
};

void rope(const Model& m, float* x, int heads, int pos) {
    apply_rope(x, heads, m.c.hd, m.c.rope_dim, pos, m.c.rope_base, m.c.rope_type == 1, m.ff.data(), (int)m.ff.size(), m.c.linear);
}

// llm.rs:276-301 Attention::project.
void project(const Model& m, const Layer& L, const float* x, int pos, float* q, float* k, float* v) {
    L.wq.forward(x, 1, q, 1);
    L.wk.forward(x, 1, k, 1);
    L.wv.forward(x, 1, v, 1);
    rope(m, q, m.c.n_head, pos);
    rope(m, k, m.c.n_kv, pos);
}

// llm.rs:305-341 Attention::attend.
void attend(const Model& m, const float* q, const float* kc, const float* vc, int len, float* out) {
    const int hd = m.c.hd, kv_dim = m.kv_dim(), group = m.c.n_head / m.c.n_kv;
    const float scale = 1.0f / std::sqrt((float)hd);
    std::vector<float> scores(len);
    for (int h = 0; h < m.c.n_head; ++h) {
        const int kvh = h / group;
        const float* qh = q + h * hd;
        for (int j = 0; j < len; ++j) {
            const float* kj = kc + (size_t)j * kv_dim + kvh * hd;
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot += qh[d] * kj[d];
            scores[j] = dot * scale;
        }
        float mx = -INFINITY;
        for (int j = 0; j < len; ++j) mx = std::max(mx, scores[j]);
        float sum = 0.0f;
        for (int j = 0; j < len; ++j) { scores[j] = expf(scores[j] - mx); sum += scores[j]; }
        float* oh = out + h * hd;
        for (int d = 0; d < hd; ++d) oh[d] = 0.0f;
        for (int j = 0; j < len; ++j) {
            const float p = scores[j] / sum;
            const float* vj = vc + (size_t)j * kv_dim + kvh * hd;
            for (int d = 0; d < hd; ++d) oh[d] += p * vj[d];
        }
    }
}

// llm.rs:417-428 FeedForward::forward.
void ffn(const Model& m, const Layer& L, const float* x, int rows, float* out) {
    const int F = m.c.ff;
    std::vector<float> g((size_t)rows * F), u((size_t)rows * F);
    L.gate.forward(x, rows, g.data(), m.threads);
    L.up.forward(x, rows, u.data(), m.threads);
    for (size_t i = 0; i < g.size(); ++i) g[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
    L.down.forward(g.data(), rows, out, m.threads);
}

// llm.rs:345-358 Attention::forward_one + llm.rs:451-461 LlamaBlock::forward_one.
void block_one(const Model& m, const Layer& L, std::vector<float>& x, int pos, std::vector<float>& kc, std::vector<float>& vc) {
    const int d = m.c.d, qd = m.q_dim(), kvd = m.kv_dim();
    std::vector<float> normed(d), q(qd), k(kvd), v(kvd), ctx(qd), a(d), f(d);
    rmsnorm_row(x.data(), L.attn_norm.data(), m.c.eps, d, normed.data());
    project(m, L, normed.data(), pos, q.data(), k.data(), v.data());
    kc.insert(kc.end(), k.begin(), k.end());
    vc.insert(vc.end(), v.begin(), v.end());
    const int len = (int)(kc.size() / kvd);
    attend(m, q.data(), kc.data(), vc.data(), len, ctx.data());
    L.wo.forward(ctx.data(), 1, a.data(), 1);
    std::vector<float> h(d);
    for (int i = 0; i < d; ++i) h[i] = x[i] + a[i];
    rmsnorm_row(h.data(), L.ffn_norm.data(), m.c.eps, d, normed.data());
    ffn(m, L, normed.data(), 1, f.data());
    for (int i = 0; i < d; ++i) x[i] = h[i] + f[i];
}

// llm.rs:362-392 Attention::forward_full + llm.rs:464-482 LlamaBlock::forward_full.
void block_full(const Model& m, const Layer& L, std::vector<float>& x, int seq) {
    const int d = m.c.d, qd = m.q_dim(), kvd = m.kv_dim();
    std::vector<float> n1((size_t)seq * d), kc((size_t)seq * kvd), vc((size_t)seq * kvd), qa((size_t)seq * qd);
    for (int t = 0; t < seq; ++t) rmsnorm_row(x.data() + (size_t)t * d, L.attn_norm.data(), m.c.eps, d, n1.data() + (size_t)t * d);
    for (int t = 0; t < seq; ++t)
        project(m, L, n1.data() + (size_t)t * d, t, qa.data() + (size_t)t * qd, kc.data() + (size_t)t * kvd, vc.data() + (size_t)t * kvd);
    std::vector<float> ctx((size_t)seq * qd), a((size_t)seq * d);
    for (int t = 0; t < seq; ++t) attend(m, qa.data() + (size_t)t * qd, kc.data(), vc.data(), t + 1, ctx.data() + (size_t)t * qd);
    L.wo.forward(ctx.data(), seq, a.data(), m.threads);     // row by row in the reference; rows are independent
    std::vector<float> h((size_t)seq * d), n2((size_t)seq * d), f((size_t)seq * d);
    for (size_t i = 0; i < h.size(); ++i) h[i] = x[i] + a[i];
    for (int t = 0; t < seq; ++t) rmsnorm_row(h.data() + (size_t)t * d, L.ffn_norm.data(), m.c.eps, d, n2.data() + (size_t)t * d);
    ffn(m, L, n2.data(), seq, f.data());
    for (size_t i = 0; i < h.size(); ++i) x[i] = h[i] + f[i];
}

// llm.rs:588-597 embed.
int embed(const Model& m, int token, float* out) {
    if (token < 0 || token >= m.c.vocab) return -2;
    std::memcpy(out, m.tok.data() + (size_t)token * m.c.d, (size_t)m.c.d * 4);
    return 0;
}

// llm.rs:622-635 forward_tokens.
int forward_tokens(const Model& m, const int32_t* ids, int seq, float* logits) {
    const int d = m.c.d;
    std::vector<float> x((size_t)seq * d);
    for (int t = 0; t < seq; ++t)
        if (embed(m, ids[t], x.data() + (size_t)t * d)) return -2;
    for (const Layer& L : m.layers) block_full(m, L, x, seq);
    std::vector<float> normed((size_t)seq * d);
    for (int t = 0; t < seq; ++t) rmsnorm_row(x.data() + (size_t)t * d, m.out_norm.data(), m.c.eps, d, normed.data() + (size_t)t * d);
    m.head.forward(normed.data(), seq, logits, m.threads);
    return 0;
}

// llm.rs:610-618 forward_one (+ the context bound of llm.rs:720-730).
int forward_one(Cache& c, int token, float* logits) {
    const Model& m = *c.m;
    if (c.pos >= m.c.ctx) return -2;
    std::vector<float> x(m.c.d);
    if (embed(m, token, x.data())) return -2;
    for (size_t l = 0; l < m.layers.size(); ++l) block_one(m, m.layers[l], x, c.pos, c.k[l], c.v[l]);
    c.pos += 1;
    std::vector<float> normed(m.c.d);
    rmsnorm_row(x.data(), m.out_norm.data(), m.c.eps, m.c.d, normed.data());
    m.head.forward(normed.data(), 1, logits, m.threads);
    return 0;
}

// llm_score.rs:21-32 plan_windows.
struct Win { int start, first, end; };
std::vector<Win> plan_windows(int n, int window, int from) {
    const int half = std::max(window / 2, 1);
    std::vector<Win> out;
    int next = std::max(from, 1);
    while (next < n) {
        const int start = next <= window ? 0 : next - half;
        const int end = std::min(start + window + 1, n);
        out.push_back({start, next, end});
        next = end;
    }
    return out;
}

// llm_score.rs:35-39 log_prob.
double log_prob(const float* logits, int n, int target) {
    float mxf = -INFINITY;
    for (int i = 0; i < n; ++i) mxf = std::max(mxf, logits[i]);
    const double mx = (double)mxf;
    double sum = 0.0;
    for (int i = 0; i < n; ++i) sum += std::exp((double)logits[i] - mx);
    return (double)logits[target] - mx - std::log(sum);
}

}  // namespace

extern "C" {

void fo_rmsnorm(const float* x, const float* w, float eps, int rows, int d, float* out) {
    for (int r = 0; r < rows; ++r) rmsnorm_row(x + (size_t)r * d, w, eps, d, out + (size_t)r * d);
}
void fo_apply_rope(float* x, int n_heads, int hd, int rope_dim, int pos, float base, int neox, const float* ff, int n_ff, float linear) {
    apply_rope(x, n_heads, hd, rope_dim, pos, base, neox, ff, n_ff, linear);
}
void fo_silu_mul(const float* g, const float* u, int n, float* out) {
    for (int i = 0; i < n; ++i) out[i] = (g[i] / (1.0f + expf(-g[i]))) * u[i];
}
int fo_llama_plan_windows(int n, int window, int from, int32_t* out, int cap) {
    const std::vector<Win> p = plan_windows(n, window, from);
    for (size_t i = 0; i < p.size() && (int)i < cap; ++i) { out[3 * i] = p[i].start; out[3 * i + 1] = p[i].first; out[3 * i + 2] = p[i].end; }
    return (int)p.size();
}
double fo_llama_log_prob(const float* logits, int n, int target) { return log_prob(logits, n, target); }

// Returns null on the configurations Attention::new / RopeScaling::check refuse (llm.rs:243-252,135-150).
void* fo_llama_create(const void* cfg, const void* weights, int threads) {
    const Cfg& c = *(const Cfg*)cfg;
    const Weights& w = *(const Weights*)weights;
    if (c.n_kv <= 0 || c.n_head % c.n_kv) return nullptr;
    if (c.rope_dim > c.hd || c.rope_dim % 2) return nullptr;
    auto ok = [](float v) { return std::isfinite(v) && v > 0.0f; };
    if (!ok(c.linear)) return nullptr;
    if (w.rope_freqs)
        for (int i = 0; i < c.rope_dim / 2; ++i)
            if (!ok(w.rope_freqs[i])) return nullptr;
    Model* m = new Model();
    m->c = c;
    m->threads = threads < 1 ? 1 : threads;
    const int d = c.d, qd = c.n_head * c.hd, kvd = c.n_kv * c.hd;
    m->tok.resize((size_t)c.vocab * d);
    fo_q8_0_decode((const uint8_t*)w.token_embd, m->tok.size(), m->tok.data());
    m->layers.resize(c.n_layer);
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerW& h = w.layers[l];
        Layer& L = m->layers[l];
        L.attn_norm.assign(h.attn_norm, h.attn_norm + d);
        L.ffn_norm.assign(h.ffn_norm, h.ffn_norm + d);
        L.wq.load(h.wq, h.bq, qd, d);
        L.wk.load(h.wk, h.bk, kvd, d);
        L.wv.load(h.wv, h.bv, kvd, d);
        L.wo.load(h.wo, nullptr, d, qd);
        L.gate.load(h.gate, nullptr, c.ff, d);
        L.up.load(h.up, nullptr, c.ff, d);
        L.down.load(h.down, nullptr, d, c.ff);
    }
    m->out_norm.assign(w.output_norm, w.output_norm + d);
    if (w.rope_freqs) m->ff.assign(w.rope_freqs, w.rope_freqs + c.rope_dim / 2);
    // a tied head is the transpose of the embedding (llm.rs:580-585)
    m->head.load(c.tied || !w.output ? w.token_embd : w.output, nullptr, c.vocab, d);
    return m;
}
// Gguf::load_llama(kind) (gguf/llama.rs:164-171): every Linear of the model, the LM head included, packed to int8 (0)
// or int4 (1); the embedding table stays f32.
void fo_llama_pack(void* mp, int kind) {
    Model& m = *(Model*)mp;
    for (Layer& L : m.layers)
        for (Lin* l : {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down}) l->pack(kind);
    m.head.pack(kind);
}
// load_llama_prec(None) (gguf/llama.rs:171-176): a matrix replaced by f32 values [n_out][n_in] decoded from the file
// (stored as Ferrum's [n_in][n_out], gguf/llama.rs:143-144). which: 0..6 = wq, wk, wv, wo, gate, up, down of `layer`;
// 7 = the LM head; 8 = the embedding table [vocab][d] (kept as is).
int fo_llama_set_f32(void* mp, int layer, int which, const float* w, int n_out, int n_in) {
    Model& m = *(Model*)mp;
    if (which == 8) {
        if ((size_t)n_out * n_in != m.tok.size()) return -1;
        m.tok.assign(w, w + m.tok.size());
        return 0;
    }
    Lin* l = nullptr;
    if (which == 7) l = &m.head;
    else {
        if (layer < 0 || layer >= (int)m.layers.size() || which < 0 || which > 6) return -1;
        Layer& L = m.layers[layer];
        Lin* all[7] = {&L.wq, &L.wk, &L.wv, &L.wo, &L.gate, &L.up, &L.down};
        l = all[which];
    }
    if (l->out != n_out || l->in != n_in) return -1;
    for (int o = 0; o < n_out; ++o)
        for (int i = 0; i < n_in; ++i) l->w[(size_t)i * n_out + o] = w[(size_t)o * n_in + i];
    l->kind = -1;
    return 0;
}
void fo_llama_free(void* m) { delete (Model*)m; }

int fo_llama_forward_tokens(void* m, const int32_t* ids, int n, float* logits) { return forward_tokens(*(Model*)m, ids, n, logits); }

void* fo_llama_cache_create(void* m) {
    Cache* c = new Cache();
    c->m = (Model*)m;
    c->k.resize(c->m->layers.size());
    c->v.resize(c->m->layers.size());
    return c;
}
void fo_llama_cache_free(void* c) { delete (Cache*)c; }
void fo_llama_cache_clear(void* cp) {
    Cache& c = *(Cache*)cp;
    for (auto& k : c.k) k.clear();
    for (auto& v : c.v) v.clear();
    c.pos = 0;
}
int fo_llama_cache_pos(void* c) { return ((Cache*)c)->pos; }
int fo_llama_forward_one(void* c, int token, float* logits) { return forward_one(*(Cache*)c, token, logits); }

// llm_score.rs:76-96 score_from. lp / greedy_flags (may be null) are indexed by target - 1.
int fo_llama_score_from(void* mp, const int32_t* ids, int n, int from, int window, double* logprob, int* n_tokens, int* greedy,
                        double* lp, uint8_t* greedy_flags) {
    const Model& m = *(Model*)mp;
    if (window < 2 || window > m.c.ctx) return -2;
    double total = 0.0;
    int count = 0, all = 1;
    const int V = m.c.vocab;
    for (const Win& w : plan_windows(n, window, from)) {
        const int rows = std::min(w.start + window, n) - w.start;
        std::vector<float> logits((size_t)rows * V);
        const int rc = forward_tokens(m, ids + w.start, rows, logits.data());
        if (rc) return rc;
        for (int t = w.first; t < w.end; ++t) {
            const float* row = logits.data() + (size_t)(t - 1 - w.start) * V;
            const double v = log_prob(row, V, ids[t]);
            const int g = fo_argmax_first(row, V) == ids[t];
            total += v;
            count += 1;
            all &= g;
            if (lp) lp[t - 1] = v;
            if (greedy_flags) greedy_flags[t - 1] = (uint8_t)g;
        }
    }
    *logprob = total; *n_tokens = count; *greedy = all;
    return 0;
}

// llm.rs:706-754 generate_inner without the hooks. Returns the number of tokens, or < 0.
int fo_llama_generate(void* cp, const int32_t* prompt, int n, int max_new, float temperature, int top_k, float top_p,
                      float rep_penalty, const int32_t* stops, int n_stops, uint64_t* rng_state, int32_t* out) {
    Cache& c = *(Cache*)cp;
    const Model& m = *c.m;
    if (n <= 0) return -2;
    if (n >= m.c.ctx) return -2;
    max_new = std::min(max_new, m.c.ctx - n);
    fo_llama_cache_clear(cp);
    std::vector<float> logits(m.c.vocab);
    for (int i = 0; i < n; ++i)
        if (forward_one(c, prompt[i], logits.data())) return -2;
    std::vector<int32_t> recent(prompt, prompt + n);
    int made = 0;
    for (int i = 0; i < max_new; ++i) {
        const int next = fo_sample_with_params(logits.data(), m.c.vocab, temperature, top_k, top_p, rep_penalty, recent.data(),
                                               (int)recent.size(), rng_state);
        out[made++] = next;
        bool stop = false;
        for (int s = 0; s < n_stops; ++s) stop |= stops[s] == next;
        if (stop) break;
        recent.push_back(next);
        if (forward_one(c, next, logits.data())) return -2;
    }
    return made;
}

}  // extern "C"
