// ferrum_oracle — CPU restatement of Ferrum's f32 GPT-2 forward path.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA path is compared
// against (and the timed CPU baseline of the benchmark). Nothing in the shipped
// library links, loads or calls it.
//
// Parity status: the Rust reference cannot be compiled in this environment (no
// cargo/rustc), so the restatement is pinned at component level against the
// known-answer values held by the reference's own unit tests (Q8_0 codec, f16
// specials, GELU, Linear, matmul, LayerNorm, Embedding, argmax ties, window
// plan, bias-only log-probs) and at cross-path level (KV-cached == full forward,
// batched scorer == one-forward-per-target). Absolute logits of the GPT-2-small
// shaped configurations are "parity unpinned": no stored logits exist upstream.
//
// Every function names the reference file:line it restates. Arithmetic rules
// that make the restatement bit-faithful: f32 everywhere, products added in
// ascending k, bias added last, no FMA contraction (-ffp-contract=off), glibc
// expf/tanhf/logf/log, two-pass LayerNorm with a division by std.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// ---------------------------------------------------------------- f16 codec
// ferrum_core/src/gguf_write/blocks.rs:12-61 — IEEE RNE with overflow to Inf,
// gradual underflow, NaN canonicalised to sign|0x7E00.
uint16_t f32_to_f16(float value) {
    const uint32_t x = f2u(value);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return sign | (ax > 0x7F800000u ? 0x7E00u : 0x7C00u);
    const int exp32 = (int)(ax >> 23);
    if (exp32 >= 143) return sign | 0x7C00u;          // >= 2^16
    if (exp32 <= 112) {                               // f16 subnormal or zero
        if (exp32 < 102) return sign;                 // < 2^-25
        const uint32_t mant = (ax & 0x007FFFFFu) | 0x00800000u;
        const uint32_t shift = (uint32_t)(126 - exp32); // 14..24
        const uint32_t lsb = (mant >> shift) & 1u;
        const uint32_t half = (mant + ((1u << (shift - 1)) - 1u) + lsb) >> shift;
        return sign | (uint16_t)half;
    }
    const uint32_t lsb = (ax >> 13) & 1u;
    const uint32_t h = ((ax - 0x38000000u) + 0x0FFFu + lsb) >> 13;
    return sign | (uint16_t)(h >= 0x7C00u ? 0x7C00u : h);
}

// ferrum_core/src/gguf/dequant.rs:7-35.
float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t mant = h & 0x3FFu;
    if (exp == 0x1F) return u2f(sign | 0x7F800000u | (mant << 13));
    if (exp != 0) return u2f(sign | ((exp + 112u) << 23) | (mant << 13));
    if (mant == 0) return u2f(sign);
    int e = 113;                                      // 2^-14 biased for f32, +0
    while (!(mant & 0x400u)) { mant <<= 1; --e; }
    return u2f(sign | ((uint32_t)e << 23) | ((mant & 0x3FFu) << 13));
}

// ---------------------------------------------------------------- Q8_0 codec
// ferrum_core/src/quant.rs:271-280 — d = amax/127, id = 1/d (0 when d == 0),
// q = round-half-away(x*id) with Rust's saturating float->i8 cast.
void q8_0_block(const float* x, uint16_t* d16, int8_t* q) {
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) {
        const float a = std::fabs(x[i]);
        if (a > amax) amax = a;                       // f32::max ignores NaN
    }
    const float d = amax / 127.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 32; ++i) {
        const float r = std::round(x[i] * id);
        int v;
        if (r != r) v = 0; else if (r >= 127.0f) v = 127; else if (r <= -128.0f) v = -128; else v = (int)r;
        q[i] = (int8_t)v;
    }
    *d16 = f32_to_f16(d);
}

// ---------------------------------------------------------------- RNG
// ferrum_core/src/rng.rs:9-48 — xorshift64*, 24-bit uniform, Box–Muller.
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed == 0 ? 0x9E3779B97F4A7C15ull : seed) {}
    uint64_t next_u64() {
        uint64_t x = s;
        x ^= x << 13; x ^= x >> 7; x ^= x << 17;
        s = x;
        return x * 0x2545F4914F6CDD1Dull;
    }
    float next_f32() { return (float)(next_u64() >> 40) / 16777216.0f; }
    float next_normal() {
        float u1 = next_f32();
        if (!(u1 > 1e-7f)) u1 = 1e-7f;
        const float u2 = next_f32();
        return std::sqrt(-2.0f * std::log(u1)) * std::cos(6.28318530717958647692f * u2);
    }
};

// ---------------------------------------------------------------- matmul engine
// ferrum_core/src/ops.rs:9-177. KC = NC = 256 cache panels, 4x8 register tile,
// edge loops in i-p-j order. For a fixed (i, j) every variant adds the products
// in ascending p onto the same running value, so all of them equal the plain
// triple loop bit for bit.
constexpr int KC = 256, NC = 256, MR = 4, NR = 8;

__attribute__((target_clones("avx2", "default")))
void micro_tile(const float* a, const float* b, int k, int n, int i, int r0, int j, int pp, int p1, float* out) {
    float acc[MR][NR];
    for (int r = 0; r < MR; ++r)
        for (int c = 0; c < NR; ++c) acc[r][c] = out[(size_t)(i + r - r0) * n + j + c];
    for (int p = pp; p < p1; ++p) {
        const float* bs = b + (size_t)p * n + j;
        for (int r = 0; r < MR; ++r) {
            const float av = a[(size_t)(i + r) * k + p];
            for (int c = 0; c < NR; ++c) acc[r][c] += av * bs[c];
        }
    }
    for (int r = 0; r < MR; ++r)
        for (int c = 0; c < NR; ++c) out[(size_t)(i + r - r0) * n + j + c] = acc[r][c];
}

__attribute__((target_clones("avx2", "default")))
void edge_rows(const float* a, const float* b, int k, int n, int ia, int ib, int r0, int ja, int jb, int pp, int p1, float* out) {
    for (int i = ia; i < ib; ++i) {
        float* o = out + (size_t)(i - r0) * n;
        for (int p = pp; p < p1; ++p) {
            const float av = a[(size_t)i * k + p];
            const float* bs = b + (size_t)p * n;
            for (int j = ja; j < jb; ++j) o[j] += av * bs[j];
        }
    }
}

// ops.rs:29-55
void matmul_block(const float* a, const float* b, int k, int n, int r0, int r1, float* out) {
    for (int jj = 0; jj < n; jj += NC) {
        const int j1 = std::min(jj + NC, n);
        for (int pp = 0; pp < k; pp += KC) {
            const int p1 = std::min(pp + KC, k);
            int i = r0;
            for (; i + MR <= r1; i += MR) {
                int j = jj;
                for (; j + NR <= j1; j += NR) micro_tile(a, b, k, n, i, r0, j, pp, p1, out);
                if (j < j1) edge_rows(a, b, k, n, i, i + MR, r0, j, j1, pp, p1, out);
            }
            if (i < r1) edge_rows(a, b, k, n, i, r1, r0, jj, j1, pp, p1, out);
        }
    }
}

// ops.rs:132-148 — contraction first, bias as the epilogue.
void matmul_bias_block(const float* a, const float* b, const float* bias, int k, int n, int r0, int r1, float* block) {
    matmul_block(a, b, k, n, r0, r1, block);
    if (bias && n > 0)
        for (int r = 0; r < r1 - r0; ++r)
            for (int j = 0; j < n; ++j) block[(size_t)r * n + j] += bias[j];
}

// parallel.rs:84-92 — rows >= 2, cost >= 2^16, more than one worker.
bool should_parallelize(size_t rows, size_t cost, int threads) {
    return rows >= 2 && cost >= (1u << 16) && threads > 1;
}

// Static split of [0, rows) into ceil(rows/threads)-sized runs on scoped threads
// (parallel.rs:168-219, 252-297). `fn(r0, r1)`.
template <class F>
void run_rows(int rows, int threads, F fn) {
    const int per = (rows + threads - 1) / threads;
    std::vector<std::thread> ts;
    for (int r0 = per; r0 < rows; r0 += per) {
        const int r1 = std::min(rows, r0 + per);
        ts.emplace_back([=] { fn(r0, r1); });
    }
    fn(0, std::min(per, rows));
    for (auto& t : ts) t.join();
}

// ops.rs:159-177 + 233-256: y = x·W + b, W [k][n].
void linear(const float* a, const float* w, const float* bias, int m, int k, int n, float* out, int threads) {
    std::fill(out, out + (size_t)m * n, 0.0f);
    const size_t cost = (size_t)m * k * n;
    if (!should_parallelize((size_t)m, cost, threads)) {
        matmul_bias_block(a, w, bias, k, n, 0, m, out);
    } else {
        run_rows(m, threads, [=](int r0, int r1) {
            matmul_bias_block(a, w, bias, k, n, r0, r1, out + (size_t)r0 * n);
        });
    }
}

// Plain triple loop the reference's tests compare the engine with (ops.rs:538-564).
void linear_naive(const float* a, const float* w, const float* bias, int m, int k, int n, float* out) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            float s = 0.0f;
            for (int p = 0; p < k; ++p) s += a[(size_t)i * k + p] * w[(size_t)p * n + j];
            out[(size_t)i * n + j] = bias ? s + bias[j] : s;
        }
}

// ---------------------------------------------------------------- row kernels
// layer/norm.rs:46-82.
void layernorm(const float* x, const float* g, const float* b, int rows, int d, float* out) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * d;
        float sum = 0.0f;
        for (int c = 0; c < d; ++c) sum += xr[c];
        const float mean = sum / (float)d;
        float vs = 0.0f;
        for (int c = 0; c < d; ++c) { const float t = xr[c] - mean; vs += t * t; }
        const float var = vs / (float)d;
        const float sd = std::sqrt(var + 1e-5f);
        for (int c = 0; c < d; ++c) out[(size_t)r * d + c] = ((xr[c] - mean) / sd) * g[c] + b[c];
    }
}

// activation.rs:9-12.
inline float gelu(float x) {
    const float K = 0.7978846f;
    return 0.5f * x * (1.0f + std::tanh(K * (x + 0.044715f * x * x * x)));
}

// ops.rs:478-502.
void softmax_rows(const float* x, int rows, int cols, float* out) {
    for (int r = 0; r < rows; ++r) {
        const float* xr = x + (size_t)r * cols;
        float* o = out + (size_t)r * cols;
        float mx = -INFINITY;
        for (int c = 0; c < cols; ++c) mx = std::fmax(mx, xr[c]);
        float sum = 0.0f;
        for (int c = 0; c < cols; ++c) { const float e = std::exp(xr[c] - mx); o[c] = e; sum += e; }
        for (int c = 0; c < cols; ++c) o[c] /= sum;
    }
}

// slm/sampling.rs:96-104 — first index on ties, total order on floats.
int argmax_first(const float* xs, int n) {
    auto key = [](float f) { int32_t b = (int32_t)f2u(f); return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1); };
    int best = 0;
    for (int i = 0; i < n; ++i)
        if (key(xs[i]) > key(xs[best])) best = i;
    return best;
}

// slm/sampling.rs:106-121 pick_by_mass: the first index whose running mass reaches r; entries
// that top-k / top-p zeroed are never picked; falls back to the last index with any mass.
int pick_by_mass(const float* probs, int n, float r) {
    float cumsum = 0.0f;
    int last = 0;
    for (int i = 0; i < n; ++i) {
        if (probs[i] > 0.0f) {
            last = i;
            cumsum += probs[i];
            if (r <= cumsum) return i;
        }
    }
    return last;
}

// rng.rs:37-40 next_f32: 24 random bits / 2^24.
float rng_next_f32(Rng& r) { return (float)(r.next_u64() >> 40) / (float)(1ull << 24); }

// slm/sampling.rs:124-210 sample_with_params: repetition penalty on the logits of `recent`
// (once per occurrence, CTRL scheme) -> temperature <= 0: argmax_first, no draw -> temperature
// softmax (t = max(temperature, 0.01)) -> top-k -> top-p -> renormalise -> pick_by_mass with one
// next_f32 draw. Sums run in index order like the Rust iterators; the sorts put equal
// probabilities in an unspecified order (sort_unstable_by), here std::sort's.
int sample_with_params(const float* logits, int n, float temperature, int top_k, float top_p, float rep_penalty,
                       const int32_t* recent, int n_recent, Rng& rng) {
    std::vector<float> work(logits, logits + n);
    if (std::fabs(rep_penalty - 1.0f) > 1.1920929e-7f && rep_penalty > 0.0f) {
        for (int i = 0; i < n_recent; ++i) {
            const int tok = recent[i];
            if (tok >= 0 && tok < n) work[tok] = work[tok] > 0.0f ? work[tok] / rep_penalty : work[tok] * rep_penalty;
        }
    }
    if (temperature <= 0.0f) return argmax_first(work.data(), n);
    const float t = std::fmax(temperature, 0.01f);
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) mx = std::fmax(mx, work[i]);
    std::vector<float> probs(n);
    for (int i = 0; i < n; ++i) probs[i] = std::exp((work[i] - mx) / t);
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += probs[i];
    if (sum != sum || sum <= 1e-10f) return (int)(rng.next_u64() % (uint64_t)n);
    for (int i = 0; i < n; ++i) probs[i] /= sum;
    if (top_k > 0 && top_k < n) {
        std::vector<float> sorted(probs);
        std::sort(sorted.begin(), sorted.end(), [](float a, float b) { return a > b; });
        const float threshold = sorted[top_k - 1];
        for (int i = 0; i < n; ++i)
            if (probs[i] < threshold) probs[i] = 0.0f;
    }
    if (top_p < 1.0f) {
        std::vector<int> order(n);
        for (int i = 0; i < n; ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](int a, int b) { return probs[a] > probs[b]; });
        float cum = 0.0f;
        std::vector<char> keep(n, 0);
        for (int i : order) {
            keep[i] = 1;
            cum += probs[i];
            if (cum >= top_p) break;
        }
        for (int i = 0; i < n; ++i)
            if (!keep[i]) probs[i] = 0.0f;
    }
    float sum2 = 0.0f;
    for (int i = 0; i < n; ++i) sum2 += probs[i];
    for (int i = 0; i < n; ++i) probs[i] /= sum2;
    return pick_by_mass(probs.data(), n, rng_next_f32(rng));
}

// ---------------------------------------------------------------- model
struct Cfg { int32_t n_layer, d_model, n_head, d_ff, ctx, vocab, tied, math_mode; };
struct LayerW {
    const void* attn_qkv; const float* attn_qkv_b;
    const void* attn_out; const float* attn_out_b;
    const float *ln1_g, *ln1_b, *ln2_g, *ln2_b;
    const void* ffn_up; const float* ffn_up_b;
    const void* ffn_down; const float* ffn_down_b;
};
struct Weights {
    const void* token_embd; const float* position_embd; const LayerW* layers;
    const float *out_norm_g, *out_norm_b; const void* output;
};

// gguf/dequant.rs:37-49 on `rows` GGML rows of length k, then the transpose to
// Ferrum's [in][out] that loader/gpt2.rs:238-249 and `r.linear` perform.
std::vector<float> dequant_rows(const void* q8, size_t rows, size_t k) {
    std::vector<float> out(rows * k);
    const uint8_t* p = (const uint8_t*)q8;
    for (size_t b = 0; b < rows * k / 32; ++b, p += 34) {
        const float d = f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
        for (int j = 0; j < 32; ++j) out[b * 32 + j] = d * (float)(int8_t)p[2 + j];
    }
    return out;
}
std::vector<float> transpose(const float* w, size_t rows, size_t cols) {
    std::vector<float> t(rows * cols);
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) t[c * rows + r] = w[r * cols + c];
    return t;
}
std::vector<float> vec(const float* p, size_t n) { return std::vector<float>(p, p + n); }

struct Layer {
    std::vector<float> wq, wk, wv, wo, wup, wdown;  // [in][out]
    std::vector<float> bq, bk, bv, bo, bup, bdown, ln1g, ln1b, ln2g, ln2b;
};
struct Model {
    Cfg c; int threads;
    std::vector<float> tok, pos, head, lnfg, lnfb, zero_bias;
    std::vector<Layer> layers;
};
// layer/transformer.rs:15-56 — one [len][d] K and V buffer per block.
struct Stream {
    Model* m; int pos;
    std::vector<std::vector<float>> k, v;
};

Model* model_create(const Cfg* c, const Weights* w, int threads) {
    const size_t d = c->d_model, F = c->d_ff, V = c->vocab, T = c->ctx;
    if (d % 32 || F % 32 || d % c->n_head) return nullptr;
    Model* m = new Model;
    m->c = *c; m->threads = threads < 1 ? 1 : threads;
    m->tok = dequant_rows(w->token_embd, V, d);
    m->pos = vec(w->position_embd, T * d);
    // loader/gpt2.rs:228-233,269-274 — tied head reuses the token embedding.
    m->head = w->output ? transpose(dequant_rows(w->output, V, d).data(), V, d) : transpose(m->tok.data(), V, d);
    m->lnfg = vec(w->out_norm_g, d); m->lnfb = vec(w->out_norm_b, d);
    m->zero_bias.assign(V, 0.0f);
    m->layers.resize(c->n_layer);
    for (int l = 0; l < c->n_layer; ++l) {
        const LayerW& s = w->layers[l]; Layer& L = m->layers[l];
        std::vector<float> qkv = dequant_rows(s.attn_qkv, 3 * d, d);
        L.wq = transpose(qkv.data(), d, d);
        L.wk = transpose(qkv.data() + d * d, d, d);
        L.wv = transpose(qkv.data() + 2 * d * d, d, d);
        L.bq = vec(s.attn_qkv_b, d); L.bk = vec(s.attn_qkv_b + d, d); L.bv = vec(s.attn_qkv_b + 2 * d, d);
        L.wo = transpose(dequant_rows(s.attn_out, d, d).data(), d, d); L.bo = vec(s.attn_out_b, d);
        L.wup = transpose(dequant_rows(s.ffn_up, F, d).data(), F, d); L.bup = vec(s.ffn_up_b, F);
        L.wdown = transpose(dequant_rows(s.ffn_down, d, F).data(), d, F); L.bdown = vec(s.ffn_down_b, d);
        L.ln1g = vec(s.ln1_g, d); L.ln1b = vec(s.ln1_b, d); L.ln2g = vec(s.ln2_g, d); L.ln2b = vec(s.ln2_b, d);
    }
    return m;
}

// layer/transformer.rs:314-534 — pre-LN causal attention + GELU MLP on R = B·T rows.
// Entries with j > i are set to -1e9 before the softmax; their exp is exactly 0,
// so they add 0 to the row sum and 0·v to the output. Skipping them leaves every
// stored value unchanged.
void block_forward(const Model& M, const Layer& L, std::vector<float>& x, int B, int T) {
    const int d = M.c.d_model, H = M.c.n_head, hd = d / H, F = M.c.d_ff, R = B * T, th = M.threads;
    std::vector<float> n1((size_t)R * d), q((size_t)R * d), k((size_t)R * d), v((size_t)R * d), att((size_t)R * d, 0.0f);
    layernorm(x.data(), L.ln1g.data(), L.ln1b.data(), R, d, n1.data());
    linear(n1.data(), L.wq.data(), L.bq.data(), R, d, d, q.data(), th);
    linear(n1.data(), L.wk.data(), L.bk.data(), R, d, d, k.data(), th);
    linear(n1.data(), L.wv.data(), L.bv.data(), R, d, d, v.data(), th);
    const float scale = 1.0f / std::sqrt((float)hd);
    auto head_job = [&](int u0, int u1) {
        std::vector<float> s(T);
        for (int u = u0; u < u1; ++u) {
            const int b = u / H, h = u % H;
            for (int i = 0; i < T; ++i) {
                const float* qi = &q[((size_t)(b * T + i)) * d + h * hd];
                // layer/matmul.rs:5-26 — dot in ascending p, then the scale.
                for (int j = 0; j <= i; ++j) {
                    const float* kj = &k[((size_t)(b * T + j)) * d + h * hd];
                    float dot = 0.0f;
                    for (int p = 0; p < hd; ++p) dot += qi[p] * kj[p];
                    s[j] = dot * scale;
                }
                float mx = -INFINITY;
                for (int j = 0; j <= i; ++j) mx = std::fmax(mx, s[j]);
                if (i + 1 < T) mx = std::fmax(mx, -1e9f);
                float sum = 0.0f;
                for (int j = 0; j <= i; ++j) { const float e = std::exp(s[j] - mx); s[j] = e; sum += e; }
                for (int j = 0; j <= i; ++j) s[j] /= sum;
                // layer/matmul.rs:52-63 — O = S·V in i-p-j order.
                float* o = &att[((size_t)(b * T + i)) * d + h * hd];
                for (int p = 0; p <= i; ++p) {
                    const float sp = s[p];
                    const float* vp = &v[((size_t)(b * T + p)) * d + h * hd];
                    for (int j = 0; j < hd; ++j) o[j] += sp * vp[j];
                }
            }
        }
    };
    if (th > 1 && B * H >= 2) run_rows(B * H, th, head_job); else head_job(0, B * H);
    std::vector<float> proj((size_t)R * d);
    linear(att.data(), L.wo.data(), L.bo.data(), R, d, d, proj.data(), th);
    for (size_t i = 0; i < (size_t)R * d; ++i) x[i] = x[i] + proj[i];
    layernorm(x.data(), L.ln2g.data(), L.ln2b.data(), R, d, n1.data());
    std::vector<float> hid((size_t)R * F);
    linear(n1.data(), L.wup.data(), L.bup.data(), R, d, F, hid.data(), th);
    for (auto& t : hid) t = gelu(t);
    linear(hid.data(), L.wdown.data(), L.bdown.data(), R, F, d, proj.data(), th);
    for (size_t i = 0; i < (size_t)R * d; ++i) x[i] = x[i] + proj[i];
}

// model.rs:51-71 over the layer list of loader/gpt2.rs:235-275:
// Embedding, Block×L, LayerNorm, Linear head, Softmax. Returns 0 or -1 (bad id).
int forward(const Model& M, const int32_t* ids, int B, int T, float* probs) {
    const int d = M.c.d_model, V = M.c.vocab, R = B * T;
    if (T > M.c.ctx) return -1;
    std::vector<float> x((size_t)R * d);
    // layer/embedding.rs:98-152.
    for (int r = 0; r < R; ++r) {
        const int id = ids[r], t = r % T;
        if (id < 0 || id >= V) return -1;
        for (int c = 0; c < d; ++c) x[(size_t)r * d + c] = M.tok[(size_t)id * d + c] + M.pos[(size_t)t * d + c];
    }
    for (const Layer& L : M.layers) block_forward(M, L, x, B, T);
    std::vector<float> n((size_t)R * d);
    layernorm(x.data(), M.lnfg.data(), M.lnfb.data(), R, d, n.data());
    std::vector<float> logits((size_t)R * V);
    linear(n.data(), M.head.data(), M.zero_bias.data(), R, d, V, logits.data(), M.threads);
    softmax_rows(logits.data(), R, V, probs);
    return 0;
}

// slm/cached.rs:100-125 + layer/transformer.rs:221-294: one token through the
// KV-cached path; probs[V] out. Returns -1 on a bad id or a full cache.
int feed(Stream& S, int token, float* probs) {
    const Model& M = *S.m;
    const int d = M.c.d_model, H = M.c.n_head, hd = d / H, F = M.c.d_ff, V = M.c.vocab;
    if (token < 0 || token >= V || S.pos >= M.c.ctx) return -1;
    std::vector<float> x(d), n1(d), q(d), kk(d), vv(d), att(d), proj(d), xa(d), hid(F);
    for (int c = 0; c < d; ++c) x[c] = M.tok[(size_t)token * d + c] + M.pos[(size_t)S.pos * d + c];
    const float scale = 1.0f / std::sqrt((float)hd);
    for (size_t l = 0; l < M.layers.size(); ++l) {
        const Layer& L = M.layers[l];
        layernorm(x.data(), L.ln1g.data(), L.ln1b.data(), 1, d, n1.data());
        linear(n1.data(), L.wq.data(), L.bq.data(), 1, d, d, q.data(), 1);
        linear(n1.data(), L.wk.data(), L.bk.data(), 1, d, d, kk.data(), 1);
        linear(n1.data(), L.wv.data(), L.bv.data(), 1, d, d, vv.data(), 1);
        S.k[l].insert(S.k[l].end(), kk.begin(), kk.end());
        S.v[l].insert(S.v[l].end(), vv.begin(), vv.end());
        const int len = S.pos + 1;
        std::fill(att.begin(), att.end(), 0.0f);
        std::vector<float> sc(len);
        for (int h = 0; h < H; ++h) {
            const int hs = h * hd;
            for (int j = 0; j < len; ++j) {
                float dot = 0.0f;
                for (int p = 0; p < hd; ++p) dot += q[hs + p] * S.k[l][(size_t)j * d + hs + p];
                sc[j] = dot * scale;
            }
            float mx = -INFINITY;
            for (int j = 0; j < len; ++j) mx = std::fmax(mx, sc[j]);
            float sum = 0.0f;
            for (int j = 0; j < len; ++j) { sc[j] = std::exp(sc[j] - mx); sum += sc[j]; }
            for (int j = 0; j < len; ++j) {
                const float p = sc[j] / sum;
                for (int c = 0; c < hd; ++c) att[hs + c] += p * S.v[l][(size_t)j * d + hs + c];
            }
        }
        linear(att.data(), L.wo.data(), L.bo.data(), 1, d, d, proj.data(), 1);
        for (int c = 0; c < d; ++c) xa[c] = x[c] + proj[c];
        layernorm(xa.data(), L.ln2g.data(), L.ln2b.data(), 1, d, n1.data());
        linear(n1.data(), L.wup.data(), L.bup.data(), 1, d, F, hid.data(), 1);
        for (auto& t : hid) t = gelu(t);
        linear(hid.data(), L.wdown.data(), L.bdown.data(), 1, F, d, proj.data(), 1);
        for (int c = 0; c < d; ++c) x[c] = xa[c] + proj[c];
    }
    layernorm(x.data(), M.lnfg.data(), M.lnfb.data(), 1, d, n1.data());
    std::vector<float> logits(V);
    linear(n1.data(), M.head.data(), M.zero_bias.data(), 1, d, V, logits.data(), 1);
    softmax_rows(logits.data(), 1, V, probs);
    S.pos += 1;
    return 0;
}

void stream_reset(Stream& S) {
    for (auto& a : S.k) a.clear();
    for (auto& a : S.v) a.clear();
    S.pos = 0;
}

}  // namespace

extern "C" {

uint16_t fo_f32_to_f16(float v) { return f32_to_f16(v); }
float fo_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// gguf_write/blocks.rs:132-140 — 34-byte blocks [u16 d LE][i8 × 32]; n % 32 == 0.
void fo_q8_0_encode(const float* x, size_t n, uint8_t* out) {
    for (size_t b = 0; b < n / 32; ++b) {
        uint16_t d16; int8_t q[32];
        q8_0_block(x + b * 32, &d16, q);
        out[b * 34] = (uint8_t)(d16 & 0xFF); out[b * 34 + 1] = (uint8_t)(d16 >> 8);
        std::memcpy(out + b * 34 + 2, q, 32);
    }
}
void fo_q8_0_decode(const uint8_t* raw, size_t n, float* out) {
    std::vector<float> v = dequant_rows(raw, 1, n);
    std::memcpy(out, v.data(), n * 4);
}

uint64_t fo_rng_seed(uint64_t seed) { return Rng(seed).s; }
uint64_t fo_rng_next_u64(uint64_t* state) { Rng r(1); r.s = *state; uint64_t v = r.next_u64(); *state = r.s; return v; }
// train_transformer/param.rs:24-28 — next_normal() * scale per element.
void fo_rng_fill_normal(uint64_t* state, float scale, size_t n, float* out) {
    Rng r(1); r.s = *state;
    for (size_t i = 0; i < n; ++i) out[i] = r.next_normal() * scale;
    *state = r.s;
}
void fo_rng_fill_ids(uint64_t* state, int32_t vocab, size_t n, int32_t* out) {
    Rng r(1); r.s = *state;
    for (size_t i = 0; i < n; ++i) out[i] = (int32_t)(r.next_u64() % (uint64_t)vocab);
    *state = r.s;
}

void fo_linear(const float* x, const float* w_kn, const float* bias, int m, int k, int n, float* y, int threads) {
    linear(x, w_kn, bias, m, k, n, y, threads);
}
void fo_linear_naive(const float* x, const float* w_kn, const float* bias, int m, int k, int n, float* y) {
    linear_naive(x, w_kn, bias, m, k, n, y);
}
// Q8_0 rows [n][k/32·34 B] expanded and transposed to [k][n] as the loader does.
void fo_q8_0_expand_kn(const void* wq, int n, int k, float* w_kn) {
    std::vector<float> t = transpose(dequant_rows(wq, n, k).data(), n, k);
    std::memcpy(w_kn, t.data(), t.size() * 4);
}
void fo_layernorm(const float* x, const float* g, const float* b, int rows, int d, float* out) { layernorm(x, g, b, rows, d, out); }
float fo_gelu(float x) { return gelu(x); }
void fo_softmax_rows(const float* x, int rows, int cols, float* out) { softmax_rows(x, rows, cols, out); }
int fo_argmax_first(const float* x, int n) { return argmax_first(x, n); }
int fo_pick_by_mass(const float* probs, int n, float r) { return pick_by_mass(probs, n, r); }
float fo_rng_next_f32(uint64_t* state) { Rng r(1); r.s = *state; const float v = rng_next_f32(r); *state = r.s; return v; }
int fo_sample_with_params(const float* logits, int n, float temperature, int top_k, float top_p, float rep_penalty,
                          const int32_t* recent, int n_recent, uint64_t* rng_state) {
    Rng r(1);
    r.s = *rng_state;
    const int tok = sample_with_params(logits, n, temperature, top_k, top_p, rep_penalty, recent, n_recent, r);
    *rng_state = r.s;
    return tok;
}

void* fo_model_create(const void* cfg, const void* weights, int threads) {
    return model_create((const Cfg*)cfg, (const Weights*)weights, threads);
}
void fo_model_free(void* m) { delete (Model*)m; }
void fo_model_set_threads(void* m, int threads) { ((Model*)m)->threads = threads < 1 ? 1 : threads; }

int fo_forward(void* m, const int32_t* ids, int B, int T, float* probs) { return forward(*(Model*)m, ids, B, T, probs); }

void* fo_stream_create(void* m) {
    Stream* s = new Stream; s->m = (Model*)m; s->pos = 0;
    s->k.resize(s->m->layers.size()); s->v.resize(s->m->layers.size());
    return s;
}
void fo_stream_free(void* s) { delete (Stream*)s; }
void fo_stream_reset(void* s) { stream_reset(*(Stream*)s); }
int fo_cached_len(void* s) { return ((Stream*)s)->pos; }
int fo_feed(void* s, int token, float* probs) { return feed(*(Stream*)s, token, probs); }
// slm/cached.rs:129-136.
int fo_prime(void* s, const int32_t* ids, int n, float* probs) {
    Stream& S = *(Stream*)s;
    stream_reset(S);
    for (int i = 0; i < n; ++i)
        if (feed(S, ids[i], probs)) return -1;
    return 0;
}

// slm/token_stream.rs:66-189 with temperature <= 0 (slm/sampling.rs:147):
// keep the last `cap` prompt ids, prime, then per step take
// argmax_first(ln(max(p, 1e-12))), stop on eos, push, and either re-prime on the
// last cap/2 ids (window longer than cap) or feed the token. `margin[i]` is the
// gap between the two largest log-values at step i. Returns tokens produced.
int fo_generate_greedy(void* s, const int32_t* prompt, int n, int max_new, int eos, int32_t* out, float* margin) {
    Stream& S = *(Stream*)s;
    const int V = S.m->c.vocab, cap = std::max(1, (int)S.m->c.ctx), keep = std::max(1, cap / 2);
    std::vector<int32_t> window(prompt, prompt + n);
    if ((int)window.size() > cap) window.erase(window.begin(), window.end() - cap);
    std::vector<float> dist(V), lg(V);
    if (fo_prime(s, window.data(), (int)window.size(), dist.data())) return -1;
    int made = 0;
    while (made < max_new) {
        for (int i = 0; i < V; ++i) lg[i] = std::log(std::fmax(dist[i], 1e-12f));
        const int next = argmax_first(lg.data(), V);
        if (margin) {
            float second = -INFINITY;
            for (int i = 0; i < V; ++i) if (i != next && lg[i] > second) second = lg[i];
            margin[made] = lg[next] - second;
        }
        if (next == eos) break;
        out[made++] = next;
        window.push_back(next);
        int rc;
        if ((int)window.size() > cap) {
            window.erase(window.begin(), window.end() - keep);
            rc = fo_prime(s, window.data(), (int)window.size(), dist.data());
        } else {
            rc = feed(S, next, dist.data());
        }
        if (rc) return -1;
    }
    return made;
}

// slm/scoring.rs:151-213. Window plan: first window at 0; a later one starts
// ctx/2 before its first new target; each target scored once. One forward per
// window here (the reference batches up to 32 windows; rows are independent).
// lp[i] / is_greedy[i] (optional, length n) are filled for targets i >= from.
int fo_token_logprobs(void* mp, const int32_t* ids, int n, int from, double* logprob, int* n_tokens, int* greedy,
                      float* lp, uint8_t* is_greedy) {
    Model& M = *(Model*)mp;
    const int T = M.c.ctx, V = M.c.vocab, half = std::max(1, T / 2);
    from = std::max(from, 1);
    *logprob = 0.0; *n_tokens = 0; *greedy = 1;
    if (from >= n) return 0;
    std::vector<float> probs((size_t)T * V);
    std::vector<int32_t> win(T);
    int next = from;
    while (next < n) {
        const int start = next <= T ? 0 : next - half;
        const int end = std::min(start + T + 1, n);
        const int wl = std::min(start + T, n) - start;
        for (int i = 0; i < T; ++i) win[i] = i < wl ? ids[start + i] : 0;
        if (forward(M, win.data(), 1, T, probs.data())) return -1;
        for (int target = next; target < end; ++target) {
            const float* row = &probs[(size_t)(target - 1 - start) * V];
            const int id = ids[target];
            float p = row[id];
            if (p == p) p = std::fmax(p, 1e-12f);      // loss.rs:12-18
            const double l = std::log((double)p);
            const int g = argmax_first(row, V) == id;
            *logprob += l; *n_tokens += 1; *greedy &= g;
            if (lp) lp[target] = (float)l;
            if (is_greedy) is_greedy[target] = (uint8_t)g;
        }
        next = end;
    }
    return 0;
}

}  // extern "C"
