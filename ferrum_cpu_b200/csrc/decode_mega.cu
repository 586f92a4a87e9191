// Persistent decode kernel: whole KV-cached tokens in ONE cooperative launch.
//
// Replaces the per-token call chain CachedTransformer::feed (ferrum_core/src/slm/cached.rs:
// 100-125) -> TransformerBlock::forward_with_cache (layer/transformer.rs:221-294) ->
// Linear::forward (layer/linear.rs:177-210) and the greedy pick of token_stream.rs:134 +
// sampling.rs:96-104, for n_steps consecutive tokens.
//
// Shape of the kernel (one CTA per SM, all co-resident):
//   * a producer warp streams this CTA's share of every Q8_0 matrix, in the fixed order the
//     token needs them, through a ring of shared-memory slots with 1-D bulk async copies
//     (cp.async.bulk + mbarrier complete_tx), and the block's LayerNorm vectors and bias
//     slices through a second, two-deep ring. Weights do not depend on activations, so the
//     producer runs ahead across the grid barriers and HBM never waits for the math;
//   * 16 consumer warps do the fp32 dot products out of shared memory (f16 scale applied per
//     16 quants in registers, half-warp shuffles), LayerNorm, attention over the f32 KV cache
//     (split over CTAs, combined flash-decoding style), and the softmax / greedy pick;
//   * the LM head, the one phase with enough rows per CTA to be bound by instruction issue,
//     runs on the integer tensor cores instead: the final LayerNorm output is held as block
//     fixed point (per 32 elements a power-of-two scale and four planes of signed base-128
//     digits, 28 bits per element), one mma.sync m16n8k32 (s8 x s8 -> s32) multiplies the four
//     digit rows by the 8 x 32 quants of a tile exactly, and the s32 sums are scaled by (f16
//     block scale x activation block scale) and accumulated in fp32 per Q8_0 block;
//   * phases are separated by a software grid barrier (5 per block, 2 per head step); what
//     crosses a barrier goes through small global buffers read with L1-bypassing loads.
// Every wait (mbarrier, grid barrier) is bounded by a cycle budget; when it runs out the
// kernel records FC_E_TIMEOUT, drains its own copies in flight and returns.
//
// Bound: HBM. Algorithmic bytes per token: every Q8_0 matrix once (34/32 B per weight) + the
// f32 KV rows of positions 0..pos + small f32 vectors.
#include "fc_common.cuh"
#include "mega.cuh"

namespace fc {

namespace {

constexpr int CONSUMERS = 512;                 // 16 consumer warps
constexpr int CWARPS = CONSUMERS / 32;
constexpr int THREADS = CONSUMERS + 32;        // + 1 producer warp
constexpr int SLOTS = 5;
constexpr int SLOT_Q = 24576;                  // quant bytes per slot
constexpr int SLOT_D = SLOT_Q / 16;            // scale bytes per slot (2 B per 32 quants)
constexpr int SLOT_BYTES = SLOT_Q + SLOT_D;
constexpr int MAX_D = 1024, MAX_F = 4096, MAX_CTX = 1024;
// The CTA's slice of the logits lives in the activation buffer behind the (d-wide) input of the
// head. Total shared memory stays below 196 KB: the next carve-out step would halve the L1.
constexpr int DIG_STRIDE = MAX_D + 32;          // bytes between digit planes: 32 mod 128, so the four planes hit distinct banks
constexpr int HEAD_SC_OFF = (4 * DIG_STRIDE) / 4 + MAX_D / 32;   // floats: digit planes, then the block scales
constexpr int MAX_ROWS_HEAD = MAX_F - HEAD_SC_OFF;
constexpr int PARAM_FLOATS = 4 * MAX_D + kMegaBiasPackMax;   // LayerNorm vectors + bias slices

struct Ctrl {
    unsigned long long full[SLOTS];
    unsigned long long empty[SLOTS];
    unsigned long long pfull[2];
    unsigned long long pempty[2];
    volatile int stop;        // consumers -> producer: stop issuing copies
    volatile int consumed;    // weight items consumed when the consumers stopped
    volatile int pconsumed;   // parameter items consumed when the consumers stopped
    volatile int abort;       // a bounded wait ran out in this CTA
};

// shared memory carve-up (bytes)
constexpr int OFF_SLOTS = 0;
constexpr int OFF_PARAM = OFF_SLOTS + SLOTS * SLOT_BYTES;        // 2 parameter buffers
constexpr int OFF_ACT = OFF_PARAM + 2 * PARAM_FLOATS * 4;        // activation vector, swizzled float4 units
constexpr int OFF_XS = OFF_ACT + MAX_F * 4;                      // residual stream x
constexpr int OFF_PSUM = OFF_XS + MAX_D * 4;                     // 2 x 256 partial sums
constexpr int OFF_RED = OFF_PSUM + 2 * 256 * 4;                  // reductions
constexpr int OFF_LAYERS = OFF_RED + 256 * 4;                    // copy of the layer table
constexpr int OFF_WORK = OFF_LAYERS + kMegaMaxLayers * (int)sizeof(MegaLayer);   // 5 work descriptors
constexpr int OFF_CTRL = OFF_WORK + 512;
constexpr int SMEM_BYTES = OFF_CTRL + (int)sizeof(Ctrl);
static_assert(sizeof(MegaLayer) % 16 == 0, "layer table entries are copied as 16-byte words");
static_assert(OFF_PARAM % 16 == 0 && OFF_ACT % 16 == 0 && OFF_LAYERS % 16 == 0 && OFF_CTRL % 8 == 0, "alignment");
static_assert(SMEM_BYTES <= 195 * 1024, "shared memory budget: 196 KB carve-out less the 1 KB the system reserves");

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
// Tests the phase; a thread that finds it incomplete is suspended by the hardware until the
// phase completes or `hint_ns` pass, so a waiting warp does not burn issue slots.
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* b, uint32_t parity, uint32_t hint_ns = 2000) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(s32(b)), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* b) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(b)) : "memory");
}
// The same for the weight stream, marked evict-first in L2: every weight byte is used once per
// token and the matrices are larger than the L2, so letting them age normally would push the KV
// cache and the exchange vectors out to HBM between tokens.
__device__ __forceinline__ void bulk_g2s_stream(void* dst, const void* src, uint32_t bytes, unsigned long long* b) {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(b)), "l"(policy) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ int rows_per_item(int K) {
    const int g = mega_row_gran(K);
    int r = min(SLOT_Q / K, 256);      // 256 = partial-sum slots per item
    return r - r % g;
}

// This CTA's share of one kind of matrix (qkv, out, up, down, head), worked out once per
// launch: the integer divisions behind it are too slow for every phase's critical path.
struct Work {
    int r0, r1;        // owned rows
    int rpi;           // rows per ring item
    int gran;          // row granularity of a bulk copy
    int iters;         // 16-lane sweeps per row
    int ks_full;       // K split of an item of rpi rows
    int ks_last;       // K split of the last (shorter) item
    int pad;
};
enum { W_QKV = 0, W_OUT = 1, W_UP = 2, W_DOWN = 3, W_HEAD = 4, W_KINDS = 5 };

// This CTA's share of the LM head in 8-row strips. A ring item holds up to spi whole strips;
// its 8 x 32 tiles are dealt to the consumer warps as units (strip, K part): warp w of an item
// with ns strips handles unit w when w < ns * ks.
struct HeadWork {
    int s0, s1;        // owned strips
    int spi;           // strips per ring item
    int kb;            // tiles per strip (K / 32)
    int strip_bytes;
    int ks[2];         // K parts per strip: full item, last (shorter) item
    int pad;
    unsigned unit[2][CWARPS];   // per warp: strip | first tile << 8 | end tile << 16 (0xffffffff: idle)
};
static_assert(W_KINDS * 32 + sizeof(HeadWork) <= 512, "work descriptors");
__device__ void make_head_work(HeadWork* w, int N, int K, int c, int G) {
    mega_cta_strips(N, c, G, &w->s0, &w->s1);
    w->kb = K >> 5;
    w->strip_bytes = mega_strip_bytes(K);
    w->spi = max(1, min(SLOT_BYTES / w->strip_bytes, CWARPS));
    w->pad = 0;
    const int n = w->s1 - w->s0;
    const int ns_v[2] = {min(w->spi, max(n, 1)), n > 0 ? n - ((n - 1) / w->spi) * w->spi : 1};
    for (int v = 0; v < 2; ++v) {
        const int ns = ns_v[v], ks = max(1, min(w->kb, CWARPS / ns));
        w->ks[v] = ks;
        for (int u = 0; u < CWARPS; ++u) {
            if (u < ns * ks) {
                const int strip = u / ks, part = u - strip * ks;
                w->unit[v][u] = (unsigned)strip | (unsigned)(part * w->kb / ks) << 8 | (unsigned)((part + 1) * w->kb / ks) << 16;
            } else {
                w->unit[v][u] = 0xffffffffu;
            }
        }
    }
}

// Split K over several half warps when an item has few rows: the split with the fewest
// sweeps on the critical path (rounds over the 32 half warps x sweeps per unit).
__device__ int pick_ksplit(int rows, int iters) {
    int ksplit = 1, best = ((rows + 31) >> 5) * iters;
    const int cand[7] = {2, 3, 4, 6, 8, 12, 16};
    for (int i = 0; i < 7; ++i) {
        const int ks = cand[i];
        if (iters % ks == 0 && rows * ks <= 128) {
            const int cost = ((rows * ks + 31) >> 5) * (iters / ks);
            if (cost < best) { best = cost; ksplit = ks; }
        }
    }
    return ksplit;
}
__device__ void make_work(Work* w, int N, int K, int c, int G) {
    mega_cta_rows(N, K, c, G, &w->r0, &w->r1);
    w->rpi = rows_per_item(K);
    w->gran = mega_row_gran(K);
    w->iters = max(1, K >> 8);
    const int n = w->r1 - w->r0;
    const int last = n > 0 ? n - ((n - 1) / w->rpi) * w->rpi : 0;
    w->ks_full = pick_ksplit(w->rpi, w->iters);
    w->ks_last = last > 0 ? pick_ksplit(last, w->iters) : 1;
    w->pad = 0;
}

template <int B>
__device__ __forceinline__ float qbyte(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - 8388736.0f;
}
// 16 biased quants (one 16-byte chunk c of a row) times the swizzled activation.
__device__ __forceinline__ float dot16(const uint4 w, const float4* __restrict__ act, int c) {
    const int sw = (c >> 1) & 3, base = 4 * c;
    const float4 x0 = act[base + (0 ^ sw)], x1 = act[base + (1 ^ sw)], x2 = act[base + (2 ^ sw)], x3 = act[base + (3 ^ sw)];
    // four independent chains of four dependent fused multiply-adds
    float a = x0.x * qbyte<0>(w.x), b = x1.x * qbyte<0>(w.y), c2 = x2.x * qbyte<0>(w.z), e = x3.x * qbyte<0>(w.w);
    a = fmaf(x0.y, qbyte<1>(w.x), a); b = fmaf(x1.y, qbyte<1>(w.y), b); c2 = fmaf(x2.y, qbyte<1>(w.z), c2); e = fmaf(x3.y, qbyte<1>(w.w), e);
    a = fmaf(x0.z, qbyte<2>(w.x), a); b = fmaf(x1.z, qbyte<2>(w.y), b); c2 = fmaf(x2.z, qbyte<2>(w.z), c2); e = fmaf(x3.z, qbyte<2>(w.w), e);
    a = fmaf(x0.w, qbyte<3>(w.x), a); b = fmaf(x1.w, qbyte<3>(w.y), b); c2 = fmaf(x2.w, qbyte<3>(w.z), c2); e = fmaf(x3.w, qbyte<3>(w.w), e);
    return (a + b) + (c2 + e);
}
// element i of the swizzled activation vector
__device__ __forceinline__ int act_index(int i) {
    const int u = i >> 2;
    return ((u ^ ((u >> 3) & 3)) << 2) | (i & 3);
}

struct Cta {
    const MegaParams& p;
    unsigned char* smem;
    Ctrl* ctrl;
    const MegaLayer* layers;   // shared-memory copy of the layer table
    const Work* work;          // shared-memory work descriptors, one per matrix kind
    const HeadWork* hwork;     // ... and the LM head's
    float4* act4;
    float* act;
    float* xs;
    float* sc;            // this CTA's slice of the logits: the tail of the activation buffer
    float* psum;
    float* red;
    int c, G, tid;
    int item;            // weight items consumed (consumers) / issued (producer)
    int pitem;           // parameter items consumed / issued
    unsigned bar_target;
    int trace_n;         // next slot of the phase timeline; < 0 when this thread does not trace
    __device__ signed char* dig() const { return (signed char*)act; }                 // head phase: digit planes
    __device__ float* xsc() const { return act + (4 * DIG_STRIDE) / 4; }             // ... and their block scales
    __device__ unsigned char* slot_q(int s) const { return smem + OFF_SLOTS + s * SLOT_BYTES; }
    __device__ const __half* slot_d(int s) const { return (const __half*)(smem + OFF_SLOTS + s * SLOT_BYTES + SLOT_Q); }
    __device__ float* param(int b) const { return (float*)(smem + OFF_PARAM) + b * PARAM_FLOATS; }
};

__device__ __forceinline__ bool timed_out(const Cta& k, long long t0) { return clock64() - t0 > k.p.wait_cycles; }

// Phase timeline: thread 0 of every CTA stores the global timer at every phase boundary.
__device__ __forceinline__ void mark(Cta& k) {
    if (k.trace_n >= 0 && k.trace_n < k.p.trace_cap) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        k.p.trace[(size_t)k.c * k.p.trace_cap + k.trace_n++] = t;
    }
}

__device__ void raise_timeout(Cta& k) {
    k.ctrl->abort = 1;
    atomicExch(k.p.status, FC_E_TIMEOUT);
}

// ------------------------------------------------------------------ producer
// Waits until `bar` completes phase `parity`; false when told to stop or out of time.
__device__ bool producer_wait(Cta& k, unsigned long long* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (k.ctrl->stop) return false;
        if (timed_out(k, t0)) { atomicExch(k.p.status, FC_E_TIMEOUT); return false; }
    }
    return k.ctrl->stop == 0;
}

// Issues the bulk copies of one matrix share. Returns false when told to stop.
__device__ bool produce_matrix(Cta& k, const QMat& w, int kind) {
    const Work wk = k.work[kind];
    const int r0 = wk.r0, r1 = wk.r1, rpi = wk.rpi, g = wk.gran;
    for (int r = r0; r < r1; r += rpi) {
        const int rows = min(rpi, r1 - r);
        const int rows_c = (rows + g - 1) & ~(g - 1);       // g is a power of two; padded rows exist up to N_pad
        const int slot = k.item % SLOTS;
        if (!producer_wait(k, &k.ctrl->empty[slot], ((k.item / SLOTS) & 1) ^ 1)) return false;
        const uint32_t qb = (uint32_t)rows_c * w.K, db = qb >> 4;
        mbar_expect_tx(&k.ctrl->full[slot], qb + db);
        bulk_g2s_stream(k.slot_q(slot), w.qu + (size_t)r * w.K, qb, &k.ctrl->full[slot]);
        bulk_g2s_stream((void*)k.slot_d(slot), w.d + (size_t)r * (w.K >> 5), db, &k.ctrl->full[slot]);
        ++k.item;
    }
    return true;
}

// The LM head share: one bulk copy per ring item (whole strips of the tile-major copy).
__device__ bool produce_head(Cta& k) {
    const HeadWork& wk = *k.hwork;
    for (int s = wk.s0; s < wk.s1; s += wk.spi) {
        const int ns = min(wk.spi, wk.s1 - s);
        const int slot = k.item % SLOTS;
        if (!producer_wait(k, &k.ctrl->empty[slot], ((k.item / SLOTS) & 1) ^ 1)) return false;
        const uint32_t bytes = (uint32_t)ns * wk.strip_bytes;
        mbar_expect_tx(&k.ctrl->full[slot], bytes);
        bulk_g2s_stream(k.slot_q(slot), k.p.head.t + (size_t)s * wk.strip_bytes, bytes, &k.ctrl->full[slot]);
        ++k.item;
    }
    return true;
}

// LayerNorm vectors (4d floats) and, for a block, this CTA's bias slices.
__device__ bool produce_params(Cta& k, const float* lnpack, const float* biaspack) {
    const int b = k.pitem & 1;
    if (!producer_wait(k, &k.ctrl->pempty[b], ((k.pitem >> 1) & 1) ^ 1)) return false;
    const uint32_t lb = (uint32_t)k.p.d * 16, bb = biaspack ? (uint32_t)k.p.bias_pack * 4 : 0;
    mbar_expect_tx(&k.ctrl->pfull[b], lb + bb);
    bulk_g2s(k.param(b), lnpack, lb, &k.ctrl->pfull[b]);
    if (biaspack) bulk_g2s(k.param(b) + 4 * MAX_D, biaspack + (size_t)k.c * k.p.bias_pack, bb, &k.ctrl->pfull[b]);
    ++k.pitem;
    return true;
}

__device__ void producer(Cta& k) {
    const MegaParams& p = k.p;
    if (p.withhold) return;   // test hook: nothing is copied, the consumers' first wait runs out
    for (int step = 0; step < p.n_steps; ++step) {
        for (int l = 0; l < p.L; ++l) {
            const MegaLayer& L = k.layers[l];
            if (!produce_params(k, L.lnpack, L.biaspack)) return;
            if (!produce_matrix(k, L.qkv, W_QKV) || !produce_matrix(k, L.out, W_OUT) || !produce_matrix(k, L.up, W_UP) ||
                !produce_matrix(k, L.down, W_DOWN))
                return;
        }
        if (step >= p.head_from) {
            if (!produce_params(k, p.lnfpack, nullptr) || !produce_head(k)) return;
        }
    }
}

// ------------------------------------------------------------------ consumer helpers
// Fixed-order sum / max over the 512 consumer threads.
__device__ float csum(Cta& k, float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    consumer_sync();
    if ((k.tid & 31) == 0) k.red[k.tid >> 5] = v;
    consumer_sync();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) t += k.red[w];
    return t;
}
__device__ float cmax(Cta& k, float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    consumer_sync();
    if ((k.tid & 31) == 0) k.red[k.tid >> 5] = v;
    consumer_sync();
    float t = -INFINITY;
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) t = fmaxf(t, k.red[w]);
    return t;
}

// The 32 values a warp holds (one per lane) become block kb of the activation vector: a
// power-of-two block scale and, per value, four signed base-128 digits (most significant
// first) of round(v / scale), |v / scale| <= 2^27.
__device__ __forceinline__ void put_block(Cta& k, int kb, float v) {
    float m = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // m < 2^e; e is kept where both 2^(27-e) and 2^(e-27) are normal floats
    int e = (int)((__float_as_uint(m) >> 23) & 0xffu) - 126;
    e = max(e, -80);
    const float up = __uint_as_float((unsigned)(127 + 27 - e) << 23);
    int X = __float2int_rn(v * up);
    const int d3 = ((X + 64) & 127) - 64;
    X = (X - d3) >> 7;
    const int d2 = ((X + 64) & 127) - 64;
    X = (X - d2) >> 7;
    const int d1 = ((X + 64) & 127) - 64;
    X = (X - d1) >> 7;                                   // the leading digit, in [-64, 64]
    signed char* dg = k.dig() + kb * 32 + (k.tid & 31);
    dg[0] = (signed char)X;
    dg[DIG_STRIDE] = (signed char)d1;
    dg[2 * DIG_STRIDE] = (signed char)d2;
    dg[3 * DIG_STRIDE] = (signed char)d3;
    if ((k.tid & 31) == 0) k.xsc()[kb] = __uint_as_float((unsigned)(127 - 27 + e) << 23);
}

// layer/norm.rs:46-82 on xs[0..d) -> act (swizzled floats, or digit planes for the LM head);
// g, b in shared memory.
// Two-level reductions: each thread owns elements tid and tid + 512, each warp leaves one
// partial per statistic in shared memory, every thread adds the 16 partials in the same order.
__device__ void layernorm_to_act(Cta& k, const float* g, const float* b, bool digits = false) {
    const int d = k.p.d, lane = k.tid & 31, wid = k.tid >> 5;
    const bool h0 = k.tid < d, h1 = k.tid + CONSUMERS < d;
    const float v0 = h0 ? k.xs[k.tid] : 0.0f, v1 = h1 ? k.xs[k.tid + CONSUMERS] : 0.0f;
    float s = v0 + v1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) k.red[wid] = s;
    consumer_sync();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) tot += k.red[w];
    const float mean = tot / (float)d;
    const float t0 = v0 - mean, t1 = v1 - mean;
    float q = (h0 ? t0 * t0 : 0.0f) + (h1 ? t1 * t1 : 0.0f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    if (lane == 0) k.red[CWARPS + wid] = q;
    consumer_sync();
    float qt = 0.0f;
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) qt += k.red[CWARPS + w];
    const float sd = sqrtf(qt / (float)d + 1e-5f);
    if (digits) {
        consumer_sync();   // every read of xs and of the old activation is over before the planes are written
        // d is a multiple of 32: a warp's 32 elements are one whole block or none
        if (h0) put_block(k, wid, (t0 / sd) * g[k.tid] + b[k.tid]);
        if (h1) put_block(k, CWARPS + wid, (t1 / sd) * g[k.tid + CONSUMERS] + b[k.tid + CONSUMERS]);
    } else {
        if (h0) k.act[act_index(k.tid)] = (t0 / sd) * g[k.tid] + b[k.tid];
        if (h1) k.act[act_index(k.tid + CONSUMERS)] = (t1 / sd) * g[k.tid + CONSUMERS] + b[k.tid + CONSUMERS];
    }
    consumer_sync();
}

// Waits (every consumer thread) for a full barrier; the abort flag is read after a CTA-wide
// sync so that all consumer threads take the same branch.
__device__ bool consumer_wait(Cta& k, unsigned long long* bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (timed_out(k, t0)) { raise_timeout(k); break; }
    }
    consumer_sync();
    return k.ctrl->abort == 0;
}

// Grid barrier over all CTAs (consumer thread 0 arrives and polls). Returns false on timeout
// or when another CTA reported one.
__device__ bool grid_barrier(Cta& k) {
    consumer_sync();                     // every thread's global writes precede the release below
    k.bar_target += (unsigned)k.G;
    if (k.tid == 0) {
        red_release_add(k.p.bar, 1u);
        const long long t0 = clock64();
        unsigned polls = 0;
        while ((int)(ld_acquire(k.p.bar) - k.bar_target) < 0) {
            // the status word and the clock are only looked at every 64 polls
            if ((++polls & 63u) == 0) {
                if (*(volatile int*)k.p.status != 0) { k.ctrl->abort = 1; break; }
                if (timed_out(k, t0)) { raise_timeout(k); break; }
            }
        }
    }
    consumer_sync();
    return k.ctrl->abort == 0;
}

// Consumes this CTA's share of matrix w against the activation in act; epi(n, i, value) is
// called once per owned output row n (i = n - first owned row) by one thread.
template <class Epi>
__device__ bool consume_matrix(Cta& k, const QMat& w, int kind, Epi epi) {
    const Work wk = k.work[kind];
    const int r0 = wk.r0, r1 = wk.r1, rpi = wk.rpi, iters = wk.iters;
    const int K = w.K, chunks = K >> 4, kb_row = K >> 5;
    const int hw = k.tid >> 4, hl = k.tid & 15;
    const unsigned hmask = 0xFFFFu << (k.tid & 16);
    for (int r = r0; r < r1; r += rpi) {
        const int rows = min(rpi, r1 - r);
        const int ksplit = rows == rpi ? wk.ks_full : wk.ks_last;   // K split over half warps
        const int slot = k.item % SLOTS;
        if (!consumer_wait(k, &k.ctrl->full[slot], (k.item / SLOTS) & 1)) return false;
        const unsigned char* q = k.slot_q(slot);
        const __half* ds = k.slot_d(slot);
        float* ps = k.psum + (k.item & 1) * 256;
        const int units = rows * ksplit, per = iters / ksplit;
        // unit u = (row, part); the first unit's quotient is the only division
        int row = hw / ksplit, part = hw - row * ksplit;
        const int drow = (CONSUMERS / 16) / ksplit, dpart = (CONSUMERS / 16) - drow * ksplit;
        for (int u = hw; u < units; u += CONSUMERS / 16) {
            float acc = 0.0f;
            for (int i = part * per; i < (part + 1) * per; ++i) {
                const int cc = i * 16 + hl;
                if (cc < chunks) {
                    const uint4 wv = *(const uint4*)(q + (size_t)row * K + cc * 16);
                    const float scale = __half2float(ds[row * kb_row + (cc >> 1)]);
                    acc = fmaf(scale, dot16(wv, k.act4, cc), acc);
                }
            }
            acc += __shfl_xor_sync(hmask, acc, 8);
            acc += __shfl_xor_sync(hmask, acc, 4);
            acc += __shfl_xor_sync(hmask, acc, 2);
            acc += __shfl_xor_sync(hmask, acc, 1);
            if (hl == 0) ps[u] = acc;
            part += dpart;
            row += drow;
            if (part >= ksplit) { part -= ksplit; row += 1; }
        }
        consumer_sync();                                   // slot fully read, partial sums visible
        if ((k.tid & 31) == 0) mbar_arrive(&k.ctrl->empty[slot]);
        for (int row = k.tid; row < rows; row += CONSUMERS) {
            float v = 0.0f;
            for (int part = 0; part < ksplit; ++part) v += ps[row * ksplit + part];
            epi(r + row, r + row - r0, v);
        }
        ++k.item;
    }
    return true;
}

// One integer MMA: D[16 x 8] = A[16 x 32] (s8, row) x B[32 x 8] (s8, col). Rows 0..3 of A are
// the digit planes of 32 activations, B is one 8 x 32 tile of quants. With lane = 4 g + t the
// lane supplies A[g][8t .. 8t+7] (a0, a2; rows 8.. are zero) and B[8t .. 8t+7][g] (b0, b1) and
// receives D[g][2t], D[g][2t+1]: digit row g against weight rows 2t and 2t+1. The k index
// inside the block is permuted the same way on both sides, which leaves the sums unchanged.
__device__ __forceinline__ void mma_s8(int& c0, int& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    int c2 __attribute__((unused)), c3 __attribute__((unused));   // rows 8..15 of D: always zero here
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
    (void)c2; (void)c3;
}

// The LM head share on the integer tensor cores: logits of the owned rows n < V go to lg[n -
// first owned row] (shared memory) and to the global logits.
__device__ bool consume_head(Cta& k, float* lg) {
    const MegaParams& p = k.p;
    const HeadWork& wk = *k.hwork;
    const int lane = k.tid & 31, wid = k.tid >> 5, g = lane >> 2, t = lane & 3;
    const int r0 = min(wk.s0 * kMegaStripRows, p.V);
    // digit g carries weight 128^(3-g); lanes of the unused rows 4..7 contribute nothing
    const float digit_w = g == 0 ? 2097152.0f : g == 1 ? 16384.0f : g == 2 ? 128.0f : g == 3 ? 1.0f : 0.0f;
    const signed char* my_dig = k.dig() + (g & 3) * DIG_STRIDE + t * 8;
    const float* xsc = k.xsc();
    for (int s = wk.s0; s < wk.s1; s += wk.spi) {
        const int ns = min(wk.spi, wk.s1 - s);
        const int var = ns == wk.spi ? 0 : 1;
        const int slot = k.item % SLOTS;
        if (!consumer_wait(k, &k.ctrl->full[slot], (k.item / SLOTS) & 1)) return false;
        float* ps = k.psum + (k.item & 1) * 256;
        const unsigned unit = wk.unit[var][wid];
        if (unit != 0xffffffffu) {
            const int strip = unit & 0xff, kb0 = (unit >> 8) & 0xff, kb1 = (unit >> 16) & 0xff;
            const unsigned char* tile = k.slot_q(slot) + strip * wk.strip_bytes + kb0 * kMegaTileBytes;
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 2
            for (int kb = kb0; kb < kb1; ++kb, tile += kMegaTileBytes) {
                const uint2 b = *(const uint2*)(tile + g * 32 + t * 8);
                const __half2 sc = *(const __half2*)(tile + 256 + t * 4);
                uint2 a = make_uint2(0u, 0u);
                if (g < 4) a = *(const uint2*)(my_dig + kb * 32);
                const float xs = xsc[kb];
                int c0, c1;
                mma_s8(c0, c1, a.x, a.y, b.x, b.y);
                const float2 f = __half22float2(sc);
                acc0 = fmaf((float)c0, f.x * xs, acc0);
                acc1 = fmaf((float)c1, f.y * xs, acc1);
            }
            acc0 *= digit_w;
            acc1 *= digit_w;
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 4);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 4);
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 8);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 8);
            if (lane < 4) { ps[wid * 8 + 2 * t] = acc0; ps[wid * 8 + 2 * t + 1] = acc1; }
        }
        consumer_sync();                                   // slot fully read, partial sums visible
        if (lane == 0) mbar_arrive(&k.ctrl->empty[slot]);
        if (k.tid < ns * kMegaStripRows) {
            const int strip = k.tid >> 3, r = k.tid & 7, ks = wk.ks[var];
            float v = 0.0f;
            for (int part = 0; part < ks; ++part) v += ps[(strip * ks + part) * 8 + r];
            const int n = (s + strip) * kMegaStripRows + r;
            if (n < p.V) { lg[n - r0] = v; p.logits[n] = v; }
        }
        ++k.item;
    }
    return true;
}

// CTAs per head for a context of `len` keys. Up to kWholeHead keys one CTA handles the whole
// head and writes the finished attention output: the split into partials costs an extra grid
// barrier and a combine phase, which only pays once a single CTA would need many sweeps.
// Beyond that about 64 keys per CTA, at most attn_splits.
constexpr int kWholeHead = 576;
__device__ __forceinline__ int attn_splits_for(const MegaParams& p, int len) {
    if (len <= kWholeHead) return 1;
    return max(1, min(p.attn_splits, (len + 63) >> 6));
}

// transformer.rs:246-283 split over CTAs: CTA (h, s) handles keys [s*len/S, (s+1)*len/S) of
// head h. Inside the CTA every half warp runs an online softmax over its own keys (no CTA-wide
// synchronisation while keys are processed); the halves of a warp merge, then the 16 warp
// partials are combined once at the end in a fixed order. With S == 1 the result is the head's attention
// output, written to attg; otherwise (max, sum-exp, unnormalised out[hd]) go to partg.
__device__ void attention_partial(Cta& k, int l, int len) {
    const MegaParams& p = k.p;
    const int S = attn_splits_for(p, len), hd = p.d / p.H;
    if (k.c >= p.H * S) return;
    const int h = k.c / S, s = k.c - h * S, hs = h * hd;
    const int j0 = (int)((long long)s * len / S), j1 = (int)((long long)(s + 1) * len / S);
    const float* kc = p.kc + (size_t)l * p.T * p.d + hs;
    const float* vc = p.vc + (size_t)l * p.T * p.d + hs;
    const int lane = k.tid & 31, wid = k.tid >> 5, hf = lane >> 4, li = lane & 15;
    // A half warp takes one key at a time: lane li owns head dimensions 4 li .. 4 li + 3
    // (hd <= 64), so a K or V row is one 16-byte load per lane and a dot product needs four
    // shuffle steps. Both halves hold the query.
    const bool has = 4 * li < hd;
    const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float4 q = has ? __ldcg((const float4*)(p.qg + hs) + li) : zero4;
    const float scale = 1.0f / sqrtf((float)hd);
    float m = -INFINITY, lsum = 0.0f;
    float4 o = zero4;
    // Warp wid owns the key pairs j0 + 2 wid, j0 + 2 wid + 32, ...; half hf takes key hf of a
    // pair. Two pairs (four keys per warp) are requested together, one step ahead of the
    // arithmetic.
    constexpr int U = 2;
    struct Rows { float4 kk[U], vv[U]; };
    auto key_of = [&](int jb, int u) { return jb + u * (2 * CWARPS) + hf; };
    auto request = [&](Rows& r, int jb) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = key_of(jb, u);
            const bool on = j < j1 && has;
            const size_t off = (size_t)j * p.d;
            r.kk[u] = on ? __ldcg((const float4*)(kc + off) + li) : zero4;
            r.vv[u] = on ? __ldcg((const float4*)(vc + off) + li) : zero4;
        }
    };
    auto absorb = [&](const Rows& r, int jb) {
        float dot[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            dot[u] = fmaf(q.w, r.kk[u].w, fmaf(q.z, r.kk[u].z, fmaf(q.y, r.kk[u].y, q.x * r.kk[u].x)));
#pragma unroll
        for (int sh = 8; sh > 0; sh >>= 1) {
#pragma unroll
            for (int u = 0; u < U; ++u) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], sh);
        }
        // keys past the range score -inf and weigh 0
        float mn = m;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            dot[u] = key_of(jb, u) < j1 ? dot[u] * scale : -INFINITY;
            mn = fmaxf(mn, dot[u]);
        }
        if (mn > -INFINITY) {                           // this half has seen a key
            const float corr = expf(m - mn);            // m == -inf: 0
            float pj[U];
#pragma unroll
            for (int u = 0; u < U; ++u) pj[u] = expf(dot[u] - mn);
            lsum = fmaf(lsum, corr, pj[0] + pj[1]);
            o.x = fmaf(o.x, corr, fmaf(pj[0], r.vv[0].x, pj[1] * r.vv[1].x));
            o.y = fmaf(o.y, corr, fmaf(pj[0], r.vv[0].y, pj[1] * r.vv[1].y));
            o.z = fmaf(o.z, corr, fmaf(pj[0], r.vv[0].z, pj[1] * r.vv[1].z));
            o.w = fmaf(o.w, corr, fmaf(pj[0], r.vv[0].w, pj[1] * r.vv[1].w));
            m = mn;
        }
    };
    {
        constexpr int STEP = U * 2 * CWARPS;            // keys per sweep of the CTA
        Rows ra, rb;
        int jb = j0 + 2 * wid;
        if (jb < j1) request(ra, jb);
        while (jb < j1) {
            if (jb + STEP < j1) request(rb, jb + STEP);
            absorb(ra, jb);
            jb += STEP;
            if (jb >= j1) break;
            if (jb + STEP < j1) request(ra, jb + STEP);
            absorb(rb, jb);
            jb += STEP;
        }
    }
    // the two halves of the warp merge their running (max, sum, out) in a fixed order
    {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, 16), l2 = __shfl_xor_sync(0xffffffffu, lsum, 16);
        const float ox = __shfl_xor_sync(0xffffffffu, o.x, 16), oy = __shfl_xor_sync(0xffffffffu, o.y, 16);
        const float oz = __shfl_xor_sync(0xffffffffu, o.z, 16), ow = __shfl_xor_sync(0xffffffffu, o.w, 16);
        const float M = fmaxf(m, m2);
        // half 0's terms first in both halves, so that they agree bit for bit
        const float ma = hf ? m2 : m, mb = hf ? m : m2;
        const float fa = ma > -INFINITY ? expf(ma - M) : 0.0f, fb = mb > -INFINITY ? expf(mb - M) : 0.0f;
        const float la = hf ? l2 : lsum, lb = hf ? lsum : l2;
        lsum = fmaf(la, fa, lb * fb);
        o.x = fmaf(hf ? ox : o.x, fa, (hf ? o.x : ox) * fb);
        o.y = fmaf(hf ? oy : o.y, fa, (hf ? o.y : oy) * fb);
        o.z = fmaf(hf ? oz : o.z, fa, (hf ? o.z : oz) * fb);
        o.w = fmaf(hf ? ow : o.w, fa, (hf ? o.w : ow) * fb);
        m = M;
    }
    float* part = k.act;                                // act is free during the attention phase
    float* mine = part + wid * 66;
    if (lane == 0) { mine[0] = m; mine[1] = lsum; }
    if (hf == 0 && has) { mine[2 + 4 * li] = o.x; mine[3 + 4 * li] = o.y; mine[4 + 4 * li] = o.z; mine[5 + 4 * li] = o.w; }
    consumer_sync();
    if (k.tid < 64) {
        // warps 0 and 1 each work out the 16 rescaling factors (lane w: warp w) and share them
        // by shuffles; thread t then owns output dimension t
        const float mw = lane < CWARPS ? part[lane * 66] : -INFINITY;
        float M = mw;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        M = __shfl_sync(0xffffffffu, M, 0);
        const float f = mw > -INFINITY ? expf(mw - M) : 0.0f;
        const float lf = lane < CWARPS ? part[lane * 66 + 1] * f : 0.0f;
        float Lsum = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < CWARPS; ++w) {
            Lsum += __shfl_sync(0xffffffffu, lf, w);
            O = fmaf(k.tid < hd ? part[w * 66 + 2 + k.tid] : 0.0f, __shfl_sync(0xffffffffu, f, w), O);
        }
        if (k.tid < hd) {
            if (S == 1) {
                p.attg[hs + k.tid] = O / Lsum;
            } else {
                float* out = p.partg + (size_t)k.c * (hd + 2);
                out[2 + k.tid] = O;
                if (k.tid == 0) { out[0] = M; out[1] = Lsum; }
            }
        }
    }
}

// Combines the S partials of every head into the attention output, written to act. A thread
// owns elements tid and tid + 512 of the row (d <= 1024) and requests everything it needs for
// both before the first use, so the whole phase costs one round trip to L2.
__device__ void attention_combine(Cta& k, int len) {
    const MegaParams& p = k.p;
    const int S = attn_splits_for(p, len), hd = p.d / p.H;
    float ms[2][8], ls[2][8], os[2][8];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int t = k.tid + e * CONSUMERS;
        const bool live = t < p.d;
        const int h = live ? t / hd : 0, cc = live ? t - h * hd : 0;
        const float* base = p.partg + (size_t)h * S * (hd + 2);
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const bool on = live && s < S;
            ms[e][s] = on ? __ldcg(base + s * (hd + 2)) : -INFINITY;
            ls[e][s] = on ? __ldcg(base + s * (hd + 2) + 1) : 0.0f;
            os[e][s] = on ? __ldcg(base + s * (hd + 2) + 2 + cc) : 0.0f;
        }
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int t = k.tid + e * CONSUMERS;
        if (t < p.d) {
            float M = -INFINITY;
#pragma unroll
            for (int s = 0; s < 8; ++s) M = fmaxf(M, ms[e][s]);
            float Lsum = 0.0f, O = 0.0f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const float f = ms[e][s] > -INFINITY ? expf(ms[e][s] - M) : 0.0f;
                Lsum = fmaf(ls[e][s], f, Lsum);
                O = fmaf(os[e][s], f, O);
            }
            k.act[act_index(t)] = O / Lsum;
        }
    }
    consumer_sync();
}

// n <= MAX_F floats from global memory into shared memory; every thread requests all of its
// elements before the first one is stored, so the whole vector costs one round trip to L2.
__device__ void load_vec(Cta& k, const float* g, float* dst, int n, bool swizzle) {
    float v[MAX_F / CONSUMERS];
#pragma unroll
    for (int j = 0; j < MAX_F / CONSUMERS; ++j) {
        const int i = k.tid + j * CONSUMERS;
        v[j] = i < n ? __ldcg(g + i) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < MAX_F / CONSUMERS; ++j) {
        const int i = k.tid + j * CONSUMERS;
        if (i < n) dst[swizzle ? act_index(i) : i] = v[j];
    }
    consumer_sync();
}

struct ArgBest { float v; int i; };
__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
// Fixed-order arg-best over the consumer threads; every thread gets the result.
__device__ ArgBest cbest(Cta& k, ArgBest best) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgBest other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
        best = better(best, other);
    }
    consumer_sync();
    if ((k.tid & 31) == 0) { k.red[k.tid >> 5] = best.v; k.red[32 + (k.tid >> 5)] = __int_as_float(best.i); }
    consumer_sync();
    ArgBest r{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int w = 0; w < CWARPS; ++w) r = better(r, ArgBest{k.red[w], __float_as_int(k.red[32 + w])});
    return r;
}

// ------------------------------------------------------------------ consumer
__device__ void consumer(Cta& k) {
    const MegaParams& p = k.p;
    const int d = p.d, V = p.V;
    // decode state, tracked identically by every CTA
    int pos = p.state->pos, fed = p.state->fed, tail = p.state->tail, done = p.state->done, error = p.state->error;
    const int eos = p.state->eos;
    int pending_idx = -1, pending_id = 0;   // the token this launch appended last (known to every CTA)
    int boff[4];
    mega_bias_offsets(d, p.F, k.c, k.G, boff);
    for (int step = 0; step < p.n_steps && !done && !error; ++step) {
        const int id = fed == pending_idx ? pending_id : (fed < p.queue_cap ? __ldcg(p.queue + fed) : -1);
        // embedding.rs:71-82, transformer.rs:237-242: errors, not traps
        if (id < 0 || id >= V || pos >= p.T) { error = FC_E_DIM; break; }
        // layer/embedding.rs:70-90: x = tok[id] + pos[pos]
        for (int cc = k.tid; cc < d; cc += CONSUMERS) {
            const float dq = __half2float(p.tok.d[(size_t)id * (d >> 5) + (cc >> 5)]);
            const int q = (int)p.tok.qu[(size_t)id * d + cc] - 128;
            k.xs[cc] = dq * (float)q + p.pos[(size_t)pos * d + cc];
        }
        consumer_sync();
        // the phase timeline covers the last step of the launch
        k.trace_n = (p.trace && k.tid == 0 && step + 1 == p.n_steps) ? 0 : -1;
        mark(k);
        const int len = pos + 1;
        bool ok = true;
        for (int l = 0; l < p.L && ok; ++l) {
            const MegaLayer& L = k.layers[l];
            float* kc = p.kc + ((size_t)l * p.T + pos) * d;
            float* vc = p.vc + ((size_t)l * p.T + pos) * d;
            const int pb = k.pitem & 1;
            ok = consumer_wait(k, &k.ctrl->pfull[pb], (k.pitem >> 1) & 1);
            if (!ok) break;
            const float* prm = k.param(pb);
            const float* bias = prm + 4 * MAX_D;
            // LN1 -> q, k, v (k, v appended to the cache at `pos`)
            layernorm_to_act(k, prm, prm + d);
            mark(k);
            ok = consume_matrix(k, L.qkv, W_QKV, [&](int n, int i, float v) {
                v += bias[boff[0] + i];
                if (n < d) p.qg[n] = v; else if (n < 2 * d) kc[n - d] = v; else vc[n - 2 * d] = v;
            });
            mark(k);
            ok = ok && grid_barrier(k);
            if (!ok) break;
            mark(k);
            attention_partial(k, l, len);
            mark(k);
            ok = grid_barrier(k);
            if (!ok) break;
            mark(k);
            if (attn_splits_for(p, len) == 1) load_vec(k, p.attg, k.act, d, true);
            else attention_combine(k, len);
            mark(k);
            // out-proj + residual: x1 = x + (W att + b)
            ok = consume_matrix(k, L.out, W_OUT, [&](int n, int i, float v) { p.x1g[n] = k.xs[n] + (v + bias[boff[1] + i]); });
            mark(k);
            ok = ok && grid_barrier(k);
            if (!ok) break;
            mark(k);
            load_vec(k, p.x1g, k.xs, d, false);
            layernorm_to_act(k, prm + 2 * d, prm + 3 * d);
            mark(k);
            ok = consume_matrix(k, L.up, W_UP, [&](int n, int i, float v) { p.hidg[n] = gelu_f(v + bias[boff[2] + i]); });
            mark(k);
            ok = ok && grid_barrier(k);
            if (!ok) break;
            mark(k);
            load_vec(k, p.hidg, k.act, p.F, true);
            mark(k);
            ok = consume_matrix(k, L.down, W_DOWN, [&](int n, int i, float v) { p.xg[n] = k.xs[n] + (v + bias[boff[3] + i]); });
            mark(k);
            ok = ok && grid_barrier(k);          // its first sync also ends every read of the parameters
            if (!ok) break;
            if ((k.tid & 31) == 0) mbar_arrive(&k.ctrl->pempty[pb]);
            ++k.pitem;
            mark(k);
            load_vec(k, p.xg, k.xs, d, false);
            mark(k);   // 15 marks per block
        }
        if (!ok) break;
        if (step >= p.head_from) {
            const int pb = k.pitem & 1;
            if (!consumer_wait(k, &k.ctrl->pfull[pb], (k.pitem >> 1) & 1)) break;
            layernorm_to_act(k, k.param(pb), k.param(pb) + d, /*digits=*/true);   // ends with a sync
            if ((k.tid & 31) == 0) mbar_arrive(&k.ctrl->pempty[pb]);
            ++k.pitem;
            const int r0 = min(k.hwork->s0 * kMegaStripRows, V), r1 = min(k.hwork->s1 * kMegaStripRows, V);
            float* lg = k.sc;                      // this CTA's logits [r1 - r0]
            ok = consume_head(k, lg);
            if (!ok) break;
            consumer_sync();
            // ops.rs:478-502: max, exp(x - max), sum — per CTA, then combined across CTAs
            float m = -INFINITY;
            for (int i = k.tid; i < r1 - r0; i += CONSUMERS) m = fmaxf(m, lg[i]);
            m = cmax(k, m);
            float e = 0.0f;
            for (int i = k.tid; i < r1 - r0; i += CONSUMERS) e += expf(lg[i] - m);
            e = csum(k, e);
            if (k.tid == 0) { p.statg[4 * k.c] = m; p.statg[4 * k.c + 1] = e; }
            mark(k);
            if (!grid_barrier(k)) break;
            mark(k);
            // every CTA combines the per-CTA (max, sum) pairs: one load per thread, then
            // fixed-order block reductions (G <= 512)
            const float mc = k.tid < k.G ? __ldcg(p.statg + 4 * k.tid) : -INFINITY;
            const float ec = k.tid < k.G ? __ldcg(p.statg + 4 * k.tid + 1) : 0.0f;
            const float M = cmax(k, mc);
            const float sum = csum(k, mc > -INFINITY ? ec * expf(mc - M) : 0.0f);
            const bool last = step + 1 == p.n_steps;
            if (p.probs && last)
                for (int i = k.tid; i < r1 - r0; i += CONSUMERS) p.probs[r0 + i] = expf(lg[i] - M) / sum;
            if (p.select) {
                // token_stream.rs:134 + sampling.rs:96-104: first index of the largest ln(max(p, 1e-12))
                ArgBest best{-INFINITY, 0x7fffffff};
                for (int i = k.tid; i < r1 - r0; i += CONSUMERS)
                    best = better(best, ArgBest{logf(fmaxf(expf(lg[i] - M) / sum, 1e-12f)), r0 + i});
                best = cbest(k, best);
                if (k.tid == 0) {
                    p.statg[4 * k.c + 2] = best.v;
                    p.statg[4 * k.c + 3] = __int_as_float(best.i);
                }
                mark(k);
                if (!grid_barrier(k)) break;
                mark(k);
                // one candidate per thread, then the same fixed-order reduction in every CTA
                ArgBest win{-INFINITY, 0x7fffffff};
                if (k.tid < k.G) win = ArgBest{__ldcg(p.statg + 4 * k.tid + 2), __float_as_int(__ldcg(p.statg + 4 * k.tid + 3))};
                win = cbest(k, win);
                mark(k);
                if (win.i == eos) {
                    done = 1;
                } else if (tail < p.queue_cap) {
                    if (k.c == 0 && k.tid == 0) p.queue[tail] = win.i;
                    pending_idx = tail;
                    pending_id = win.i;
                    tail += 1;
                } else {
                    error = FC_E_DIM;
                }
            }
        }
        pos += 1;
        fed += 1;
    }
    if (k.c == 0 && k.tid == 0) {
        p.state->pos = pos; p.state->fed = fed; p.state->tail = tail; p.state->done = done;
        if (error) p.state->error = error;
    }
}

}  // namespace

__global__ void __launch_bounds__(THREADS, 1) decode_mega_kernel(const __grid_constant__ MegaParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Ctrl* ctrl = (Ctrl*)(smem + OFF_CTRL);
    if (threadIdx.x == 0) {
        for (int s = 0; s < SLOTS; ++s) {
            mbar_init(&ctrl->full[s], 1);
            mbar_init(&ctrl->empty[s], CWARPS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctrl->pfull[b], 1);
            mbar_init(&ctrl->pempty[b], CWARPS);
        }
        ctrl->stop = 0; ctrl->consumed = 0; ctrl->pconsumed = 0; ctrl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the layer table is read from shared memory: its entries sit on every phase's critical path
    {
        const uint4* src = (const uint4*)p.layers;
        uint4* dst = (uint4*)(smem + OFF_LAYERS);
        const int words = p.L * (int)(sizeof(MegaLayer) / 16);
        for (int i = threadIdx.x; i < words; i += blockDim.x) dst[i] = src[i];
    }
    if (threadIdx.x < W_KINDS) {
        const int kind = threadIdx.x, d = p.d, F = p.F;
        const int N = kind == W_QKV ? 3 * d : (kind == W_UP ? F : (kind == W_HEAD ? p.V : d));
        const int K = kind == W_DOWN ? F : d;
        make_work((Work*)(smem + OFF_WORK) + kind, N, K, (int)blockIdx.x, (int)gridDim.x);
    }
    if (threadIdx.x == W_KINDS) make_head_work((HeadWork*)(smem + OFF_WORK + W_KINDS * 32), p.V, p.d, (int)blockIdx.x, (int)gridDim.x);
    __syncthreads();
    Cta k{p, smem, ctrl, (const MegaLayer*)(smem + OFF_LAYERS), (const Work*)(smem + OFF_WORK), (const HeadWork*)(smem + OFF_WORK + W_KINDS * 32),
          (float4*)(smem + OFF_ACT), (float*)(smem + OFF_ACT),
          (float*)(smem + OFF_XS), (float*)(smem + OFF_ACT) + HEAD_SC_OFF, (float*)(smem + OFF_PSUM), (float*)(smem + OFF_RED),
          (int)blockIdx.x, (int)gridDim.x, (int)threadIdx.x, 0, 0, 0u, -1};
    if (threadIdx.x >= CONSUMERS) {
        if (threadIdx.x == CONSUMERS) producer(k);
        __syncwarp();
    } else {
        consumer(k);
        consumer_sync();
        if (threadIdx.x == 0) { ctrl->consumed = k.item; ctrl->pconsumed = k.pitem; ctrl->stop = 1; }
    }
    __syncthreads();
    // drain: wait for bulk copies that were issued but never consumed before the CTA exits
    if (threadIdx.x == CONSUMERS) {
        for (int i = ctrl->consumed; i < k.item; ++i) {
            const long long t0 = clock64();
            while (!mbar_try_wait(&ctrl->full[i % SLOTS], (i / SLOTS) & 1))
                if (clock64() - t0 > p.wait_cycles) { atomicExch(p.status, FC_E_TIMEOUT); break; }
        }
        for (int i = ctrl->pconsumed; i < k.pitem; ++i) {
            const long long t0 = clock64();
            while (!mbar_try_wait(&ctrl->pfull[i & 1], (i >> 1) & 1))
                if (clock64() - t0 > p.wait_cycles) { atomicExch(p.status, FC_E_TIMEOUT); break; }
        }
    }
}

size_t mega_smem_bytes() { return SMEM_BYTES; }
int mega_head_rows_max() { return MAX_ROWS_HEAD; }
int mega_threads() { return THREADS; }

int mega_supported(const fc_config& c) {
    const int hd = c.d_model / c.n_head;
    return c.d_model <= MAX_D && c.d_ff <= MAX_F && c.ctx <= MAX_CTX && hd <= 64 && c.d_model <= 2 * CONSUMERS &&
           c.n_layer <= kMegaMaxLayers;
}

int launch_decode_mega(const MegaParams& p, int grid, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        FC_CUDA(cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set[dev] = true;
    }
    FC_CUDA(cudaMemsetAsync(p.bar, 0, sizeof(unsigned), st));
    void* args[] = {(void*)&p};
    FC_CUDA(cudaLaunchCooperativeKernel((void*)decode_mega_kernel, dim3(grid), dim3(THREADS), args, SMEM_BYTES, st));
    ++g_launches;
    return FC_OK;
}

int mega_max_grid(int* grid) {
    int dev = 0, sms = 0, per_sm = 0;
    FC_CUDA(cudaGetDevice(&dev));
    FC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    FC_CUDA(cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    FC_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel, THREADS, SMEM_BYTES));
    if (per_sm < 1) return fail(FC_E_CUDA, "the persistent decode kernel does not fit on an SM");
    *grid = sms < CONSUMERS ? sms : CONSUMERS;
    return FC_OK;
}

// ------------------------------------------------------------------ tile-major weight copy
// One thread per (tile, row): 32 quants (bias of 128 removed) and the row's f16 scale.
__global__ void repack_tiles_kernel(const uint8_t* __restrict__ qu, const __half* __restrict__ d,
                                    unsigned char* __restrict__ out, int N_pad, int K) {
    const int KB = K >> 5;
    const size_t total = (size_t)(N_pad / kMegaStripRows) * KB * kMegaStripRows;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int g = (int)(i & 7);
        const size_t tile = i >> 3, strip = tile / KB;
        const int kb = (int)(tile - strip * KB);
        const size_t row = strip * kMegaStripRows + g;
        const uint4* src = (const uint4*)(qu + row * K + (size_t)kb * 32);
        uint4 a = src[0], b = src[1];
        a.x ^= 0x80808080u; a.y ^= 0x80808080u; a.z ^= 0x80808080u; a.w ^= 0x80808080u;
        b.x ^= 0x80808080u; b.y ^= 0x80808080u; b.z ^= 0x80808080u; b.w ^= 0x80808080u;
        unsigned char* t = out + tile * kMegaTileBytes;
        ((uint4*)(t + g * 32))[0] = a;
        ((uint4*)(t + g * 32))[1] = b;
        ((__half*)(t + 256))[g] = d[row * KB + kb];
    }
}

int launch_repack_tiles(const QMat& w, unsigned char* out, cudaStream_t st) {
    if (w.N_pad % kMegaStripRows) return fail(FC_E_SHAPE, "padded row count %d is not a multiple of %d", w.N_pad, kMegaStripRows);
    const size_t total = (size_t)w.N_pad * (w.K >> 5);
    const int threads = 256;
    const size_t want = (total + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    repack_tiles_kernel<<<blocks, threads, 0, st>>>(w.qu, w.d, out, w.N_pad, w.K);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
