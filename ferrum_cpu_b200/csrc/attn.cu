// Causal multi-head attention: the single-query KV-cached form used by decode, and the
// full-window form used by scoring/prefill. fp32 throughout; the T x T probability matrix
// the reference stores (transformer.rs:458-478 `last_attention`) is never materialised.
#include "fc_common.cuh"
#include "pdl.cuh"

namespace fc {

// --------------------------------------------------------------------------- decode form
// layer/transformer.rs:246-283 forward_with_cache, per head h: scores[j] = (q_h · k_h(j)) *
// 1/sqrt(hd) over the len cached rows, softmax (max, exp, sum), out_h = sum_j (e_j/sum) v_h(j).
// One block per query head. Cache rows are kvd floats apart; query head h reads key/value head
// h / group (grouped-query attention, llm.rs:305-341; group == 1 is the GPT-2 form).
__global__ void __launch_bounds__(256) attn_decode_kernel(const float* __restrict__ q, const float* __restrict__ kc,
                                                          const float* __restrict__ vc, int kvd, int group, int hd, int ctx,
                                                          const StepState* st, float* __restrict__ out) {
    extern __shared__ float sm[];   // scores[ctx] | q_h[hd] | red[64] | part[8][hd]
    pdl_trigger();
    pdl_wait();
    if (st->done | st->error) return;
    const int len = st->pos + 1;    // the new row was appended by the QKV GEMV
    const int h = blockIdx.x, hs = h * hd, ks = (h / group) * hd;
    float* sc = sm;
    float* qh = sm + ctx;
    float* red = qh + hd;
    float* part = red + 64;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int c = threadIdx.x; c < hd; c += blockDim.x) qh[c] = q[hs + c];
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)hd);
    // scores: one warp per cached row, lanes across the head dimension
    float mx = -INFINITY;
    for (int j = wid; j < len; j += nw) {
        const float* kr = kc + (size_t)j * kvd + ks;
        float dot = 0.0f;
        for (int c = lane; c < hd; c += 32) dot = fmaf(qh[c], kr[c], dot);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = dot * scale;
        if (lane == 0) sc[j] = s;
        mx = fmaxf(mx, s);
    }
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < nw; ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float s = 0.0f;
    for (int j = threadIdx.x; j < len; j += blockDim.x) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        s += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[32 + wid] = s;
    __syncthreads();
    float sum = 0.0f;
    for (int w = 0; w < nw; ++w) sum += red[32 + w];
    // out: thread (g, c) accumulates rows j = g, g+G, ... for dimension c, then the G
    // partials are added in a fixed order.
    const int G = blockDim.x / hd;   // hd <= blockDim.x
    const int g = threadIdx.x / hd, c = threadIdx.x - g * hd;
    if (g < G) {
        float acc = 0.0f;
        for (int j = g; j < len; j += G) acc = fmaf(sc[j] / sum, vc[(size_t)j * kvd + ks + c], acc);
        part[g * hd + c] = acc;
    }
    __syncthreads();
    if (threadIdx.x < hd) {
        float acc = 0.0f;
        for (int gg = 0; gg < G; ++gg) acc += part[gg * hd + threadIdx.x];
        out[hs + threadIdx.x] = acc;
    }
}

int launch_attn_decode_gqa(const float* q, const float* kcache, const float* vcache, int H, int KV, int hd, int ctx,
                           const StepState* state, float* out, cudaStream_t st) {
    if (hd > 256) return fail(FC_E_SHAPE, "head_dim %d exceeds 256", hd);
    const int threads = 256;
    const size_t smem = (size_t)(ctx + hd + 64 + (threads / hd) * hd) * sizeof(float);
    if (smem > 200 * 1024) return fail(FC_E_SHAPE, "context %d exceeds what the decode attention holds in shared memory", ctx);
    if (smem > 48 * 1024) FC_CUDA(cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    FC_CUDA(launch_pdl(attn_decode_kernel, dim3(H), dim3(threads), smem, st, q, kcache, vcache, KV * hd, H / KV, hd, ctx, state, out));
    ++g_launches;
    return FC_OK;
}

int launch_attn_decode(const float* q, const float* kcache, const float* vcache, int d, int H, int ctx,
                       const StepState* state, float* out, cudaStream_t st) {
    const int hd = d / H, threads = 256;
    if (hd > 256) return fail(FC_E_SHAPE, "head_dim %d exceeds 256", hd);
    const size_t smem = (size_t)(ctx + hd + 64 + (threads / hd) * hd) * sizeof(float);
    if (smem > 200 * 1024) return fail(FC_E_SHAPE, "context %d exceeds what the decode attention holds in shared memory", ctx);
    if (smem > 48 * 1024) FC_CUDA(cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attn_decode_kernel<<<H, threads, smem, st>>>(q, kcache, vcache, d, 1, hd, ctx, state, out);
    FC_LAUNCHED();
    return FC_OK;
}

// --------------------------------------------------------------------------- window form
// layer/transformer.rs:395-477 per (window b, head h): S = Q Kᵀ · 1/sqrt(hd), entries j > i
// masked (their softmax weight is exactly 0), row softmax, O = P V. Computed as an online
// softmax over key tiles: a block owns QT query rows; 4 threads share a query, each taking
// every 4th key of the tile for the scores and the P·V partial sums.
constexpr int QT = 64;   // query rows per block
constexpr int KT = 64;   // keys per tile
// Rows of q, k and v are ld floats apart (they may be slices of one fused buffer); query head
// h reads key/value head h / group; output rows are ldo floats apart.
template <int HD>
__global__ void __launch_bounds__(256) attn_prefill_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                           const float* __restrict__ v, int T, int ld, int group, int ldo,
                                                           float* __restrict__ out) {
    constexpr int LDS = HD + 4;                 // row stride in floats: 16-byte aligned, bank-shifted by 4
    extern __shared__ float4 sm4[];
    float* ks = (float*)sm4;                    // [KT][LDS]
    float* vs = ks + KT * LDS;                  // [KT][LDS]
    const int qt = (gridDim.x - 1) - blockIdx.x; // heavy (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int qi = threadIdx.x >> 2, part = threadIdx.x & 3;
    const int i = qt * QT + qi;                 // query row within the window
    const size_t row3 = (size_t)ld;
    const float* base = q + (size_t)b * T * row3 + (size_t)h * HD;
    const float* kbase = k + (size_t)b * T * row3 + (size_t)(h / group) * HD;
    const float* vbase = v + (size_t)b * T * row3 + (size_t)(h / group) * HD;
    const float scale = 1.0f / sqrtf((float)HD);

    float qreg[HD];
    if (i < T) {
        const float4* qp = (const float4*)(base + (size_t)i * row3);
#pragma unroll
        for (int c = 0; c < HD / 4; ++c) {
            const float4 t = qp[c];
            qreg[4 * c] = t.x; qreg[4 * c + 1] = t.y; qreg[4 * c + 2] = t.z; qreg[4 * c + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int c = 0; c < HD; ++c) qreg[c] = 0.0f;
    }
    float o[HD];
#pragma unroll
    for (int c = 0; c < HD; ++c) o[c] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    const int last_key = min(T, (qt + 1) * QT);          // keys needed by this query tile
    for (int k0 = 0; k0 < last_key; k0 += KT) {
        __syncthreads();
        // load K and V tiles (rows k0..k0+KT), zero beyond T
        for (int u = threadIdx.x; u < KT * (HD / 4); u += blockDim.x) {
            const int r = u / (HD / 4), c4 = u - r * (HD / 4);
            float4 kv = make_float4(0, 0, 0, 0), vv = kv;
            if (k0 + r < T) {
                kv = ((const float4*)(kbase + (size_t)(k0 + r) * row3))[c4];
                vv = ((const float4*)(vbase + (size_t)(k0 + r) * row3))[c4];
            }
            ((float4*)(ks + r * LDS))[c4] = kv;
            ((float4*)(vs + r * LDS))[c4] = vv;
        }
        __syncthreads();
        // scores for keys part, part+4, ...
        float s[KT / 4];
        float tmax = -INFINITY;
#pragma unroll
        for (int jj = 0; jj < KT / 4; ++jj) {
            const int jl = jj * 4 + part, j = k0 + jl;
            const float4* kr = (const float4*)(ks + jl * LDS);
            float dot = 0.0f;
#pragma unroll
            for (int c = 0; c < HD / 4; ++c) {
                const float4 kv = kr[c];
                dot = fmaf(qreg[4 * c], kv.x, dot); dot = fmaf(qreg[4 * c + 1], kv.y, dot);
                dot = fmaf(qreg[4 * c + 2], kv.z, dot); dot = fmaf(qreg[4 * c + 3], kv.w, dot);
            }
            s[jj] = (j <= i) ? dot * scale : -INFINITY;
            tmax = fmaxf(tmax, s[jj]);
        }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float mnew = fmaxf(m, tmax);
        if (mnew > -INFINITY) {                            // at least one visible key so far
            const float corr = expf(m - mnew);             // m == -inf -> 0
            l *= corr;
#pragma unroll
            for (int c = 0; c < HD; ++c) o[c] *= corr;
#pragma unroll
            for (int jj = 0; jj < KT / 4; ++jj) {
                const float p = expf(s[jj] - mnew);        // masked -> exp(-inf) = 0
                l += p;
                const float4* vr = (const float4*)(vs + (jj * 4 + part) * LDS);
#pragma unroll
                for (int c = 0; c < HD / 4; ++c) {
                    const float4 vv = vr[c];
                    o[4 * c] = fmaf(p, vv.x, o[4 * c]); o[4 * c + 1] = fmaf(p, vv.y, o[4 * c + 1]);
                    o[4 * c + 2] = fmaf(p, vv.z, o[4 * c + 2]); o[4 * c + 3] = fmaf(p, vv.w, o[4 * c + 3]);
                }
            }
            m = mnew;
        }
    }
    // combine the 4 partial sums of a query (same running max in all 4 lanes)
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
#pragma unroll
    for (int c = 0; c < HD; ++c) {
        float v = o[c];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        o[c] = v;
    }
    if (i < T) {
        float* op = out + ((size_t)b * T + i) * ldo + (size_t)h * HD;
        // lane `part` stores its quarter of the head dimension
#pragma unroll
        for (int c = 0; c < HD / 4; ++c)
            if ((c & 3) == part) ((float4*)op)[c] = make_float4(o[4 * c] / l, o[4 * c + 1] / l, o[4 * c + 2] / l, o[4 * c + 3] / l);
    }
}

// Any head width (a multiple of 4, at most 256): one warp per query row, lanes across the head
// dimension, keys read straight from global memory. Slower than the tiled kernel; used for the
// head widths that kernel is not instantiated for.
__global__ void __launch_bounds__(256) attn_prefill_any_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                               const float* __restrict__ v, int T, int ld, int group, int hd,
                                                               int ldo, float* __restrict__ out) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int i = (gridDim.x - 1 - blockIdx.x) * 8 + wid;      // late (long) rows first
    const int h = blockIdx.y, b = blockIdx.z;
    if (i >= T) return;
    const float* qr = q + ((size_t)b * T + i) * ld + (size_t)h * hd;
    const float* kb = k + (size_t)b * T * ld + (size_t)(h / group) * hd;
    const float* vb = v + (size_t)b * T * ld + (size_t)(h / group) * hd;
    const float scale = 1.0f / sqrtf((float)hd);
    float qv[8], o[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int c = lane + 32 * u;
        qv[u] = c < hd ? qr[c] : 0.0f;
        o[u] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int j = 0; j <= i; ++j) {
        const float* kr = kb + (size_t)j * ld;
        float dot = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = lane + 32 * u;
            if (c < hd) dot = fmaf(qv[u], kr[c], dot);
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
        const float sc = dot * scale;
        const float mnew = fmaxf(m, sc);
        const float corr = expf(m - mnew), p = expf(sc - mnew);
        l = l * corr + p;
        const float* vr = vb + (size_t)j * ld;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = lane + 32 * u;
            if (c < hd) o[u] = fmaf(p, vr[c], o[u] * corr);
        }
        m = mnew;
    }
    float* op = out + ((size_t)b * T + i) * ldo + (size_t)h * hd;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int c = lane + 32 * u;
        if (c < hd) op[c] = o[u] / l;
    }
}

int launch_attn_prefill_gqa(const float* q, const float* k, const float* v, int B, int T, int ld, int H, int KV, int hd,
                            int ldo, float* out, cudaStream_t st) {
    if (KV <= 0 || H % KV) return fail(FC_E_DIM, "n_heads %d must be a multiple of n_kv_heads %d", H, KV);
    const int group = H / KV;
    dim3 grid((T + QT - 1) / QT, H, B);
    const bool aligned = ((ld | ldo) & 3) == 0 && ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)out)) & 15) == 0;
    if (hd == 64 && aligned) {
        const size_t smem = (size_t)2 * KT * (64 + 4) * sizeof(float);
        attn_prefill_kernel<64><<<grid, 256, smem, st>>>(q, k, v, T, ld, group, ldo, out);
    } else if (hd == 32 && aligned) {
        const size_t smem = (size_t)2 * KT * (32 + 4) * sizeof(float);
        attn_prefill_kernel<32><<<grid, 256, smem, st>>>(q, k, v, T, ld, group, ldo, out);
    } else if (hd <= 256) {
        dim3 g2((T + 7) / 8, H, B);
        attn_prefill_any_kernel<<<g2, 256, 0, st>>>(q, k, v, T, ld, group, hd, ldo, out);
    } else {
        return fail(FC_E_SHAPE, "window attention supports head_dim up to 256, got %d", hd);
    }
    FC_LAUNCHED();
    return FC_OK;
}

int launch_attn_prefill(const float* qkv, int B, int T, int d, int H, float* out, cudaStream_t st) {
    return launch_attn_prefill_gqa(qkv, qkv + d, qkv + 2 * d, B, T, 3 * d, H, H, d / H, d, out, st);
}

}  // namespace fc
