// Row kernels of the imported Llama / Qwen decoder (ferrum_core/src/llm.rs): token lookup,
// RMSNorm, rotary positions, the SwiGLU gate, the exact log-softmax scoring tail of
// llm_score.rs and the greedy pick. All are HBM-bound elementwise / row-reduction work: one
// block per row, coalesced accesses, fixed-order block reductions.
#include <cuda_bf16.h>

#include "llama_ops.cuh"
#include "pdl.cuh"

namespace fc {

namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Fixed-order block reductions; `red` holds 33 values.
template <class T>
__device__ T block_sum_t(T v, T* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if constexpr (sizeof(T) == 8) v = warp_sum_d(v); else v = warp_sum_f(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        T t = lane < nw ? red[lane] : (T)0;
        if constexpr (sizeof(T) == 8) t = warp_sum_d(t); else t = warp_sum_f(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// Value c of row `id` of a Q8_0 table: d * q, the single rounding of gguf::dequant_q8_0
// (gguf/dequant.rs:37-49).
__device__ __forceinline__ float table_value(const QMat& tok, int id, int c) {
    const float dq = __half2float(tok.d[(size_t)id * (tok.K >> 5) + (c >> 5)]);
    const int q = (int)tok.qu[(size_t)id * tok.K + c] - 128;
    return dq * (float)q;
}

}  // namespace

// ------------------------------------------------------------------------------ embedding
// LlamaModel::embed (llm.rs:588-597): the token's row, no position term. A bad id is an error
// flag, never a trap.
__global__ void llama_embed_rows_kernel(QMat tok, const int* __restrict__ ids, float* __restrict__ x, int* error_flag) {
    const int r = blockIdx.x;
    int id = ids[r];
    if (id < 0 || id >= tok.N) {
        if (threadIdx.x == 0) atomicExch(error_flag, FC_E_DIM);
        id = 0;
    }
    for (int c = threadIdx.x; c < tok.K; c += blockDim.x) x[(size_t)r * tok.K + c] = table_value(tok, id, c);
}
int launch_llama_embed_rows(const QMat& tok, const int* ids, int R, float* x, int* error_flag, cudaStream_t st) {
    llama_embed_rows_kernel<<<R, 256, 0, st>>>(tok, ids, x, error_flag);
    FC_LAUNCHED();
    return FC_OK;
}

// forward_one (llm.rs:610-618): the queued token at the cache position. A full context is
// refused like a bad id (generation stops at the window, llm.rs:720-730).
__global__ void llama_embed_step_kernel(QMat tok, int ctx, const int* __restrict__ queue, StepState* st, float* __restrict__ x) {
    pdl_trigger();
    pdl_wait();
    if (st->done | st->error) return;
    const int pos = st->pos, id = queue[st->fed];
    if (id < 0 || id >= tok.N || pos >= ctx) {
        __syncthreads();
        if (threadIdx.x == 0) st->error = FC_E_DIM;
        return;
    }
    for (int c = threadIdx.x; c < tok.K; c += blockDim.x) x[c] = table_value(tok, id, c);
}
int launch_llama_embed_step(const QMat& tok, int ctx, const int* queue, StepState* state, float* x, cudaStream_t st) {
    FC_CUDA(launch_pdl(llama_embed_step_kernel, dim3(1), dim3(256), 0, st, tok, ctx, queue, state, x));
    ++g_launches;
    return FC_OK;
}

// -------------------------------------------------------------------------------- RMSNorm
// RmsNorm::forward_row (llm.rs:57-64): ms = sum(x^2) / d, inv = 1 / sqrt(ms + eps),
// y = (x * inv) * w. The sum is a block tree, not the reference's ascending order.
__global__ void __launch_bounds__(256) llama_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                            int d, float* __restrict__ y, const StepState* st) {
    __shared__ float red[33];
    if (st && (st->done | st->error)) return;
    const float* xr = x + (size_t)blockIdx.x * d;
    float s = 0.0f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = xr[c]; s = fmaf(v, v, s); }
    const float ms = block_sum_t(s, red) / (float)d;
    const float inv = 1.0f / sqrtf(ms + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) y[(size_t)blockIdx.x * d + c] = __fmul_rn(__fmul_rn(xr[c], inv), w[c]);
}
// The same with the result written as the bf16 hi / lo planes (y = hi + lo to 2^-17 relative)
// that the tensor-core GEMM reads.
__device__ __forceinline__ void store_planes(float y, __nv_bfloat16* hi, __nv_bfloat16* lo, size_t i) {
    const __nv_bfloat16 h = __float2bfloat16_rn(y);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(y - __bfloat162float(h));
}
__global__ void __launch_bounds__(256) llama_rmsnorm_planes_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps,
                                                                   int d, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    __shared__ float red[33];
    const float* xr = x + (size_t)blockIdx.x * d;
    float s = 0.0f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) { const float v = xr[c]; s = fmaf(v, v, s); }
    const float ms = block_sum_t(s, red) / (float)d;
    const float inv = 1.0f / sqrtf(ms + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) store_planes(__fmul_rn(__fmul_rn(xr[c], inv), w[c]), hi, lo, (size_t)blockIdx.x * d + c);
}
int launch_llama_rmsnorm_planes(const float* x, const float* w, float eps, int rows, int d, void* hi, void* lo, cudaStream_t st) {
    llama_rmsnorm_planes_kernel<<<rows, 256, 0, st>>>(x, w, eps, d, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_llama_rmsnorm(const float* x, const float* w, float eps, int rows, int d, float* y, const StepState* state,
                         cudaStream_t st) {
    llama_rmsnorm_kernel<<<rows, 256, 0, st>>>(x, w, eps, d, y, state);
    FC_LAUNCHED();
    return FC_OK;
}

// ----------------------------------------------------------------------------------- RoPE
// apply_rope (llm.rs:158-185) with RopeScaling::angle (llm.rs:129-132): pair i of a head turns
// by theta = ((pos * freq_i) / ff_i) * (1 / linear_factor), freq_i = (f32) base^(-2i/rope_dim)
// computed in f64 on the host. Multiplies and adds are rounded separately, as the reference's.
__device__ __forceinline__ void rotate_pair(float* x, int ia, int ib, float theta) {
    float s, c;
    sincosf(theta, &s, &c);
    const float a = x[ia], b = x[ib];
    x[ia] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
    x[ib] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
}
__device__ __forceinline__ float rope_angle(int pos, float2 f, float inv_linear) {
    return __fmul_rn(__fdiv_rn(__fmul_rn((float)pos, f.x), f.y), inv_linear);
}

// Window form: row r of the fused [R][ld] buffer sits at position r % T; its first n_q heads
// (queries) and the n_kv heads that follow them at `k_off` are rotated in place.
__global__ void llama_rope_rows_kernel(float* __restrict__ qkv, int ld, int T, int n_q, int n_kv, int k_off, int hd, int half,
                                       int neox, const float2* __restrict__ ftab, float inv_linear) {
    const int r = blockIdx.x, pos = r % T;
    float* row = qkv + (size_t)r * ld;
    const int pairs = (n_q + n_kv) * half;
    for (int u = threadIdx.x; u < pairs; u += blockDim.x) {
        const int h = u / half, i = u - h * half;
        const int off = h < n_q ? h * hd : k_off + (h - n_q) * hd;
        const int ia = neox ? off + i : off + 2 * i, ib = neox ? off + i + half : off + 2 * i + 1;
        rotate_pair(row, ia, ib, rope_angle(pos, ftab[i], inv_linear));
    }
}
// The same rotation with the row handed on as bf16 hi / lo planes (the input of the tensor-core
// attention): the f32 row is staged in shared memory, rotated there and written once.
__global__ void llama_rope_planes_kernel(const float* __restrict__ qkv, int ld, int T, int n_q, int n_kv, int k_off, int hd, int half,
                                         int neox, const float2* __restrict__ ftab, float inv_linear,
                                         __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    extern __shared__ float srow[];
    const int r = blockIdx.x, pos = r % T;
    const float* row = qkv + (size_t)r * ld;
    for (int c = threadIdx.x; c < ld; c += blockDim.x) srow[c] = row[c];
    __syncthreads();
    const int pairs = (n_q + n_kv) * half;
    for (int u = threadIdx.x; u < pairs; u += blockDim.x) {
        const int h = u / half, i = u - h * half;
        const int off = h < n_q ? h * hd : k_off + (h - n_q) * hd;
        const int ia = neox ? off + i : off + 2 * i, ib = neox ? off + i + half : off + 2 * i + 1;
        rotate_pair(srow, ia, ib, rope_angle(pos, ftab[i], inv_linear));
    }
    __syncthreads();
    for (int c = threadIdx.x; c < ld; c += blockDim.x) store_planes(srow[c], hi, lo, (size_t)r * ld + c);
}
int launch_llama_rope_planes(const float* qkv, int R, int ld, int T, int n_q, int n_kv, int k_off, int hd, int rope_dim, int neox,
                             const float2* ftab, float inv_linear, void* hi, void* lo, cudaStream_t st) {
    const size_t smem = (size_t)ld * sizeof(float);
    if (smem > 48 * 1024) return fail(FC_E_SHAPE, "fused q | k | v rows of %d floats exceed the rotation kernel's staging", ld);
    llama_rope_planes_kernel<<<R, 256, smem, st>>>(qkv, ld, T, n_q, n_kv, k_off, hd, rope_dim / 2, neox, ftab, inv_linear,
                                                   (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_llama_rope_rows(float* qkv, int R, int ld, int T, int n_q, int n_kv, int k_off, int hd, int rope_dim, int neox,
                           const float2* ftab, float inv_linear, cudaStream_t st) {
    llama_rope_rows_kernel<<<R, 256, 0, st>>>(qkv, ld, T, n_q, n_kv, k_off, hd, rope_dim / 2, neox, ftab, inv_linear);
    FC_LAUNCHED();
    return FC_OK;
}

// Batched prime: the rotated key rows and the value rows of a window forward become the first R
// cache rows of a layer (what R calls of forward_one would have appended, llm.rs:349-350).
__global__ void llama_store_kv_rows_kernel(const float* __restrict__ qkv, int ld, int q_dim, int kv_dim, float* __restrict__ kc,
                                           float* __restrict__ vc) {
    const float* row = qkv + (size_t)blockIdx.x * ld + q_dim;
    for (int c = threadIdx.x; c < kv_dim; c += blockDim.x) {
        kc[(size_t)blockIdx.x * kv_dim + c] = row[c];
        vc[(size_t)blockIdx.x * kv_dim + c] = row[kv_dim + c];
    }
}
int launch_llama_store_kv_rows(const float* qkv, int R, int ld, int q_dim, int kv_dim, float* kc, float* vc, cudaStream_t st) {
    llama_store_kv_rows_kernel<<<R, 256, 0, st>>>(qkv, ld, q_dim, kv_dim, kc, vc);
    FC_LAUNCHED();
    return FC_OK;
}

// Decode attention with the rotation folded in (Attention::project + forward_one + attend,
// llm.rs:276-358): one block per query head. The block rotates its query head and the key head
// of its group for the current position into shared memory, the first head of a group appends
// the rotated key and the value row to the caches, and the scores run over the cached rows plus
// that new row — so no other block's write is ever read.
__global__ void __launch_bounds__(512) llama_attn_decode_kernel(const float* __restrict__ qkv, int n_q, int n_kv, int hd, int half,
                                                                int neox, const float2* __restrict__ ftab, float inv_linear,
                                                                float* __restrict__ kc, float* __restrict__ vc, int ctx,
                                                                const StepState* st, float* __restrict__ out) {
    extern __shared__ float sm[];   // scores[ctx] | q[hd] | k[hd] | v[hd] | red[64] | part[(threads / hd) * hd]
    pdl_trigger();
    pdl_wait();
    if (st->done | st->error) return;
    const int pos = st->pos, len = pos + 1, kv_dim = n_kv * hd, q_dim = n_q * hd;
    const int h = blockIdx.x, group = n_q / n_kv, kvh = h / group;
    float* sc = sm;
    float* qh = sm + ((ctx + 3) & ~3);      // 16-byte aligned: read as float4
    float* kh = qh + hd;
    float* vh = kh + hd;
    float* red = vh + hd;
    float* part = red + 64;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
    const float* qsrc = qkv + (size_t)h * hd;
    const float* ksrc = qkv + q_dim + (size_t)kvh * hd;
    const float* vsrc = qkv + q_dim + kv_dim + (size_t)kvh * hd;
    // threads 0..hd-1 build q, hd..2hd-1 build k (rotated pairs, then the unrotated tail)
    for (int u = tid; u < 2 * hd; u += blockDim.x) {
        const bool is_k = u >= hd;
        const int t = is_k ? u - hd : u;
        const float* src = is_k ? ksrc : qsrc;
        float* dst = is_k ? kh : qh;
        if (t < half) {
            const int ia = neox ? t : 2 * t, ib = neox ? t + half : 2 * t + 1;
            float s, c;
            sincosf(rope_angle(pos, ftab[t], inv_linear), &s, &c);
            const float a = src[ia], b = src[ib];
            dst[ia] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            dst[ib] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
        } else if (t >= 2 * half) {
            dst[t] = src[t];
        }
    }
    for (int c = tid; c < hd; c += blockDim.x) vh[c] = vsrc[c];
    __syncthreads();
    float* krow = kc + (size_t)pos * kv_dim + (size_t)kvh * hd;
    float* vrow = vc + (size_t)pos * kv_dim + (size_t)kvh * hd;
    if (h == kvh * group)
        for (int c = tid; c < hd; c += blockDim.x) { krow[c] = kh[c]; vrow[c] = vh[c]; }
    const float scale = 1.0f / sqrtf((float)hd);
    // scores: one half warp per row, float4 per lane
    const int hw = tid >> 4, hl = tid & 15, nhw = blockDim.x >> 4;
    const unsigned hmask = 0xFFFFu << (tid & 16);
    float mx = -INFINITY;
    // two rows per half warp and sweep: their loads are requested together
    for (int j = hw; j < len; j += 2 * nhw) {
        const int j2 = j + nhw;
        const bool has2 = j2 < len;
        const float4* kr = j == pos ? (const float4*)kh : (const float4*)(kc + (size_t)j * kv_dim + (size_t)kvh * hd);
        const float4* kr2 = !has2 ? kr : (j2 == pos ? (const float4*)kh : (const float4*)(kc + (size_t)j2 * kv_dim + (size_t)kvh * hd));
        float dot = 0.0f, dot2 = 0.0f;
        for (int c4 = hl; c4 < (hd >> 2); c4 += 16) {
            const float4 kv = kr[c4], kv2 = kr2[c4], qv = ((const float4*)qh)[c4];
            dot = fmaf(qv.x, kv.x, dot); dot = fmaf(qv.y, kv.y, dot); dot = fmaf(qv.z, kv.z, dot); dot = fmaf(qv.w, kv.w, dot);
            dot2 = fmaf(qv.x, kv2.x, dot2); dot2 = fmaf(qv.y, kv2.y, dot2); dot2 = fmaf(qv.z, kv2.z, dot2); dot2 = fmaf(qv.w, kv2.w, dot2);
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            dot += __shfl_xor_sync(hmask, dot, o);
            dot2 += __shfl_xor_sync(hmask, dot2, o);
        }
        const float s = dot * scale, s2 = dot2 * scale;
        if (hl == 0) { sc[j] = s; if (has2) sc[j2] = s2; }
        mx = fmaxf(mx, s);
        if (has2) mx = fmaxf(mx, s2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < nw; ++w) mx = fmaxf(mx, red[w]);
    float s = 0.0f;
    for (int j = tid; j < len; j += blockDim.x) {
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
    // out: thread (g, c) accumulates rows j = g, g + G, ... for dimension c; partials added in order
    const int G = blockDim.x / hd;
    const int g = tid / hd, c = tid - g * hd;
    if (g < G) {
        // four rows in flight per thread; the four partial sums are added in a fixed order
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        const float* vbase = vc + (size_t)kvh * hd + c;
        int j = g;
        for (; j + 3 * G < len; j += 4 * G) {
            const int j1 = j + G, j2 = j + 2 * G, j3 = j + 3 * G;
            const float v0 = j == pos ? vh[c] : vbase[(size_t)j * kv_dim], v1 = j1 == pos ? vh[c] : vbase[(size_t)j1 * kv_dim];
            const float v2 = j2 == pos ? vh[c] : vbase[(size_t)j2 * kv_dim], v3 = j3 == pos ? vh[c] : vbase[(size_t)j3 * kv_dim];
            a0 = fmaf(sc[j] / sum, v0, a0); a1 = fmaf(sc[j1] / sum, v1, a1);
            a2 = fmaf(sc[j2] / sum, v2, a2); a3 = fmaf(sc[j3] / sum, v3, a3);
        }
        for (; j < len; j += G) a0 = fmaf(sc[j] / sum, j == pos ? vh[c] : vbase[(size_t)j * kv_dim], a0);
        part[g * hd + c] = (a0 + a1) + (a2 + a3);
    }
    __syncthreads();
    if (tid < hd) {
        float acc = 0.0f;
        for (int gg = 0; gg < G; ++gg) acc += part[gg * hd + tid];
        out[(size_t)h * hd + tid] = acc;
    }
}
int launch_llama_attn_decode(const float* qkv, int n_q, int n_kv, int hd, int rope_dim, int neox, const float2* ftab, float inv_linear,
                             float* kc, float* vc, int ctx, const StepState* state, float* out, cudaStream_t st) {
    if (hd > 256 || hd % 4) return fail(FC_E_SHAPE, "head_dim %d must be a multiple of 4, at most 256", hd);
    const int threads = 512;
    const size_t smem = (size_t)(((ctx + 3) & ~3) + 3 * hd + 64 + (threads / hd) * hd) * sizeof(float);
    if (smem > 200 * 1024) return fail(FC_E_SHAPE, "context %d exceeds what the decode attention holds in shared memory", ctx);
    if (smem > 48 * 1024) FC_CUDA(cudaFuncSetAttribute(llama_attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    FC_CUDA(launch_pdl(llama_attn_decode_kernel, dim3(n_q), dim3(threads), smem, st, qkv, n_q, n_kv, hd, rope_dim / 2, neox, ftab,
                       inv_linear, kc, vc, ctx, state, out));
    ++g_launches;
    return FC_OK;
}

// --------------------------------------------------------------------------------- SwiGLU
// FeedForward::forward (llm.rs:417-428): h = (g / (1 + exp(-g))) * u on rows of interleaved
// (gate_i, up_i) pairs, the row order of the fused gate/up matrix.
__global__ void llama_swiglu_kernel(const float* __restrict__ gu, int F, float* __restrict__ h, const StepState* st) {
    if (st && (st->done | st->error)) return;
    const float* row = gu + (size_t)blockIdx.y * 2 * F;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < F) {
        const float g = row[2 * c], u = row[2 * c + 1];
        h[(size_t)blockIdx.y * F + c] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
    }
}
int launch_llama_swiglu(const float* gu, int rows, int F, float* h, const StepState* state, cudaStream_t st) {
    dim3 grid((F + 255) / 256, rows);
    llama_swiglu_kernel<<<grid, 256, 0, st>>>(gu, F, h, state);
    FC_LAUNCHED();
    return FC_OK;
}

// --------------------------------------------------------------------------- scoring tail
// log_prob (llm_score.rs:35-39): ln softmax(row)[target] in f64 with no probability floor —
// max in f32, sum of exp((f64)x - max) in f64, x[target] - max - ln(sum); and
// argmax_first(row) == target (llm_score.rs:92). The f64 sum is a block tree.
__global__ void __launch_bounds__(512) llama_score_rows_kernel(const float* __restrict__ logits, int ldl, int V,
                                                               const int* __restrict__ targets, double* __restrict__ logprob,
                                                               uint8_t* __restrict__ is_greedy) {
    __shared__ double dred[33];
    __shared__ float fred[32];
    __shared__ int ired[32];
    const int r = blockIdx.x, target = targets[r];
    if (target < 0 || target >= V) {
        if (threadIdx.x == 0) { logprob[r] = 0.0; is_greedy[r] = 0; }
        return;
    }
    const float* row = logits + (size_t)r * ldl;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float mx = -INFINITY;
    int first = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > mx) { mx = v; first = i; }       // ascending i per thread: the first of a tie stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int of = __shfl_xor_sync(0xffffffffu, first, o);
        if (om > mx || (om == mx && of < first)) { mx = om; first = of; }
    }
    if (lane == 0) { fred[wid] = mx; ired[wid] = first; }
    __syncthreads();
    mx = fred[0]; first = ired[0];
    for (int w = 1; w < nw; ++w)
        if (fred[w] > mx || (fred[w] == mx && ired[w] < first)) { mx = fred[w]; first = ired[w]; }
    const double dmax = (double)mx;
    double s = 0.0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += exp((double)row[i] - dmax);
    const double sum = block_sum_t(s, dred);
    if (threadIdx.x == 0) {
        logprob[r] = (double)row[target] - dmax - log(sum);
        is_greedy[r] = (uint8_t)(first == target);
    }
}
int launch_llama_score_rows(const float* logits, int ldl, int V, const int* targets, int R, double* logprob, uint8_t* is_greedy,
                            cudaStream_t st) {
    llama_score_rows_kernel<<<R, 512, 0, st>>>(logits, ldl, V, targets, logprob, is_greedy);
    FC_LAUNCHED();
    return FC_OK;
}

// ---------------------------------------------------------------------------- greedy pick
// sample_with_params at temperature <= 0 with no repetition penalty is argmax_first of the raw
// logits (slm/sampling.rs:96-104,147): the id is appended to the queue for the next step.
__global__ void __launch_bounds__(1024) llama_pick_kernel(const float* __restrict__ logits, int V, int* __restrict__ queue,
                                                          int queue_cap, StepState* st) {
    __shared__ float fred[32];
    __shared__ int ired[32];
    pdl_trigger();
    pdl_wait();
    if (st->done | st->error) return;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float mx = -INFINITY;
    int first = 0x7fffffff;
    // eight loads in flight per thread: the row is 128 KB read by one block
    for (int i0 = threadIdx.x; i0 < V; i0 += 8 * blockDim.x) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = i < V ? logits[i] : -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
            if (v[u] > mx) { mx = v[u]; first = i0 + u * blockDim.x; }     // ascending i per thread: the first of a tie stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const int of = __shfl_xor_sync(0xffffffffu, first, o);
        if (om > mx || (om == mx && of < first)) { mx = om; first = of; }
    }
    if (lane == 0) { fred[wid] = mx; ired[wid] = first; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < nw; ++w)
            if (fred[w] > mx || (fred[w] == mx && ired[w] < first)) { mx = fred[w]; first = ired[w]; }
        if (first == 0x7fffffff) first = 0;      // all -inf / NaN: argmax_first answers 0
        if (st->tail < queue_cap) { queue[st->tail] = first; st->tail += 1; }
        else st->error = FC_E_DIM;
    }
}
int launch_llama_pick(const float* logits, int V, int* queue, int queue_cap, StepState* state, cudaStream_t st) {
    llama_pick_kernel<<<1, 1024, 0, st>>>(logits, V, queue, queue_cap, state);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
