// Row kernels of the forward path: embedding gather, LayerNorm, the decode tail
// (softmax statistics + greedy select) and the scoring tail (per-target log-prob).
#include <cuda_bf16.h>

#include <algorithm>

#include "fc_common.cuh"
#include "pdl.cuh"

namespace fc {

// ------------------------------------------------------------------------ block reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Fixed-order block reductions (deterministic run to run). `red` has >= 33 floats.
__device__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ------------------------------------------------------------------------------ embedding
// layer/embedding.rs:70-90 embed_one / :98-152 forward: x = tok[id] + pos[t]. The token
// table stays Q8_0; d * q is the same single rounding gguf::dequant_q8_0 performs.
__device__ __forceinline__ float tok_value(const QMat& tok, int id, int c) {
    const float dq = __half2float(tok.d[(size_t)id * (tok.K >> 5) + (c >> 5)]);
    const int q = (int)tok.qu[(size_t)id * tok.K + c] - 128;
    return dq * (float)q;
}

__global__ void embed_step_kernel(QMat tok, const float* __restrict__ pos_emb, int ctx,
                                  const int* __restrict__ queue, StepState* st, float* __restrict__ x) {
    if (st->done | st->error) return;
    const int pos = st->pos, id = queue[st->fed];
    // embedding.rs:71-82 and transformer.rs:237-242: bad id / full cache are errors, not traps
    if (id < 0 || id >= tok.N || pos >= ctx) {
        __syncthreads();
        if (threadIdx.x == 0) st->error = FC_E_DIM;
        return;
    }
    for (int c = threadIdx.x; c < tok.K; c += blockDim.x) x[c] = tok_value(tok, id, c) + pos_emb[(size_t)pos * tok.K + c];
}

int launch_embed_step(const QMat& tok, const float* pos_emb, int ctx, const int* queue, StepState* state,
                      float* x, cudaStream_t st) {
    embed_step_kernel<<<1, 256, 0, st>>>(tok, pos_emb, ctx, queue, state, x);
    FC_LAUNCHED();
    return FC_OK;
}

__global__ void embed_rows_kernel(QMat tok, const float* __restrict__ pos_emb, const int* __restrict__ ids,
                                  int T, float* __restrict__ x, int* error_flag) {
    const int r = blockIdx.x, t = r % T;
    int id = ids[r];
    if (id < 0 || id >= tok.N) {
        if (threadIdx.x == 0) atomicExch(error_flag, FC_E_DIM);
        id = 0;
    }
    for (int c = threadIdx.x; c < tok.K; c += blockDim.x)
        x[(size_t)r * tok.K + c] = tok_value(tok, id, c) + pos_emb[(size_t)t * tok.K + c];
}

int launch_embed_rows(const QMat& tok, const float* pos_emb, const int* ids, int R, int T, float* x,
                      int* error_flag, cudaStream_t st) {
    embed_rows_kernel<<<R, 256, 0, st>>>(tok, pos_emb, ids, T, x, error_flag);
    FC_LAUNCHED();
    return FC_OK;
}

// ------------------------------------------------------------------------------ LayerNorm
// layer/norm.rs:46-82: mean, then the variance of (x - mean), std = sqrt(var + 1e-5),
// y = ((x - mean) / std) * gamma + beta. One block per row; the row is held in registers.
template <int PER>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ b,
                                 int d, float* __restrict__ y, const StepState* st) {
    __shared__ float red[33];
    if (st && (st->done | st->error)) return;
    const float* xr = x + (size_t)blockIdx.x * d;
    float v[PER];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        v[i] = c < d ? xr[c] : 0.0f;
        s += v[i];
    }
    const float mean = block_sum(s, red) / (float)d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        const float t = v[i] - mean;
        q += c < d ? t * t : 0.0f;
    }
    const float var = block_sum(q, red) / (float)d;
    const float sd = sqrtf(var + 1e-5f);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < d) y[(size_t)blockIdx.x * d + c] = ((v[i] - mean) / sd) * g[c] + b[c];
    }
}

// The same LayerNorm with the result written as the bf16 hi / lo planes (y = hi + lo to 2^-17
// relative) that the tensor-core GEMM reads.
template <int PER>
__global__ void layernorm_planes_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ b,
                                        int d, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    __shared__ float red[33];
    const float* xr = x + (size_t)blockIdx.x * d;
    float v[PER];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        v[i] = c < d ? xr[c] : 0.0f;
        s += v[i];
    }
    const float mean = block_sum(s, red) / (float)d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        const float t = v[i] - mean;
        q += c < d ? t * t : 0.0f;
    }
    const float var = block_sum(q, red) / (float)d;
    const float sd = sqrtf(var + 1e-5f);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < d) {
            const float y = ((v[i] - mean) / sd) * g[c] + b[c];
            const __nv_bfloat16 h = __float2bfloat16_rn(y);
            hi[(size_t)blockIdx.x * d + c] = h;
            lo[(size_t)blockIdx.x * d + c] = __float2bfloat16_rn(y - __bfloat162float(h));
        }
    }
}

// The same for rows of up to 1024 columns (a multiple of 128): a warp per row, the row in registers as 16-byte loads,
// the two sums by shuffles (no block-wide synchronisation), the planes written 8 bytes per lane. Eight rows per CTA.
template <int NV>
__global__ void __launch_bounds__(256) layernorm_planes_warp_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                    const float* __restrict__ b, int rows, int d,
                                                                    __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int nv = d >> 7;                                  // 16-byte chunks per lane
    const float4* xr = (const float4*)(x + (size_t)row * d);
    float4 v[NV];
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        v[i] = i < nv ? xr[lane + 32 * i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / (float)d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            const float a = v[i].x - mean, c = v[i].y - mean, e = v[i].z - mean, f = v[i].w - mean;
            q += (a * a + c * c) + (e * e + f * f);
        }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float sd = sqrtf(q / (float)d + 1e-5f);
    const float4* g4 = (const float4*)g;
    const float4* b4 = (const float4*)b;
    uint2* h2 = (uint2*)(hi + (size_t)row * d);
    uint2* l2 = (uint2*)(lo + (size_t)row * d);
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (i < nv) {
            const float4 gg = __ldg(g4 + lane + 32 * i), bb = __ldg(b4 + lane + 32 * i);
            const float y[4] = {((v[i].x - mean) / sd) * gg.x + bb.x, ((v[i].y - mean) / sd) * gg.y + bb.y,
                                ((v[i].z - mean) / sd) * gg.z + bb.z, ((v[i].w - mean) / sd) * gg.w + bb.w};
            __nv_bfloat16 hh[4], ll[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                hh[k] = __float2bfloat16_rn(y[k]);
                ll[k] = __float2bfloat16_rn(y[k] - __bfloat162float(hh[k]));
            }
            h2[lane + 32 * i] = *(const uint2*)hh;
            l2[lane + 32 * i] = *(const uint2*)ll;
        }
}

int launch_layernorm_planes(const float* x, const float* g, const float* b, int rows, int d, void* hi, void* lo, cudaStream_t st) {
    if (d % 128 == 0 && d <= 1024 && aligned16(x) && aligned16(g) && aligned16(b) && aligned16(hi) && aligned16(lo)) {
        const int blocks = (rows + 7) / 8;
        if (d <= 512) layernorm_planes_warp_kernel<4><<<blocks, 256, 0, st>>>(x, g, b, rows, d, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
        else layernorm_planes_warp_kernel<8><<<blocks, 256, 0, st>>>(x, g, b, rows, d, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
        FC_LAUNCHED();
        return FC_OK;
    }
    const int threads = 256;
    const int per = (d + threads - 1) / threads;
    if (per <= 4) layernorm_planes_kernel<4><<<rows, threads, 0, st>>>(x, g, b, d, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    else if (per <= 8) layernorm_planes_kernel<8><<<rows, threads, 0, st>>>(x, g, b, d, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    else if (per <= 16) layernorm_planes_kernel<16><<<rows, threads, 0, st>>>(x, g, b, d, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    else return fail(FC_E_SHAPE, "LayerNorm width %d exceeds 4096", d);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_layernorm(const float* x, const float* g, const float* b, int rows, int d, float* y,
                     const StepState* state, cudaStream_t st) {
    const int threads = 256;
    const int per = (d + threads - 1) / threads;
    if (per <= 4) layernorm_kernel<4><<<rows, threads, 0, st>>>(x, g, b, d, y, state);
    else if (per <= 8) layernorm_kernel<8><<<rows, threads, 0, st>>>(x, g, b, d, y, state);
    else if (per <= 16) layernorm_kernel<16><<<rows, threads, 0, st>>>(x, g, b, d, y, state);
    else return fail(FC_E_SHAPE, "LayerNorm width %d exceeds 4096", d);
    FC_LAUNCHED();
    return FC_OK;
}

// ------------------------------------------------------------------------------ decode tail
// ops.rs:478-502 softmax_rows on one row, then (when selecting) token_stream.rs:134 +
// sampling.rs:96-104,147: logit_i = ln(max(p_i, 1e-12)), first index of the largest.
// One block. The sum runs in a fixed tree order, not the reference's ascending order.
struct ArgPair { float v; int i; };
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
    // larger value wins; equal values: smaller index (first on ties)
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__global__ void __launch_bounds__(1024) step_tail_kernel(const float* __restrict__ logits, int V, float* __restrict__ probs,
                                                         int do_select, int* __restrict__ queue, int queue_cap,
                                                         StepState* st, float* sel_logit) {
    __shared__ float red[33];
    __shared__ ArgPair pred[32];
    if (st->done | st->error) return;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, logits[i]);
    mx = block_max(mx, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(logits[i] - mx);
    const float sum = block_sum(s, red);
    if (probs)
        for (int i = threadIdx.x; i < V; i += blockDim.x) probs[i] = expf(logits[i] - mx) / sum;
    if (do_select) {
        ArgPair best{-INFINITY, 0x7fffffff};
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float p = expf(logits[i] - mx) / sum;
            best = better(best, ArgPair{logf(fmaxf(p, 1e-12f)), i});
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
            best = better(best, other);
        }
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        if (lane == 0) pred[wid] = best;
        __syncthreads();
        if (wid == 0) {
            best = lane < (int)((blockDim.x + 31) >> 5) ? pred[lane] : ArgPair{-INFINITY, 0x7fffffff};
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
                best = better(best, other);
            }
            if (lane == 0) {
                if (sel_logit) sel_logit[st->tail < queue_cap ? st->tail : queue_cap - 1] = best.v;
                if (best.i == st->eos) {
                    st->done = 1;
                } else if (st->tail < queue_cap) {
                    queue[st->tail] = best.i;
                    st->tail += 1;
                } else {
                    st->error = FC_E_DIM;
                }
            }
        }
    }
    if (threadIdx.x == 0) { st->pos += 1; st->fed += 1; }
}

int launch_step_tail(const float* logits, int V, float* probs_or_null, int do_select, int* queue, int queue_cap,
                     StepState* state, float* sel_logit_or_null, cudaStream_t st) {
    step_tail_kernel<<<1, 1024, 0, st>>>(logits, V, probs_or_null, do_select, queue, queue_cap, state, sel_logit_or_null);
    FC_LAUNCHED();
    return FC_OK;
}

__global__ void step_advance_kernel(StepState* st) {
    pdl_trigger();
    pdl_wait();
    if (st->done | st->error) return;
    st->pos += 1;
    st->fed += 1;
}
int launch_step_advance(StepState* state, cudaStream_t st) {
    step_advance_kernel<<<1, 1, 0, st>>>(state);
    FC_LAUNCHED();
    return FC_OK;
}
// The same as a programmatic dependent of the kernel ahead (steps whose kernels all wait first).
int launch_step_advance_pdl(StepState* state, cudaStream_t st) {
    FC_CUDA(launch_pdl(step_advance_kernel, dim3(1), dim3(1), 0, st, state));
    ++g_launches;
    return FC_OK;
}

// ------------------------------------------------------------------------------ scoring tail
// scoring.rs:175-181: p = softmax(row)[target] in f32, clamp_prob (loss.rs:12-18), ln in
// f64; greedy = argmax_first(row) == target, where the row is the probability row: the
// first index whose exp(x - max) / sum equals the largest such value.
__global__ void __launch_bounds__(256) score_rows_kernel(const float* __restrict__ logits, int ldl, int V,
                                                         const int* __restrict__ targets, double* __restrict__ logprob,
                                                         uint8_t* __restrict__ is_greedy) {
    __shared__ float red[33];
    __shared__ int ired[32];
    const int r = blockIdx.x, target = targets[r];
    if (target < 0 || target >= V) {
        if (threadIdx.x == 0) { logprob[r] = 0.0; is_greedy[r] = 0; }
        return;
    }
    const float* row = logits + (size_t)r * ldl;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float s = 0.0f;
    int first = 0x7fffffff;          // first index whose probability ties the maximum's
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float e = expf(row[i] - mx);
        s += e;
        if (e == 1.0f && i < first) first = i;
    }
    const float sum = block_sum(s, red);
    for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    if ((threadIdx.x & 31) == 0) ired[threadIdx.x >> 5] = first;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) first = min(first, ired[w]);
        float p = expf(row[target] - mx) / sum;
        if (p == p) p = fmaxf(p, 1e-12f);
        logprob[r] = log((double)p);
        is_greedy[r] = (uint8_t)(first == target);
    }
}

// The same tail with the row staged in shared memory: one CTA per SM walks rows, fetches a
// whole row of logits with one bulk async copy (a single pass over HBM, hundreds of KB in flight
// per SM) and makes its three passes (max, sum of exponentials + first maximal index, target)
// out of shared memory. Same arithmetic per row as score_rows_kernel with 1024 threads.
// Bound: HBM, 4 * ldl bytes per scored row.
constexpr int STAGED_THREADS = 1024;
constexpr long long STAGED_WAIT_CYCLES = 4000000000LL;
__global__ void __launch_bounds__(STAGED_THREADS, 1)
score_rows_staged_kernel(const float* __restrict__ logits, int ldl, int V, const int* __restrict__ targets, int R,
                         double* __restrict__ logprob, uint8_t* __restrict__ is_greedy, int* status) {
    extern __shared__ __align__(16) float srow[];
    __shared__ float red[33];
    __shared__ int ired[32];
    __shared__ unsigned long long bar;
    const uint32_t bar_a = (uint32_t)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_a) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t bytes = (uint32_t)ldl * 4u;
    uint32_t copies = 0;                                   // bulk copies issued so far (phase parity)
    for (int r = blockIdx.x; r < R; r += gridDim.x) {
        const int target = targets[r];
        if (target < 0 || target >= V) {
            if (threadIdx.x == 0) { logprob[r] = 0.0; is_greedy[r] = 0; }
            continue;
        }
        bool failed = false;
        if (threadIdx.x == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_a), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"((uint32_t)__cvta_generic_to_shared(srow)), "l"(logits + (size_t)r * ldl), "r"(bytes), "r"(bar_a) : "memory");
            const long long t0 = clock64();
            for (;;) {
                uint32_t ok;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}"
                    : "=r"(ok) : "r"(bar_a), "r"(copies & 1u), "r"(2000u) : "memory");
                if (ok) break;
                if (clock64() - t0 > STAGED_WAIT_CYCLES) { failed = true; break; }
            }
        }
        ++copies;
        if (__syncthreads_or(failed)) {                      // the row never arrived: report and stop
            if (threadIdx.x == 0) atomicExch(status, FC_E_TIMEOUT);
            break;
        }
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < V; i += STAGED_THREADS) mx = fmaxf(mx, srow[i]);
        mx = block_max(mx, red);
        float s = 0.0f;
        int first = 0x7fffffff;          // first index whose probability ties the maximum's
        for (int i = threadIdx.x; i < V; i += STAGED_THREADS) {
            const float e = expf(srow[i] - mx);
            s += e;
            if (e == 1.0f && i < first) first = i;
        }
        const float sum = block_sum(s, red);
        for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
        if ((threadIdx.x & 31) == 0) ired[threadIdx.x >> 5] = first;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < STAGED_THREADS / 32; ++w) first = min(first, ired[w]);
            float p = expf(srow[target] - mx) / sum;
            if (p == p) p = fmaxf(p, 1e-12f);
            logprob[r] = log((double)p);
            is_greedy[r] = (uint8_t)(first == target);
        }
        __syncthreads();                                     // the row buffer is free for the next copy
    }
}

int launch_score_rows(const float* logits, int ldl, int V, const int* targets, int R, double* logprob,
                      uint8_t* is_greedy, int* status, cudaStream_t st) {
    static int sms[64] = {};
    const size_t smem = (size_t)ldl * 4;
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    // rows staged in shared memory when a row fits and the copy is legal (16-byte multiples)
    if (status && dev < 64 && smem <= 200 * 1024 && (ldl & 3) == 0 && (((uintptr_t)logits) & 15) == 0 && R > 0) {
        if (!sms[dev]) {
            FC_CUDA(cudaFuncSetAttribute(score_rows_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            FC_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
        }
        score_rows_staged_kernel<<<R < sms[dev] ? R : sms[dev], STAGED_THREADS, smem, st>>>(logits, ldl, V, targets, R, logprob, is_greedy, status);
        FC_LAUNCHED();
        return FC_OK;
    }
    score_rows_kernel<<<R, 256, 0, st>>>(logits, ldl, V, targets, logprob, is_greedy);
    FC_LAUNCHED();
    return FC_OK;
}

__global__ void __launch_bounds__(1024) softmax_row_kernel(const float* __restrict__ logits, int V, float* __restrict__ probs) {
    __shared__ float red[33];
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, logits[i]);
    mx = block_max(mx, red);
    float s = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) s += expf(logits[i] - mx);
    const float sum = block_sum(s, red);
    for (int i = threadIdx.x; i < V; i += blockDim.x) probs[i] = expf(logits[i] - mx) / sum;
}
int launch_softmax_row(const float* logits, int V, float* probs, cudaStream_t st) {
    softmax_row_kernel<<<1, 1024, 0, st>>>(logits, V, probs);
    FC_LAUNCHED();
    return FC_OK;
}

// ------------------------------------------------------------------------------ layer statistics
// verbose::stats + verbose::check_nan_inf (verbose.rs:85-110) of one layer output: min, max, f64 sum, and the
// counts of NaN and Inf. Two stages with a fixed order (per-block partials, then one block), so the figures are
// the same from run to run. planes_lo != null: the tensor is held as bf16 hi / lo planes, value = hi + lo.
struct StatPart { float mn, mx; double sum; unsigned long long nan, inf; };

__global__ void __launch_bounds__(256) layer_stats_partial_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ hi,
                                                                  const __nv_bfloat16* __restrict__ lo, size_t n, StatPart* part) {
    __shared__ StatPart sh[256];
    StatPart p{INFINITY, -INFINITY, 0.0, 0ull, 0ull};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x ? x[i] : __bfloat162float(hi[i]) + __bfloat162float(lo[i]);
        if (v != v) { p.nan += 1; continue; }      // as the reference's comparisons, NaN never becomes min or max
        if (isinf(v)) p.inf += 1;
        p.mn = fminf(p.mn, v);
        p.mx = fmaxf(p.mx, v);
        p.sum += (double)v;
    }
    sh[threadIdx.x] = p;
    __syncthreads();
    if (threadIdx.x == 0) {
        StatPart t = sh[0];
        for (int i = 1; i < (int)blockDim.x; ++i) {
            t.mn = fminf(t.mn, sh[i].mn); t.mx = fmaxf(t.mx, sh[i].mx); t.sum += sh[i].sum; t.nan += sh[i].nan; t.inf += sh[i].inf;
        }
        part[blockIdx.x] = t;
    }
}

__global__ void layer_stats_final_kernel(const StatPart* part, int n_part, size_t n, LayerStatsDev* out) {
    StatPart t = part[0];
    for (int i = 1; i < n_part; ++i) {
        t.mn = fminf(t.mn, part[i].mn); t.mx = fmaxf(t.mx, part[i].mx); t.sum += part[i].sum; t.nan += part[i].nan; t.inf += part[i].inf;
    }
    out->min = n ? t.mn : 0.0f;
    out->max = n ? t.mx : 0.0f;
    out->mean = n ? (float)(t.sum / (double)n) : 0.0f;
    out->nan_count = (long long)t.nan;
    out->inf_count = (long long)t.inf;
    out->n = (long long)n;
}

size_t layer_stats_scratch_bytes() { return 148 * sizeof(StatPart); }

int launch_layer_stats(const float* x, const void* hi, const void* lo, size_t n, void* scratch, LayerStatsDev* out, cudaStream_t st) {
    const int blocks = (int)std::min<size_t>(148, std::max<size_t>(1, (n + 255) / 256));
    layer_stats_partial_kernel<<<blocks, 256, 0, st>>>(x, (const __nv_bfloat16*)hi, (const __nv_bfloat16*)lo, n, (StatPart*)scratch);
    FC_LAUNCHED();
    layer_stats_final_kernel<<<1, 1, 0, st>>>((const StatPart*)scratch, blocks, n, out);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
