// Q8_0 dequant-GEMV for one activation row (batch-1 decode), and the upload-time repack
// of GGML Q8_0 blocks into the two device planes.
//
// Replaces, for M == 1, ops::linear_forward -> matmul_rows -> matmul_block
// (ferrum_core/src/ops.rs:29-55,159-177,233-256) on a weight that the reference would have
// expanded to f32 with gguf::dequant_q8_0 (ferrum_core/src/gguf/dequant.rs:37-49):
//     y[n] = sum_kb d[n][kb] * sum_{j<32} x[32 kb + j] * q[n][32 kb + j]  + bias[n]
// fp32 FMA on CUDA cores; the f16 scale is applied once per 16 quants in registers.
//
// Bound: HBM. Algorithmic bytes per call = N*K*34/32 (weights) + 4K + 4N.
#include "fc_common.cuh"

namespace fc {

// ------------------------------------------------------------------------------- repack
// raw: N rows of K/32 blocks of 34 bytes. One thread per block.
__global__ void repack_q8_kernel(const uint8_t* __restrict__ raw, int N, int K, int N_pad,
                                 uint8_t* __restrict__ qu, __half* __restrict__ d) {
    const int kb_per_row = K / 32;
    const size_t total = (size_t)N_pad * kb_per_row;
    for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < total; b += (size_t)gridDim.x * blockDim.x) {
        const size_t row = b / kb_per_row;
        uint32_t w[8];
        __half scale = __ushort_as_half((unsigned short)0);
        if (row < (size_t)N) {
            const uint8_t* p = raw + b * 34;
            scale = __ushort_as_half((unsigned short)(p[0] | (p[1] << 8)));
            // the 32 quants start 2 bytes into the block: only 2-byte aligned
            const uint16_t* p16 = (const uint16_t*)(p + 2);
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = ((uint32_t)p16[2 * i] | ((uint32_t)p16[2 * i + 1] << 16)) ^ 0x80808080u;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = 0x80808080u;
        }
        uint4* dst = (uint4*)(qu + b * 32);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
        d[b] = scale;
    }
}

int launch_repack_q8(const uint8_t* raw, int N, int K, int N_pad, uint8_t* qu, __half* d, cudaStream_t st) {
    const size_t total = (size_t)N_pad * (K / 32);
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    repack_q8_kernel<<<blocks, threads, 0, st>>>(raw, N, K, N_pad, qu, d);
    FC_LAUNCHED();
    return FC_OK;
}

// --------------------------------------------------------------------------------- GEMV
// Biased byte b (= q + 128) of word w -> float q, exactly: the byte is placed in the low
// mantissa bits of 2^23, then 2^23 + 128 is subtracted.
template <int B>
__device__ __forceinline__ float qbyte(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - 8388736.0f;
}

__device__ __forceinline__ float dot16(const uint4& w, const float4* __restrict__ xs, int c) {
    // xs is the activation in shared memory, 16-byte units XOR-swizzled so that the
    // 16 lanes of a half warp (64-byte stride) hit distinct banks.
    const int sw = (c >> 1) & 3;
    const int base = 4 * c;
    const float4 x0 = xs[base + (0 ^ sw)], x1 = xs[base + (1 ^ sw)], x2 = xs[base + (2 ^ sw)], x3 = xs[base + (3 ^ sw)];
    // four independent chains of four dependent fused multiply-adds
    float a = x0.x * qbyte<0>(w.x), b = x1.x * qbyte<0>(w.y), c2 = x2.x * qbyte<0>(w.z), e = x3.x * qbyte<0>(w.w);
    a = fmaf(x0.y, qbyte<1>(w.x), a); b = fmaf(x1.y, qbyte<1>(w.y), b); c2 = fmaf(x2.y, qbyte<1>(w.z), c2); e = fmaf(x3.y, qbyte<1>(w.w), e);
    a = fmaf(x0.z, qbyte<2>(w.x), a); b = fmaf(x1.z, qbyte<2>(w.y), b); c2 = fmaf(x2.z, qbyte<2>(w.z), c2); e = fmaf(x3.z, qbyte<2>(w.w), e);
    a = fmaf(x0.w, qbyte<3>(w.x), a); b = fmaf(x1.w, qbyte<3>(w.y), b); c2 = fmaf(x2.w, qbyte<3>(w.z), c2); e = fmaf(x3.w, qbyte<3>(w.w), e);
    return (a + b) + (c2 + e);
}

struct GemvArgs {
    const uint8_t* qu; const __half* d; int N, K;
    const float* x; const float* bias; const float* residual; int epi;
    float* out0; float* out1; float* out2; int seg; size_t pos_stride;
    const StepState* state;
};

// Each half warp owns RIF rows at a time: 16 lanes x 16 bytes = 256 contiguous bytes of a
// row per load instruction, RIF independent 128-bit loads in flight per lane.
template <int RIF>
__global__ void __launch_bounds__(256) gemv_q8_kernel(GemvArgs a) {
    extern __shared__ float4 xs[];
    if (a.state && (a.state->done | a.state->error)) return;
    const int K = a.K, chunks = K >> 4;
    // stage x (swizzled 16-byte units)
    for (int u = threadIdx.x; u < (K >> 2); u += blockDim.x) xs[u ^ ((u >> 3) & 3)] = ((const float4*)a.x)[u];
    __syncthreads();

    const int hw = threadIdx.x >> 4, hl = threadIdx.x & 15;
    const int rows_per_block = (blockDim.x >> 4) * RIF;
    const int row0 = blockIdx.x * rows_per_block + hw * RIF;
    if (row0 >= a.N) return;   // half-warp uniform; shuffles below stay inside the half warp
    const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);

    float acc[RIF];
#pragma unroll
    for (int r = 0; r < RIF; ++r) acc[r] = 0.0f;
    const int kb_per_row = K >> 5;
    for (int c = hl; c < chunks; c += 16) {
        uint4 w[RIF];
        float sc[RIF];
#pragma unroll
        for (int r = 0; r < RIF; ++r) {
            // rows past N are inside the zero padding up to N_pad (kRowPad >= rows per pass)
            const size_t row = (size_t)(row0 + r);
            w[r] = __ldg((const uint4*)(a.qu + row * K) + c);
            sc[r] = __half2float(__ldg(a.d + row * kb_per_row + (c >> 1)));
        }
#pragma unroll
        for (int r = 0; r < RIF; ++r) acc[r] = fmaf(sc[r], dot16(w[r], xs, c), acc[r]);
    }
#pragma unroll
    for (int r = 0; r < RIF; ++r) {
        float v = acc[r];
        v += __shfl_xor_sync(hmask, v, 8);
        v += __shfl_xor_sync(hmask, v, 4);
        v += __shfl_xor_sync(hmask, v, 2);
        v += __shfl_xor_sync(hmask, v, 1);
        acc[r] = v;
    }
    if (hl == 0) {
        const int pos = a.state ? a.state->pos : 0;
#pragma unroll
        for (int r = 0; r < RIF; ++r) {
            const int n = row0 + r;
            if (n >= a.N) break;
            float v = acc[r];
            if (a.bias) v += a.bias[n];            // bias after the contraction (ops.rs:132-148)
            if (a.epi == EPI_GELU) v = gelu_f(v);
            if (a.residual) v = a.residual[n] + v; // x + proj (transformer.rs:286,292)
            const int s = n / a.seg, o = n - s * a.seg;
            float* dst = s == 0 ? a.out0 : (s == 1 ? a.out1 + (size_t)pos * a.pos_stride : a.out2 + (size_t)pos * a.pos_stride);
            dst[o] = v;
        }
    }
}

int launch_gemv_q8(const QMat& w, const float* x, const float* bias, const float* residual, int epi,
                   const GemvOut& out, const StepState* state, cudaStream_t st) {
    GemvArgs a;
    a.qu = w.qu; a.d = w.d; a.N = w.N; a.K = w.K;
    a.x = x; a.bias = bias; a.residual = residual; a.epi = epi;
    a.out0 = out.out[0]; a.out1 = out.out[1]; a.out2 = out.out[2];
    a.seg = out.seg > 0 ? out.seg : w.N; a.pos_stride = out.pos_stride;
    a.state = state;
    const size_t smem = (size_t)w.K * sizeof(float);
    const size_t weights = (size_t)w.N * w.K;
    if (weights >= (size_t)8 << 20) {
        const int threads = 256, rpb = (threads / 16) * 4;
        gemv_q8_kernel<4><<<(w.N + rpb - 1) / rpb, threads, smem, st>>>(a);
    } else if (w.N > 1024) {
        const int threads = 128, rpb = threads / 16;
        gemv_q8_kernel<1><<<(w.N + rpb - 1) / rpb, threads, smem, st>>>(a);
    } else {
        const int threads = 64, rpb = threads / 16;
        gemv_q8_kernel<1><<<(w.N + rpb - 1) / rpb, threads, smem, st>>>(a);
    }
    FC_LAUNCHED();
    return FC_OK;
}

// ------------------------------------------------------------------- split-K GEMV (Llama)
// The same product for the wide matrices of the Llama family (K up to 12288, N from 2048 to
// the vocabulary). A block of 16 half warps is G groups x S k-slices: a group owns RIF rows, its
// slices take interleaved runs of 16 chunks (256 B) of those rows and their partial sums are
// added in slice order through shared memory, so that even a [2048][8192] matrix spreads over
// several hundred blocks with RIF independent 128-bit loads in flight per lane.
// Prologue (optional): RMSNorm of the input row while it is staged (llm.rs:57-64).
// Epilogue: bias, residual, or SwiGLU over interleaved (gate, up) row pairs (llm.rs:417-428).
struct GemvWideArgs {
    const uint8_t* qu; const __half* d; int N, K;
    const float* x; const float* norm_w; float eps;
    const float* bias; const float* residual; int epi;
    float* out; int S;
    const StepState* state;
};

template <int RIF>
__global__ void __launch_bounds__(256) gemv_q8_wide_kernel(GemvWideArgs a) {
    extern __shared__ float4 xs[];
    __shared__ float red[33];
    __shared__ float part[16 * RIF];
    if (a.state && (a.state->done | a.state->error)) return;
    const int K = a.K, chunks = K >> 4, units = K >> 2;
    const int S = a.S, G = 16 / S;
    const int hw = threadIdx.x >> 4, hl = threadIdx.x & 15;
    const int g = hw / S, sl = hw - g * S;
    const int row0 = (blockIdx.x * G + g) * RIF;          // rows past N lie in the zero padding up to N_pad
    const int kb_per_row = K >> 5;
    // the first weights of this thread are requested before the activation is staged: they do
    // not depend on it, and their latency hides behind the staging and the norm
    uint4 w0[RIF];
    float sc0[RIF];
    const int c0 = sl * 16 + hl;
    const bool active = row0 < a.N && c0 < chunks;
    if (active) {
#pragma unroll
        for (int r = 0; r < RIF; ++r) {
            const size_t row = (size_t)(row0 + r);
            w0[r] = __ldg((const uint4*)(a.qu + row * K) + c0);
            sc0[r] = __half2float(__ldg(a.d + row * kb_per_row + (c0 >> 1)));
        }
    }
    // stage x (swizzled 16-byte units), normalising it on the way when asked
    float ss = 0.0f;
    for (int u = threadIdx.x; u < units; u += blockDim.x) {
        const float4 v = ((const float4*)a.x)[u];
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        xs[u ^ ((u >> 3) & 3)] = v;
    }
    if (a.norm_w) {
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[wid] = ss;
        __syncthreads();
        if (wid == 0) {
            float t = lane < 8 ? red[lane] : 0.0f;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0) red[32] = t;
        }
        __syncthreads();
        const float inv = 1.0f / sqrtf(red[32] / (float)K + a.eps);
        for (int u = threadIdx.x; u < units; u += blockDim.x) {      // the units this thread staged itself
            float4 v = xs[u ^ ((u >> 3) & 3)];
            const float4 w = ((const float4*)a.norm_w)[u];
            v.x = __fmul_rn(__fmul_rn(v.x, inv), w.x); v.y = __fmul_rn(__fmul_rn(v.y, inv), w.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv), w.z); v.w = __fmul_rn(__fmul_rn(v.w, inv), w.w);
            xs[u ^ ((u >> 3) & 3)] = v;
        }
    }
    __syncthreads();

    const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
    float acc[RIF];
#pragma unroll
    for (int r = 0; r < RIF; ++r) acc[r] = 0.0f;
    if (active) {
#pragma unroll
        for (int r = 0; r < RIF; ++r) acc[r] = sc0[r] * dot16(w0[r], xs, c0);
        for (int c = c0 + 16 * S; c < chunks; c += 16 * S) {
            uint4 w[RIF];
            float sc[RIF];
#pragma unroll
            for (int r = 0; r < RIF; ++r) {
                const size_t row = (size_t)(row0 + r);
                w[r] = __ldg((const uint4*)(a.qu + row * K) + c);
                sc[r] = __half2float(__ldg(a.d + row * kb_per_row + (c >> 1)));
            }
#pragma unroll
            for (int r = 0; r < RIF; ++r) acc[r] = fmaf(sc[r], dot16(w[r], xs, c), acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < RIF; ++r) {
        float v = acc[r];
        v += __shfl_xor_sync(hmask, v, 8);
        v += __shfl_xor_sync(hmask, v, 4);
        v += __shfl_xor_sync(hmask, v, 2);
        v += __shfl_xor_sync(hmask, v, 1);
        if (hl == 0) part[hw * RIF + r] = v;
    }
    __syncthreads();
    // thread t < G * RIF finishes row (t / RIF group, t % RIF): slices added in a fixed order
    const int t = threadIdx.x;
    float v = 0.0f;
    int n = a.N;
    if (t < G * RIF) {
        const int tg = t / RIF, tr = t - tg * RIF;
        for (int s2 = 0; s2 < S; ++s2) v += part[(tg * S + s2) * RIF + tr];
        n = (blockIdx.x * G + tg) * RIF + tr;
        if (n < a.N && a.bias) v += a.bias[n];
    }
    if (a.epi == EPI_SWIGLU) {
        __syncthreads();
        if (t < G * RIF) part[t] = v;
        __syncthreads();
        if (t < G * RIF && !(t & 1) && n < a.N) {
            const float gte = part[t], up = part[t + 1];
            a.out[n >> 1] = __fmul_rn(__fdiv_rn(gte, __fadd_rn(1.0f, expf(-gte))), up);
        }
        return;
    }
    if (t < G * RIF && n < a.N) {
        if (a.residual) v = a.residual[n] + v;
        a.out[n] = v;
    }
}

int launch_gemv_q8_wide(const QMat& w, const float* x, const float* norm_w, float eps, const float* bias, const float* residual,
                        int epi, float* out, const StepState* state, cudaStream_t st) {
    if (w.K % 16 || w.K > 12288) return fail(FC_E_SHAPE, "GEMV row length %d must be a multiple of 16, at most 12288", w.K);
    if (epi == EPI_SWIGLU && ((w.N & 1) || residual)) return fail(FC_E_SHAPE, "the SwiGLU epilogue pairs rows and takes no residual");
    GemvWideArgs a;
    a.qu = w.qu; a.d = w.d; a.N = w.N; a.K = w.K;
    a.x = x; a.norm_w = norm_w; a.eps = eps; a.bias = bias; a.residual = residual; a.epi = epi; a.out = out; a.state = state;
    const int chunks = w.K >> 4;
    const bool big = (size_t)w.N * w.K >= (size_t)8 << 20;
    const int rif = big ? 4 : 2;
    // more k-slices (fewer rows per block) until the grid fills the SMs four times over
    int S = 1;
    while (S < 16 && (w.N + (16 / S) * rif - 1) / ((16 / S) * rif) < 592 && chunks / (16 * S * 2) >= 1) S *= 2;
    a.S = S;
    const int rows_per_block = (16 / S) * rif;
    const int blocks = (w.N + rows_per_block - 1) / rows_per_block;
    const size_t smem = (size_t)w.K * sizeof(float);
    if (big) gemv_q8_wide_kernel<4><<<blocks, 256, smem, st>>>(a);
    else gemv_q8_wide_kernel<2><<<blocks, 256, smem, st>>>(a);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
