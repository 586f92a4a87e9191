// Streaming Q8_0 GEMV for one activation row against a wide matrix (the projections of the
// Llama family: K 2048..12288, N 2048..vocabulary).
//
// One persistent CTA per SM and call. A producer warp streams tiles of RT whole rows (RT*K quant bytes
// and RT*K/16 scale bytes, two bulk async copies) into a ring in shared memory, so that well
// over 100 KB per SM are in flight whatever the consumers are doing; 16 consumer warps take a
// tile as 32 units of (R2 rows, K part), one per half warp — the 16 activations of a chunk are
// read from shared memory once for the R2 rows — and the parts of a row are added in part order. The activation row is staged once per CTA, optionally RMS-normalised on the way
// (llm.rs:57-64); the epilogue adds bias and residual or applies SwiGLU to interleaved
// (gate, up) row pairs (llm.rs:417-428).
//
// Bound: HBM. Algorithmic bytes per call = N*K*34/32 + 4K + 4N.
// Every wait is bounded: a wait that runs out raises *status to FC_E_TIMEOUT and the CTA leaves.
// Launched as a programmatic dependent: the weight stream of a call starts while the kernel
// ahead of it in the step is still finishing.
#include <algorithm>

#include "fc_common.cuh"
#include "pdl.cuh"

namespace fc {

namespace {

constexpr int CONS = 512;                 // 16 consumer warps
constexpr int THREADS = CONS + 32;        // + 1 producer warp
constexpr int MAX_SLOTS = 8;
constexpr int RING_BYTES = 136 * 1024;
constexpr long long WAIT_CYCLES = 4000000000LL;   // ~2 s

struct StreamArgs {
    const uint8_t* qu; const __half* d; int N, N_pad, K;
    const float* x; const float* norm_w; float eps;
    const float* bias; const float* residual; int epi;
    float* out;
    const StepState* state; int* status;
    int RT;          // rows per tile (a power of two, at most 32)
    int slots;       // ring depth
    int slot_bytes;  // RT * K * 17 / 16 rounded up to 128
};

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
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(s32(b)), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// Bounded wait: false when the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(unsigned long long* b, uint32_t parity) {
    if (mbar_try_wait(b, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(b, parity))
        if (clock64() - t0 > WAIT_CYCLES) return false;
    return true;
}
// 1-D bulk copy global -> shared, evict-first in L2 (every weight byte is used once per token).
__device__ __forceinline__ void bulk_g2s_stream(void* dst, const void* src, uint32_t bytes, unsigned long long* b) {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(b)), "l"(policy) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONS) : "memory"); }

template <int B>
__device__ __forceinline__ float qbyte(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - 8388736.0f;
}
// 16 quants (biased bytes) against 16 activations held in registers (shared by the rows of a unit).
__device__ __forceinline__ float dot16x(const uint4& w, const float4& x0, const float4& x1, const float4& x2, const float4& x3) {
    float a = x0.x * qbyte<0>(w.x), b = x1.x * qbyte<0>(w.y), c2 = x2.x * qbyte<0>(w.z), e = x3.x * qbyte<0>(w.w);
    a = fmaf(x0.y, qbyte<1>(w.x), a); b = fmaf(x1.y, qbyte<1>(w.y), b); c2 = fmaf(x2.y, qbyte<1>(w.z), c2); e = fmaf(x3.y, qbyte<1>(w.w), e);
    a = fmaf(x0.z, qbyte<2>(w.x), a); b = fmaf(x1.z, qbyte<2>(w.y), b); c2 = fmaf(x2.z, qbyte<2>(w.z), c2); e = fmaf(x3.z, qbyte<2>(w.w), e);
    a = fmaf(x0.w, qbyte<3>(w.x), a); b = fmaf(x1.w, qbyte<3>(w.y), b); c2 = fmaf(x2.w, qbyte<3>(w.z), c2); e = fmaf(x3.w, qbyte<3>(w.w), e);
    return (a + b) + (c2 + e);
}

template <int R2>
__global__ void __launch_bounds__(THREADS, 1) gemv_q8_stream_kernel(StreamArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ unsigned long long full[MAX_SLOTS], empty[MAX_SLOTS];
    __shared__ float part[2][32 * R2];
    __shared__ float red[33];
    __shared__ int failed;
    // The weights are constants: the producer streams them while the kernel ahead is still
    // running. Everything that touches the activation, the state or the outputs waits first.
    pdl_trigger();
    const int K = a.K, chunks = K >> 4, units = K >> 2;
    float4* xs = (float4*)smem;
    unsigned char* ring = smem + (((size_t)K * 4 + 127) & ~(size_t)127);
    const int tid = threadIdx.x;
    const int tiles = a.N_pad / a.RT;
    const int my_tiles = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t q_bytes = (uint32_t)a.RT * K, d_bytes = (uint32_t)a.RT * (K >> 4);

    if (tid == 0) {
        for (int s = 0; s < a.slots; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CONS / 32); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (tid >= CONS) {
        // ------------------------------------------------------------------ producer warp
        if (tid == CONS) {
            for (int i = 0; i < my_tiles; ++i) {
                const int s = i % a.slots;
                if (i >= a.slots && !mbar_wait(&empty[s], (uint32_t)((i / a.slots - 1) & 1))) {
                    atomicExch(a.status, FC_E_TIMEOUT);
                    break;
                }
                const size_t row0 = (size_t)(blockIdx.x + (size_t)i * gridDim.x) * a.RT;
                unsigned char* slot = ring + (size_t)s * a.slot_bytes;
                mbar_expect_tx(&full[s], q_bytes + d_bytes);
                bulk_g2s_stream(slot, a.qu + row0 * K, q_bytes, &full[s]);
                bulk_g2s_stream(slot + q_bytes, (const unsigned char*)a.d + row0 * (K >> 4), d_bytes, &full[s]);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    pdl_wait();
    // a finished or failed stream still drains the ring (its copies are in flight) but writes nothing
    const bool dead = a.state && (a.state->done | a.state->error);
    // stage x (swizzled 16-byte units), normalising it on the way when asked
    float ss = 0.0f;
    for (int u = tid; u < units; u += CONS) {
        const float4 v = ((const float4*)a.x)[u];
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        xs[u ^ ((u >> 3) & 3)] = v;
    }
    const int lane = tid & 31, wid = tid >> 5;
    if (a.norm_w) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[wid] = ss;
        consumer_sync();
        if (wid == 0) {
            float t = lane < CONS / 32 ? red[lane] : 0.0f;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0) red[32] = t;
        }
        consumer_sync();
        const float inv = 1.0f / sqrtf(red[32] / (float)K + a.eps);
        for (int u = tid; u < units; u += CONS) {               // the units this thread staged itself
            float4 v = xs[u ^ ((u >> 3) & 3)];
            const float4 w = ((const float4*)a.norm_w)[u];
            v.x = __fmul_rn(__fmul_rn(v.x, inv), w.x); v.y = __fmul_rn(__fmul_rn(v.y, inv), w.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv), w.z); v.w = __fmul_rn(__fmul_rn(v.w, inv), w.w);
            xs[u ^ ((u >> 3) & 3)] = v;
        }
    }
    consumer_sync();

    // unit of this half warp inside a tile: rows (hw / P) * R2 .. + R2, K part hw % P
    const int P = 32 * R2 / a.RT;
    const int hw = tid >> 4, hl = tid & 15;
    const int ugrp = hw / P, upart = hw - ugrp * P;
    const int cpp = (chunks + P - 1) / P;
    const int c_begin = upart * cpp, c_end = min(chunks, c_begin + cpp);
    const unsigned hmask = 0xFFFFu << (tid & 16);
    const int kb_per_row = K >> 5;
    int buf = 0;
    for (int i = 0; i < my_tiles; ++i) {
        const int s = i % a.slots;
        const bool ok = mbar_wait(&full[s], (uint32_t)((i / a.slots) & 1));
        if (!ok) failed = 1;
        const unsigned char* slot = ring + (size_t)s * a.slot_bytes;
        const uint4* wq = (const uint4*)(slot + (size_t)(ugrp * R2) * K);
        const __half* wd = (const __half*)(slot + q_bytes) + (size_t)(ugrp * R2) * kb_per_row;
        float acc[R2];
#pragma unroll
        for (int r = 0; r < R2; ++r) acc[r] = 0.0f;
        if (ok) {
            for (int c = c_begin + hl; c < c_end; c += 16) {
                const int sw = (c >> 1) & 3, base = 4 * c;
                const float4 x0 = xs[base + (0 ^ sw)], x1 = xs[base + (1 ^ sw)], x2 = xs[base + (2 ^ sw)], x3 = xs[base + (3 ^ sw)];
#pragma unroll
                for (int r = 0; r < R2; ++r) {
                    const uint4 w = wq[(size_t)r * (K >> 4) + c];
                    const float sc = __half2float(wd[r * kb_per_row + (c >> 1)]);
                    acc[r] = fmaf(sc, dot16x(w, x0, x1, x2, x3), acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R2; ++r) {
            float v = acc[r];
            v += __shfl_xor_sync(hmask, v, 8);
            v += __shfl_xor_sync(hmask, v, 4);
            v += __shfl_xor_sync(hmask, v, 2);
            v += __shfl_xor_sync(hmask, v, 1);
            if (hl == 0) part[buf][hw * R2 + r] = v;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);                   // this warp no longer reads the slot
        consumer_sync();
        if (failed) {                                            // a tile never arrived: report and leave
            if (tid == 0) atomicExch(a.status, FC_E_TIMEOUT);
            break;
        }
        if (wid == 0) {
            // lane t < RT finishes row t of the tile: parts added in part order
            float r = 0.0f;
            const int t = lane;
            if (t < a.RT) {
                const int tg = t / R2, tr = t - tg * R2;
                for (int p = 0; p < P; ++p) r += part[buf][(tg * P + p) * R2 + tr];
            }
            const int n = (blockIdx.x + i * gridDim.x) * a.RT + t;
            const bool live = t < a.RT && n < a.N && !dead;
            if (live && a.bias) r += a.bias[n];
            if (a.epi == EPI_SWIGLU) {
                const float up = __shfl_down_sync(0xffffffffu, r, 1);
                if (live && !(t & 1)) a.out[n >> 1] = __fmul_rn(__fdiv_rn(r, __fadd_rn(1.0f, expf(-r))), up);
            } else if (live) {
                if (a.residual) r = a.residual[n] + r;
                a.out[n] = r;
            }
        }
        buf ^= 1;
    }
}

}  // namespace

// Shapes the ring covers: rows of whole 16-byte scale runs per tile and an x row that leaves
// room for at least two slots. Others take the register-pipelined kernel.
static bool stream_shape(const QMat& w, int* RT_out, int* slots_out, int* slot_bytes_out, int sms) {
    if (w.K % 32 || w.K > 12288 || w.N_pad % 32) return false;
    int RT = 32;
    // rows per tile: at most 32 KB of quants, and at least two tiles per CTA
    while (RT > 1 && ((size_t)RT * w.K > 32768 || w.N_pad / RT < 2 * sms)) RT >>= 1;
    if (RT < 2 || ((size_t)RT * (w.K >> 4)) % 16) return false;   // row pairs stay in one tile; scale bytes of a tile: a 16-byte multiple
    const int slot_bytes = (int)((((size_t)RT * w.K * 17 / 16) + 127) & ~(size_t)127);
    const int slots = std::min(MAX_SLOTS, RING_BYTES / slot_bytes);
    if (slots < 2) return false;
    *RT_out = RT; *slots_out = slots; *slot_bytes_out = slot_bytes;
    return true;
}

int launch_gemv_q8_stream(const QMat& w, const float* x, const float* norm_w, float eps, const float* bias, const float* residual,
                          int epi, float* out, const StepState* state, int* status, cudaStream_t st) {
    static int sms[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev >= 64) return fail(FC_E_ARG, "device index %d", dev);
    if (!sms[dev]) {
        FC_CUDA(cudaFuncSetAttribute(gemv_q8_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        FC_CUDA(cudaFuncSetAttribute(gemv_q8_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        FC_CUDA(cudaFuncSetAttribute(gemv_q8_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        FC_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    }
    int RT = 0, slots = 0, slot_bytes = 0;
    if (!status || !stream_shape(w, &RT, &slots, &slot_bytes, sms[dev]))
        return launch_gemv_q8_wide(w, x, norm_w, eps, bias, residual, epi, out, state, st);
    if (epi == EPI_SWIGLU && ((w.N & 1) || residual)) return fail(FC_E_SHAPE, "the SwiGLU epilogue pairs rows and takes no residual");
    StreamArgs a;
    a.qu = w.qu; a.d = w.d; a.N = w.N; a.N_pad = w.N_pad; a.K = w.K;
    a.x = x; a.norm_w = norm_w; a.eps = eps; a.bias = bias; a.residual = residual; a.epi = epi; a.out = out;
    a.state = state; a.status = status;
    a.RT = RT; a.slots = slots; a.slot_bytes = slot_bytes;
    const size_t smem = (((size_t)w.K * 4 + 127) & ~(size_t)127) + (size_t)slots * slot_bytes;
    const int tiles = w.N_pad / RT;
    // rows per unit: as many as keep every lane of a half warp on a chunk of its own
    const int chunks = w.K >> 4;
    int R2 = 4;
    while (R2 > 1 && (R2 > RT || 32 * R2 / RT > std::max(1, chunks / 16))) R2 >>= 1;
    const dim3 grid(std::min(tiles, sms[dev])), block(THREADS);
    if (R2 == 4) FC_CUDA(launch_pdl(gemv_q8_stream_kernel<4>, grid, block, smem, st, a));
    else if (R2 == 2) FC_CUDA(launch_pdl(gemv_q8_stream_kernel<2>, grid, block, smem, st, a));
    else FC_CUDA(launch_pdl(gemv_q8_stream_kernel<1>, grid, block, smem, st, a));
    ++g_launches;
    return FC_OK;
}

}  // namespace fc
