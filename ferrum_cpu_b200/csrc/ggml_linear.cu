// Linear layers on weights kept in their GGML block format (gguf/dequant.rs:37-315): y = x · dequant(W)ᵀ + bias with
// the blocks decoded inside the kernel, so a matrix occupies its file footprint on the device (4.5 bits per weight for
// Q4_0 and Q4_K, 5.5 for Q5_0 / Q5_K, 6.56 for Q6_K, ...) and is never expanded.
//
// This is the reference's precision-preserving import (`load_llama_prec(None)`, gguf/llama.rs:171-176: every tensor
// decoded to f32, Linear::forward on f32 weights) with the decode moved into the product. Every decoded value is
// formed exactly as the reference's decoder forms it (the order of the f32 products and subtractions), so
// w[n][k] is bit-identical; the sum over k runs in a fixed order of its own (a lane per 32-value (sub-)block, then a
// shuffle tree), not the reference's ascending order.
//
// One warp per output row; the lanes take the row's 32-value sub-blocks in turn; up to 8 activation rows share a pass
// over the weights. Bound: HBM for M <= 8 at the format's own bytes. A format-generic kernel: the Q8_0 kernels of
// this library are 2-5x faster on Q8_0.
#include <algorithm>

#include "fc_common.cuh"

struct fc_ggml_weight {
    int device = 0;
    int type = 0, N = 0, K = 0;
    size_t row_bytes = 0;
    fc::Arena arena;
    uint8_t* raw = nullptr;
};

namespace fc {

namespace {

__device__ __forceinline__ float half_at(const uint8_t* p) { return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8)))); }

// gguf/dequant.rs:133-141
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* q, int* sc, int* mn) {
    if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
    else { *sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4); *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

struct Fmt { int vals, bytes; };
__host__ __device__ inline Fmt fmt_of(int t) {
    switch (t) {
        case FC_GGML_F32: return {32, 128};     // treated as blocks of 32 values here
        case FC_GGML_F16: return {32, 64};
        case FC_GGML_Q4_0: return {32, 18};
        case FC_GGML_Q4_1: return {32, 20};
        case FC_GGML_Q5_0: return {32, 22};
        case FC_GGML_Q5_1: return {32, 24};
        case FC_GGML_Q8_0: return {32, 34};
        case FC_GGML_Q8_1: return {32, 36};
        case FC_GGML_Q2_K: return {256, 84};
        case FC_GGML_Q3_K: return {256, 110};
        case FC_GGML_Q4_K: return {256, 144};
        case FC_GGML_Q5_K: return {256, 176};
        case FC_GGML_Q6_K: return {256, 210};
        default: return {0, 0};
    }
}

// The 32 values of sub-block sb of the (super-)block at b, in the order they have in the row: positions
// 32 sb .. 32 sb + 31 of the block's 32 or 256 values. The arithmetic follows gguf/dequant.rs line by line.
__device__ __forceinline__ void dequant32(int t, const uint8_t* b, int sb, float* out) {
    switch (t) {
        case FC_GGML_F32:
            for (int j = 0; j < 32; ++j) { uint32_t u = b[4 * j] | (b[4 * j + 1] << 8) | (b[4 * j + 2] << 16) | ((uint32_t)b[4 * j + 3] << 24); out[j] = __uint_as_float(u); }
            break;
        case FC_GGML_F16:
            for (int j = 0; j < 32; ++j) out[j] = half_at(b + 2 * j);
            break;
        case FC_GGML_Q8_0: case FC_GGML_Q8_1: {
            const float d = half_at(b);
            const int8_t* q = (const int8_t*)(b + (t == FC_GGML_Q8_0 ? 2 : 4));
            for (int j = 0; j < 32; ++j) out[j] = d * (float)q[j];
            break;
        }
        case FC_GGML_Q4_0: {
            const float d = half_at(b);
            for (int j = 0; j < 16; ++j) {
                out[j] = d * (float)((int)(b[2 + j] & 0x0F) - 8);
                out[j + 16] = d * (float)((int)(b[2 + j] >> 4) - 8);
            }
            break;
        }
        case FC_GGML_Q4_1: {
            const float d = half_at(b), m = half_at(b + 2);
            for (int j = 0; j < 16; ++j) {
                out[j] = __fadd_rn(__fmul_rn(d, (float)(b[4 + j] & 0x0F)), m);
                out[j + 16] = __fadd_rn(__fmul_rn(d, (float)(b[4 + j] >> 4)), m);
            }
            break;
        }
        case FC_GGML_Q5_0: case FC_GGML_Q5_1: {
            const bool with_min = t == FC_GGML_Q5_1;
            const float d = half_at(b), m = with_min ? half_at(b + 2) : 0.0f;
            const uint8_t* hb = b + (with_min ? 4 : 2);
            const uint32_t qh = (uint32_t)hb[0] | ((uint32_t)hb[1] << 8) | ((uint32_t)hb[2] << 16) | ((uint32_t)hb[3] << 24);
            const uint8_t* qs = hb + 4;
            for (int j = 0; j < 16; ++j) {
                const int x0 = (qs[j] & 0x0F) | (int)(((qh >> j) & 1u) << 4);
                const int x1 = (qs[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
                out[j] = with_min ? __fadd_rn(__fmul_rn(d, (float)x0), m) : d * (float)(x0 - 16);
                out[j + 16] = with_min ? __fadd_rn(__fmul_rn(d, (float)x1), m) : d * (float)(x1 - 16);
            }
            break;
        }
        case FC_GGML_Q4_K: case FC_GGML_Q5_K: {
            // sub-block sb: low (sb even) or high (sb odd) nibbles of bytes 32 (sb / 2) .. + 31; its own 6-bit scale and minimum
            const bool five = t == FC_GGML_Q5_K;
            const float d = half_at(b), dmin = half_at(b + 2);
            const uint8_t* qh = b + 16;
            const uint8_t* qs = b + (five ? 48 : 16) + 32 * (sb >> 1);
            int sc, mn;
            k4_scale_min(sb, b + 4, &sc, &mn);
            const float ds = __fmul_rn(d, (float)sc), ms = __fmul_rn(dmin, (float)mn);
            for (int l = 0; l < 32; ++l) {
                const int nib = (sb & 1) ? (qs[l] >> 4) : (qs[l] & 0x0F);
                const int hi = five && (qh[l] & (1u << sb)) ? 16 : 0;
                out[l] = __fsub_rn(__fmul_rn(ds, (float)(nib + hi)), ms);
            }
            break;
        }
        case FC_GGML_Q6_K: {
            // sub-block sb = 4 half + k: values 128 half + 32 k + l
            const int half = sb >> 2, k = sb & 3;
            const uint8_t *ql = b + 64 * half + ((k & 1) ? 32 : 0), *qh = b + 128 + 32 * half;
            const int8_t* sc = (const int8_t*)(b + 192) + 8 * half + 2 * k;
            const float d = half_at(b + 208);
            for (int l = 0; l < 32; ++l) {
                const int nib = (k & 2) ? (ql[l] >> 4) : (ql[l] & 0x0F);
                const int q = (nib | (((qh[l] >> (2 * k)) & 3) << 4)) - 32;
                out[l] = __fmul_rn(__fmul_rn(d, (float)sc[l / 16]), (float)q);
            }
            break;
        }
        case FC_GGML_Q2_K: {
            // sub-block sb = 4 half + shift / 2: two runs of 16
            const int half = sb >> 2, shift = 2 * (sb & 3);
            const uint8_t *scales = b + 2 * sb, *qs = b + 16 + 32 * half;
            const float d = half_at(b + 80), dmin = half_at(b + 82);
            for (int r = 0; r < 2; ++r) {
                const float dl = __fmul_rn(d, (float)(scales[r] & 0x0F)), ml = __fmul_rn(dmin, (float)(scales[r] >> 4));
                for (int l = 0; l < 16; ++l) out[16 * r + l] = __fsub_rn(__fmul_rn(dl, (float)((qs[16 * r + l] >> shift) & 3)), ml);
            }
            break;
        }
        case FC_GGML_Q3_K: {
            const int half = sb >> 2, shift = 2 * (sb & 3);
            const uint8_t *hmask = b, *qs = b + 32 + 32 * half, *sc = b + 96;
            const float d = half_at(b + 108);
            const unsigned m = 1u << sb;                   // the high-bit selector doubles after each shift group
            for (int r = 0; r < 2; ++r) {
                const int j = 2 * sb + r;                  // scale index
                int s6 = j < 8 ? (sc[j] & 0x0F) : (sc[j - 8] >> 4);
                s6 |= ((sc[8 + j / 4] >> (2 * (j % 4))) & 3) << 4;
                const float dl = __fmul_rn(d, (float)((int)(int8_t)s6 - 32));
                for (int l = 16 * r; l < 16 * r + 16; ++l) {
                    const int low = (qs[l] >> shift) & 3;
                    out[l] = __fmul_rn(dl, (float)(low - ((hmask[l] & m) ? 0 : 4)));
                }
            }
            break;
        }
    }
}

constexpr int MT = 8;   // activation rows per pass over the weights

struct LinArgs {
    const uint8_t* raw; size_t row_bytes; int type, N, K;
    const float* x; const float* bias; const float* residual; float* y; int ldy, M;
};

// grid.x: groups of (blockDim.x / 32) output rows, grid.y: passes of MT activation rows. A warp brings the bytes of 32
// sub-blocks of its row into shared memory with coalesced loads (2 or 4 bytes per lane: the blocks are only 2-byte
// aligned in general) and every lane decodes its own sub-block from there: byte-wise global loads of the blocks stall
// on their latency and throttle the load queue (5.0 and 1.5 stalls per issue, 65 us for a 16384 x 2048 Q4_K matrix).
constexpr int STAGE_BYTES = 32 * 128;      // the widest 32 sub-blocks: f32

// T: the ggml type, a compile-time constant so that each instance carries one decoder only.
template <int T>
__global__ void __launch_bounds__(256) ggml_linear_kernel(LinArgs a) {
    __shared__ __align__(16) uint8_t stage_all[8 * STAGE_BYTES];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= a.N) return;
    uint8_t* stage = stage_all + warp * STAGE_BYTES;
    const int m0 = blockIdx.y * MT, mt = min(MT, a.M - m0);
    const Fmt f = fmt_of(T);
    const int per = f.vals >> 5;                               // 32-value sub-blocks per block
    const int n_sub = a.K >> 5;
    const uint8_t* row = a.raw + (size_t)n * a.row_bytes;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.0f;
    for (int s0 = 0; s0 < n_sub; s0 += 32) {
        const int b0 = s0 / per, b1 = (min(s0 + 32, n_sub) + per - 1) / per;       // blocks of this chunk
        const uint8_t* src = row + (size_t)b0 * f.bytes;
        const int len = (b1 - b0) * f.bytes;
        if ((((uintptr_t)src | (uintptr_t)len) & 3) == 0)
            for (int i = lane; i < (len >> 2); i += 32) ((uint32_t*)stage)[i] = __ldg((const uint32_t*)src + i);
        else
            for (int i = lane; i < (len >> 1); i += 32) ((uint16_t*)stage)[i] = __ldg((const uint16_t*)src + i);
        __syncwarp();
        const int s = s0 + lane;
        if (s < n_sub) {
            float w[32];
            dequant32(T, stage + (size_t)(s / per - b0) * f.bytes, s % per, w);
            for (int m = 0; m < mt; ++m) {
                const float4* xr = (const float4*)(a.x + (size_t)(m0 + m) * a.K + 32 * s);
                float t = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 v = xr[j];
                    t = fmaf(v.x, w[4 * j], t); t = fmaf(v.y, w[4 * j + 1], t); t = fmaf(v.z, w[4 * j + 2], t); t = fmaf(v.w, w[4 * j + 3], t);
                }
                acc[m] += t;
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    if (lane == 0)
        for (int m = 0; m < mt; ++m) {
            const size_t at = (size_t)(m0 + m) * a.ldy + n;
            const float v = acc[m] + (a.bias ? a.bias[n] : 0.0f);
            a.y[at] = a.residual ? a.residual[at] + v : v;
        }
}

// Rows ids[r] of a table kept in its block format, decoded: the embedding lookup (llm.rs:588-597 copies the decoded
// row). One warp per row; a bad id raises the error word and leaves the row zero. With `state` (one row): the queued
// token at the cache position, refused like a bad id when the context is full (llm.rs:610-618, :720-730), nothing at
// all once the stream is done or in error.
__global__ void ggml_rows_kernel(const uint8_t* raw, size_t row_bytes, int type, int N, int K, const int* ids, StepState* state,
                                 const int* queue, int ctx, int R, float* x, int* error_flag) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    if (state && (state->done | state->error)) return;
    const int id = ids ? ids[r] : queue[state->fed];
    if (id < 0 || id >= N || (state && state->pos >= ctx)) {
        if (state) {
            __syncwarp();
            if (lane == 0) state->error = FC_E_DIM;
            return;
        }
        if (lane == 0 && error_flag) atomicExch(error_flag, FC_E_DIM);
        for (int c = lane; c < K; c += 32) x[(size_t)r * K + c] = 0.0f;
        return;
    }
    const Fmt f = fmt_of(type);
    const int per = f.vals >> 5;
    const uint8_t* row = raw + (size_t)id * row_bytes;
    for (int s = lane; s < (K >> 5); s += 32) {
        float w[32];
        dequant32(type, row + (size_t)(s / per) * f.bytes, s % per, w);
        for (int j = 0; j < 32; ++j) x[(size_t)r * K + 32 * s + j] = w[j];
    }
}

}  // namespace

int launch_ggml_linear(const fc_ggml_weight* w, const float* x, const float* bias, const float* residual, float* y, int ldy, int M,
                       cudaStream_t st) {
    if (ldy < w->N) return fail(FC_E_SHAPE, "ggml linear: row stride %d below %d columns", ldy, w->N);
    LinArgs a{w->raw, w->row_bytes, w->type, w->N, w->K, x, bias, residual, y, ldy, M};
    const dim3 grid((w->N + 7) / 8, (M + MT - 1) / MT);
    switch (w->type) {
#define FC_CASE(T) case T: ggml_linear_kernel<T><<<grid, 256, 0, st>>>(a); break;
        FC_CASE(FC_GGML_F32) FC_CASE(FC_GGML_F16) FC_CASE(FC_GGML_Q4_0) FC_CASE(FC_GGML_Q4_1) FC_CASE(FC_GGML_Q5_0) FC_CASE(FC_GGML_Q5_1)
        FC_CASE(FC_GGML_Q8_0) FC_CASE(FC_GGML_Q8_1) FC_CASE(FC_GGML_Q2_K) FC_CASE(FC_GGML_Q3_K) FC_CASE(FC_GGML_Q4_K) FC_CASE(FC_GGML_Q5_K)
        FC_CASE(FC_GGML_Q6_K)
#undef FC_CASE
        default: return fail(FC_E_FORMAT, "ggml type %d", w->type);
    }
    FC_LAUNCHED();
    return FC_OK;
}

int launch_ggml_rows(const fc_ggml_weight* w, const int* ids, StepState* state, const int* queue, int ctx, int R, float* x,
                     int* error_flag, cudaStream_t st) {
    ggml_rows_kernel<<<(R + 7) / 8, 256, 0, st>>>(w->raw, w->row_bytes, w->type, w->N, w->K, ids, state, queue, ctx, R, x, error_flag);
    FC_LAUNCHED();
    return FC_OK;
}

int ggml_weight_rows(const fc_ggml_weight* w) { return w->N; }
int ggml_weight_cols(const fc_ggml_weight* w) { return w->K; }

}  // namespace fc

using namespace fc;

extern "C" {

int fc_ggml_weight_upload(int device, int ggml_type, const void* raw, size_t nbytes, int N, int K, fc_ggml_weight** out) {
    if (!raw || !out) return fail(FC_E_ARG, "fc_ggml_weight_upload: null argument");
    *out = nullptr;
    if (N <= 0 || K <= 0) return fail(FC_E_SHAPE, "fc_ggml_weight_upload: [%d][%d]", N, K);
    const Fmt f = fmt_of(ggml_type);
    if (!f.vals) return fail(FC_E_FORMAT, "ggml type %d is not one the importer reads", ggml_type);
    if (K % f.vals || K % 32) return fail(FC_E_FORMAT, "rows of %d values do not hold whole blocks of ggml type %d", K, ggml_type);
    const size_t row_bytes = (size_t)(K / f.vals) * f.bytes;
    if (nbytes < row_bytes * (size_t)N) return fail(FC_E_FORMAT, "ggml tensor data is shorter than [%d][%d] of type %d", N, K, ggml_type);
    FC_TRY(select_device(device));
    fc_ggml_weight* w = new fc_ggml_weight();
    w->device = device; w->type = ggml_type; w->N = N; w->K = K; w->row_bytes = row_bytes;
    auto build = [&]() -> int {
        FC_TRY(w->arena.alloc_n(&w->raw, row_bytes * (size_t)N));
        FC_CUDA(cudaMemcpy(w->raw, raw, row_bytes * (size_t)N, cudaMemcpyHostToDevice));
        return FC_OK;
    };
    const int rc = build();
    if (rc != FC_OK) { fc_ggml_weight_free(w); return rc; }
    *out = w;
    return FC_OK;
}

void fc_ggml_weight_free(fc_ggml_weight* w) {
    if (!w) return;
    cudaSetDevice(w->device);
    cudaDeviceSynchronize();
    w->arena.release();
    delete w;
}

int fc_ggml_linear_dev(const fc_ggml_weight* w, const float* x_dev, const float* bias_dev, float* y_dev, int M, void* stream) {
    if (!w || !x_dev || !y_dev) return fail(FC_E_ARG, "fc_ggml_linear_dev: null argument");
    if (!aligned16(x_dev)) return fail(FC_E_ARG, "fc_ggml_linear_dev: x_dev must be 16-byte aligned");
    if (M <= 0) return fail(FC_E_SHAPE, "fc_ggml_linear_dev: M = %d", M);
    FC_CUDA(cudaSetDevice(w->device));
    return launch_ggml_linear(w, x_dev, bias_dev, nullptr, y_dev, w->N, M, (cudaStream_t)stream);
}

int fc_ggml_linear(const fc_ggml_weight* w, const float* x, const float* bias, float* y, int M) {
    if (!w || !x || !y) return fail(FC_E_ARG, "fc_ggml_linear: null argument");
    if (M <= 0) return fail(FC_E_SHAPE, "fc_ggml_linear: M = %d", M);
    FC_CUDA(cudaSetDevice(w->device));
    Arena a;
    float *xd = nullptr, *bd = nullptr, *yd = nullptr;
    int rc = a.alloc_n(&xd, (size_t)M * w->K);
    if (rc == FC_OK && bias) rc = a.alloc_n(&bd, (size_t)w->N);
    if (rc == FC_OK) rc = a.alloc_n(&yd, (size_t)M * w->N);
    auto copy = [&](void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
        if (rc == FC_OK && cudaMemcpy(dst, src, bytes, kind) != cudaSuccess) rc = fail(FC_E_CUDA, "fc_ggml_linear: copy failed");
    };
    copy(xd, x, (size_t)M * w->K * 4, cudaMemcpyHostToDevice);
    if (bias) copy(bd, bias, (size_t)w->N * 4, cudaMemcpyHostToDevice);
    if (rc == FC_OK) rc = launch_ggml_linear(w, xd, bd, nullptr, yd, w->N, M, nullptr);
    if (rc == FC_OK && cudaDeviceSynchronize() != cudaSuccess) rc = fail(FC_E_CUDA, "fc_ggml_linear: the kernel failed");
    copy(y, yd, (size_t)M * w->N * 4, cudaMemcpyDeviceToHost);
    a.release();
    return rc;
}

}  // extern "C"
