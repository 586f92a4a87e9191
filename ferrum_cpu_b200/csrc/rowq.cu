// Per-row-scale int8 / int4 linear: ops::qlinear (ferrum_core/src/ops.rs:268-377) on a QWeight
// (quant.rs:122-263) kept packed on the device.
//
//     y[i][j] = bias[j] + sum_p (x[i][p] * scale[p]) * level[p][j]
//
// The matrix is [K = in][N = out] with the outputs contiguous, so a thread owns a run of 4 to 16
// packed bytes of every row — that many columns (int8) or twice as many (int4: the low nibbles
// are columns b.., the high nibbles half+b..) — and walks down the rows: loads are coalesced
// across the warp, no cross-thread reduction is needed, and the K dimension is cut into slices
// so that a single activation row still fills the GPU. Slice partials are added in slice order.
// Up to 8 activation rows share one pass over the weights.
//
// Bound: HBM for M <= 8. Algorithmic bytes = K * row_bytes + 4K (scales) + 4 M (K + N).
#include <algorithm>

#include "fc_common.cuh"

struct fc_rowq {
    int device = 0;
    int rows = 0, cols = 0, kind = 0;
    int ld = 0;                    // bytes between rows on the device (row_bytes rounded up to 16)
    fc::Arena arena;
    uint8_t* q = nullptr;
    float* scales = nullptr;
    // scratch: slice partials, grown on demand. A single activation row has a buffer of its own, whose size never
    // changes once it exists: a captured decode step keeps pointing at it whatever the batched calls do to the other.
    fc::Arena ws, ws1;
    float* partial = nullptr;
    size_t partial_floats = 0;
    float* partial1 = nullptr;
    size_t partial1_floats = 0;
};

namespace fc {

namespace {

constexpr int MT = 8;            // most activation rows per pass
constexpr int TPB = 128;

// Byte B of w as a float, w holding levels biased to unsigned (level + bias): the byte lands in
// the low mantissa bits of 2^23 and 2^23 + bias is subtracted — exact.
template <int B>
__device__ __forceinline__ float level(uint32_t w, float magic) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - magic;
}

struct RowqArgs {
    const uint8_t* q; const float* scales; int K, N, ld, half;
    const float* x; const float* bias; float* y; float* partial;
    int M, kper, KS;
    int ldy;                       // floats between output rows
    const float* residual;         // [M][ldy] or null: y = residual + (bias + sum); may be y itself
};

template <int W> struct Words;
template <> struct Words<1> { using T = uint32_t; };
template <> struct Words<2> { using T = uint2; };
template <> struct Words<4> { using T = uint4; };

// grid: (runs of 4 W bytes of a row, k-slices, passes of MTT rows). A thread owns 4 W packed
// bytes of every weight row: 4 W columns (int8) or 8 W (int4). One activation row takes 16-byte
// loads (W = 4) and keeps 8 rows of the slice in flight; more rows trade width for accumulators.
// KL > 1 (single activation row): the block's threads are TPB / KL column runs x KL row lanes,
// lane l takes rows l, l + KL, ... of the slice and the lanes are added in lane order through
// shared memory, so that few k-slices (little partial traffic) still mean many threads.
template <int INT4, int W, int MTT, int KL>
__global__ void __launch_bounds__(TPB) rowq_linear_kernel(RowqArgs a) {
    extern __shared__ float as[];                 // [rows of this pass][kper]: x * scale
    constexpr int NB = 4 * W;                     // bytes per thread and row
    constexpr int C = INT4 ? 2 * NB : NB;         // columns per thread
    const int m0 = blockIdx.z * MTT, mt = min(MTT, a.M - m0);
    const int p0 = blockIdx.y * a.kper, p1 = min(a.K, p0 + a.kper), np = p1 - p0;
    for (int u = threadIdx.x; u < mt * np; u += TPB) {
        const int m = u / np, p = u - m * np;
        as[m * a.kper + p] = a.x[(size_t)(m0 + m) * a.K + p0 + p] * a.scales[p0 + p];   // ops.rs:336-342
    }
    __syncthreads();
    constexpr int TX = TPB / KL;
    const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const int b0 = (blockIdx.x * TX + tx) * NB;                   // byte offset inside a row
    const bool inside = b0 < a.ld;
    if (KL == 1 && !inside) return;
    float acc[MTT][C];
#pragma unroll
    for (int m = 0; m < MTT; ++m)
#pragma unroll
        for (int c = 0; c < C; ++c) acc[m][c] = 0.0f;
    const uint8_t* col = a.q + (inside ? b0 : 0);
#pragma unroll 8
    for (int p = ty; p < np; p += KL) {
        union { typename Words<W>::T v; uint32_t w[W]; } ld;
        ld.v = __ldg((const typename Words<W>::T*)(col + (size_t)(p0 + p) * a.ld));
        float lv[C];
#pragma unroll
        for (int i = 0; i < W; ++i) {
            if (INT4) {
                // nibble n (two's complement) -> n ^ 8 is level + 8 as an unsigned byte
                const uint32_t lo = (ld.w[i] & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((ld.w[i] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
                lv[4 * i] = level<0>(lo, 8388616.0f); lv[4 * i + 1] = level<1>(lo, 8388616.0f);
                lv[4 * i + 2] = level<2>(lo, 8388616.0f); lv[4 * i + 3] = level<3>(lo, 8388616.0f);
                lv[(NB + 4 * i) % C] = level<0>(hi, 8388616.0f); lv[(NB + 4 * i + 1) % C] = level<1>(hi, 8388616.0f);
                lv[(NB + 4 * i + 2) % C] = level<2>(hi, 8388616.0f); lv[(NB + 4 * i + 3) % C] = level<3>(hi, 8388616.0f);
            } else {
                const uint32_t b = ld.w[i] ^ 0x80808080u;          // i8 -> level + 128
                lv[4 * i] = level<0>(b, 8388736.0f); lv[4 * i + 1] = level<1>(b, 8388736.0f);
                lv[4 * i + 2] = level<2>(b, 8388736.0f); lv[4 * i + 3] = level<3>(b, 8388736.0f);
            }
        }
#pragma unroll
        for (int m = 0; m < MTT; ++m) {
            if (m < mt) {
                const float ap = as[m * a.kper + p];
#pragma unroll
                for (int c = 0; c < C; ++c) acc[m][c] = fmaf(ap, lv[c], acc[m][c]);
            }
        }
    }
    if (KL > 1) {
        // lanes 1 .. KL-1 hand their sums to lane 0, which adds them in lane order (MTT == 1 here)
        float* red = as + MTT * a.kper;                            // [KL][TX][C]
        __syncthreads();
        if (ty > 0) {
#pragma unroll
            for (int c = 0; c < C; ++c) red[(ty * TX + tx) * C + c] = acc[0][c];
        }
        __syncthreads();
        if (ty > 0 || !inside) return;
        for (int l = 1; l < KL; ++l)
#pragma unroll
            for (int c = 0; c < C; ++c) acc[0][c] += red[(l * TX + tx) * C + c];
    }
    // columns of this thread: b0 .. b0 + NB - 1, and for int4 also half + b0 .. half + b0 + NB - 1
    for (int m = 0; m < mt; ++m) {
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const int j = c < NB ? b0 + c : a.half + b0 + (c - NB);
            const bool live = INT4 ? (c < NB ? j < a.half : j < a.N) : j < a.N;
            if (!live) continue;
            if (a.KS == 1) {
                const float v = (a.bias ? a.bias[j] : 0.0f) + acc[m][c];
                const size_t at = (size_t)(m0 + m) * a.ldy + j;
                a.y[at] = a.residual ? a.residual[at] + v : v;
            }
            else a.partial[((size_t)blockIdx.y * a.M + m0 + m) * a.N + j] = acc[m][c];
        }
    }
}

// y = bias + partial[0] + partial[1] + ... in slice order.
__global__ void rowq_reduce_kernel(const float* __restrict__ partial, const float* __restrict__ bias, const float* residual, float* y,
                                   int M, int N, int KS, int ldy) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * N) return;
    const size_t m = i / N, j = i - m * N;
    float v = bias ? bias[j] : 0.0f;
    for (int s = 0; s < KS; ++s) v += partial[(size_t)s * M * N + i];
    const size_t at = m * ldy + j;
    y[at] = residual ? residual[at] + v : v;
}

int rowq_launch(fc_rowq* w, const float* x, const float* bias, const float* residual, float* y, int ldy, int M, cudaStream_t st) {
    static int sms[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !sms[dev]) FC_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    const int n_sm = dev < 64 ? sms[dev] : 148;
    // bytes per thread and rows per pass: one row takes 16-byte loads, a few rows 8, many 4
    const int W = M == 1 ? 4 : (M <= 4 ? 2 : 1), mtt = M == 1 ? 1 : (M <= 4 ? 4 : MT);
    const int KL = M == 1 ? 8 : 1, tx = TPB / KL;
    const int bx = (w->ld / (4 * W) + tx - 1) / tx, mz = (M + mtt - 1) / mtt;
    // k-slices: enough blocks to fill the SMs four times over, at least 64 rows per slice (the
    // partials then cost under a tenth of the weight bytes), and a slice of x * scale within 32 KB
    int KS = std::max(1, (4 * n_sm + bx * mz - 1) / (bx * mz));
    KS = std::min(KS, std::max(1, w->rows / 64));
    int kper = (w->rows + KS - 1) / KS;
    const int kper_max = 32768 / (4 * std::min(M, mtt));
    if (kper > kper_max) kper = kper_max;
    KS = (w->rows + kper - 1) / kper;
    float* scratch = nullptr;
    if (KS > 1) {
        const size_t need = (size_t)KS * M * w->cols;
        fc::Arena& arena = M == 1 ? w->ws1 : w->ws;
        float*& buf = M == 1 ? w->partial1 : w->partial;
        size_t& have = M == 1 ? w->partial1_floats : w->partial_floats;
        if (need > have) {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            FC_CUDA(cudaStreamIsCapturing(st, &cap));
            if (cap != cudaStreamCaptureStatusNone) return fail(FC_E_CUDA, "rowq linear: scratch must exist before a stream capture");
            FC_CUDA(cudaStreamSynchronize(st));
            arena.release();
            buf = nullptr; have = 0;
            FC_TRY(arena.alloc_n(&buf, need));
            have = need;
        }
        scratch = buf;
    }
    RowqArgs a;
    a.q = w->q; a.scales = w->scales; a.K = w->rows; a.N = w->cols; a.ld = w->ld; a.half = (w->cols + 1) / 2;
    a.x = x; a.bias = bias; a.y = y; a.partial = scratch; a.M = M; a.kper = kper; a.KS = KS;
    a.ldy = ldy; a.residual = residual;
    const dim3 grid(bx, KS, mz);
    const bool i4 = w->kind == FC_Q_INT4;
    const size_t smem = ((size_t)std::min(M, mtt) * kper + (KL > 1 ? (size_t)TPB * (i4 ? 32 : 16) : 0)) * sizeof(float);
    if (W == 4) { if (i4) rowq_linear_kernel<1, 4, 1, 8><<<grid, TPB, smem, st>>>(a); else rowq_linear_kernel<0, 4, 1, 8><<<grid, TPB, smem, st>>>(a); }
    else if (W == 2) { if (i4) rowq_linear_kernel<1, 2, 4, 1><<<grid, TPB, smem, st>>>(a); else rowq_linear_kernel<0, 2, 4, 1><<<grid, TPB, smem, st>>>(a); }
    else { if (i4) rowq_linear_kernel<1, 1, MT, 1><<<grid, TPB, smem, st>>>(a); else rowq_linear_kernel<0, 1, MT, 1><<<grid, TPB, smem, st>>>(a); }
    FC_LAUNCHED();
    if (KS > 1) {
        const size_t n = (size_t)M * w->cols;
        rowq_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(scratch, bias, residual, y, M, w->cols, KS, ldy);
        FC_LAUNCHED();
    }
    return FC_OK;
}

}  // namespace

// y[M][ldy] (columns 0 .. cols-1) = [residual +] bias + x · W for a packed matrix; bias and residual may be null.
int launch_rowq_linear(fc_rowq* w, const float* x, const float* bias, const float* residual, float* y, int ldy, int M, cudaStream_t st) {
    if (ldy < w->cols) return fail(FC_E_SHAPE, "rowq linear: row stride %d below %d columns", ldy, w->cols);
    return rowq_launch(w, x, bias, residual, y, ldy, M, st);
}
int rowq_in(const fc_rowq* w) { return w->rows; }
int rowq_out(const fc_rowq* w) { return w->cols; }
}  // namespace fc

using namespace fc;

extern "C" {

int fc_rowq_upload(int device, const uint8_t* q, const float* scales, int rows, int cols, int kind, fc_rowq** out) {
    if (!q || !scales || !out) return fail(FC_E_ARG, "fc_rowq_upload: null argument");
    *out = nullptr;
    if (rows <= 0 || cols <= 0) return fail(FC_E_SHAPE, "fc_rowq_upload: [%d][%d]", rows, cols);
    if (kind != FC_Q_INT8 && kind != FC_Q_INT4) return fail(FC_E_ARG, "fc_rowq_upload: kind %d", kind);
    FC_TRY(select_device(device));
    fc_rowq* w = new fc_rowq();
    w->device = device; w->rows = rows; w->cols = cols; w->kind = kind;
    const size_t rb = kind == FC_Q_INT4 ? (size_t)(cols + 1) / 2 : (size_t)cols;
    w->ld = (int)((rb + 15) & ~(size_t)15);
    auto build = [&]() -> int {
        FC_TRY(w->arena.alloc_n(&w->q, (size_t)rows * w->ld));
        FC_TRY(w->arena.alloc_n(&w->scales, (size_t)rows));
        FC_CUDA(cudaMemset(w->q, 0, (size_t)rows * w->ld));
        FC_CUDA(cudaMemcpy2D(w->q, (size_t)w->ld, q, rb, rb, (size_t)rows, cudaMemcpyHostToDevice));
        FC_CUDA(cudaMemcpy(w->scales, scales, (size_t)rows * sizeof(float), cudaMemcpyHostToDevice));
        return FC_OK;
    };
    const int rc = build();
    if (rc != FC_OK) { fc_rowq_free(w); return rc; }
    *out = w;
    return FC_OK;
}

void fc_rowq_free(fc_rowq* w) {
    if (!w) return;
    cudaSetDevice(w->device);
    cudaDeviceSynchronize();
    w->ws.release();
    w->ws1.release();
    w->arena.release();
    delete w;
}

int fc_rowq_linear_dev(const fc_rowq* w, const float* x_dev, const float* bias_dev, float* y_dev, int M, void* stream) {
    if (!w || !x_dev || !bias_dev || !y_dev) return fail(FC_E_ARG, "fc_rowq_linear_dev: null argument");
    if (!aligned16(x_dev) || !aligned16(y_dev) || !aligned16(bias_dev))
        return fail(FC_E_ARG, "fc_rowq_linear_dev: x_dev, y_dev and bias_dev must be 16-byte aligned");
    if (M <= 0) return fail(FC_E_SHAPE, "fc_rowq_linear_dev: M = %d", M);
    FC_CUDA(cudaSetDevice(w->device));
    return rowq_launch(const_cast<fc_rowq*>(w), x_dev, bias_dev, nullptr, y_dev, w->cols, M, (cudaStream_t)stream);
}

int fc_rowq_linear(const fc_rowq* w, const float* x, const float* bias, float* y, int M) {
    if (!w || !x || !bias || !y) return fail(FC_E_ARG, "fc_rowq_linear: null argument");
    if (M <= 0) return fail(FC_E_SHAPE, "fc_rowq_linear: M = %d", M);
    FC_CUDA(cudaSetDevice(w->device));
    Arena a;
    float *xd = nullptr, *bd = nullptr, *yd = nullptr;
    int rc = a.alloc_n(&xd, (size_t)M * w->rows);
    if (rc == FC_OK) rc = a.alloc_n(&bd, (size_t)w->cols);
    if (rc == FC_OK) rc = a.alloc_n(&yd, (size_t)M * w->cols);
    auto copy = [&](void* dst, const void* src, size_t bytes, cudaMemcpyKind kind) {
        if (rc == FC_OK && cudaMemcpy(dst, src, bytes, kind) != cudaSuccess) rc = fail(FC_E_CUDA, "fc_rowq_linear: copy failed");
    };
    copy(xd, x, (size_t)M * w->rows * 4, cudaMemcpyHostToDevice);
    copy(bd, bias, (size_t)w->cols * 4, cudaMemcpyHostToDevice);
    if (rc == FC_OK) rc = rowq_launch(const_cast<fc_rowq*>(w), xd, bd, nullptr, yd, w->cols, M, nullptr);
    if (rc == FC_OK && cudaDeviceSynchronize() != cudaSuccess) rc = fail(FC_E_CUDA, "fc_rowq_linear: the kernel failed");
    copy(y, yd, (size_t)M * w->cols * 4, cudaMemcpyDeviceToHost);
    a.release();
    return rc;
}

}  // extern "C"
