// Q8_0 GEMM on fp32 CUDA cores (math mode FC_MATH_FP32): Y = X·Wᵀ + bias (+GELU) (+res).
//
// Replaces ops::linear_forward (ferrum_core/src/ops.rs:233-256) for M >= 2 with the weight
// kept packed: each 128 x 32 weight tile is dequantised into shared memory as d * q (the
// single rounding of gguf::dequant_q8_0, ferrum_core/src/gguf/dequant.rs:37-49), and the
// products are accumulated in ascending k per output element with fused multiply-adds.
// This is the exactly-rounded fallback math mode and the yardstick for the tensor-core
// GEMM; it is CUDA-core bound (2MNK FLOP).
#include "fc_common.cuh"

namespace fc {

namespace {
constexpr int BM = 128, BN = 128, BK = 32, PAD = 4;
constexpr int LDA = BM + PAD, LDB = BN + PAD;

template <int B>
__device__ __forceinline__ float qb(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - 8388736.0f;
}
}  // namespace

struct GemmArgs {
    const uint8_t* qu; const __half* d; int N, K;
    const float* x; const float* bias; const float* residual; int epi;
    float* y; int M, ldy;
};

__global__ void __launch_bounds__(256) gemm_q8_fp32_kernel(GemmArgs a) {
    __shared__ __align__(16) float As[BK * LDA];   // [k][m]
    __shared__ __align__(16) float Bs[BK * LDB];   // [k][n]
    const int t = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int K = a.K, kb_per_row = K >> 5;

    // global -> register staging
    float4 ar[4];
    uint4 wr;
    float wscale;
    const int a_row = t >> 3, a_c4 = t & 7;         // + 32*i rows
    const int w_row = t >> 1, w_half = t & 1;
    auto load_tiles = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = m0 + a_row + 32 * i;
            ar[i] = m < a.M ? ((const float4*)(a.x + (size_t)m * K + k0))[a_c4] : make_float4(0, 0, 0, 0);
        }
        const size_t n = (size_t)(n0 + w_row);      // < N_pad (zero rows past N)
        wr = __ldg((const uint4*)(a.qu + n * K + k0) + w_half);
        wscale = __half2float(__ldg(a.d + n * kb_per_row + (k0 >> 5)));
    };
    auto store_tiles = [&]() {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = a_row + 32 * i, k = a_c4 * 4;
            As[(k + 0) * LDA + m] = ar[i].x; As[(k + 1) * LDA + m] = ar[i].y;
            As[(k + 2) * LDA + m] = ar[i].z; As[(k + 3) * LDA + m] = ar[i].w;
        }
        const int kb = w_half * 16;
        const uint32_t ws[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            Bs[(kb + 4 * j + 0) * LDB + w_row] = wscale * qb<0>(ws[j]);
            Bs[(kb + 4 * j + 1) * LDB + w_row] = wscale * qb<1>(ws[j]);
            Bs[(kb + 4 * j + 2) * LDB + w_row] = wscale * qb<2>(ws[j]);
            Bs[(kb + 4 * j + 3) * LDB + w_row] = wscale * qb<3>(ws[j]);
        }
    };

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    const int ty = t >> 4, tx = t & 15;

    load_tiles(0);
    for (int k0 = 0; k0 < K; k0 += BK) {
        __syncthreads();
        store_tiles();
        __syncthreads();
        if (k0 + BK < K) load_tiles(k0 + BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a0 = *(const float4*)&As[k * LDA + ty * 4];
            const float4 a1 = *(const float4*)&As[k * LDA + 64 + ty * 4];
            const float4 b0 = *(const float4*)&Bs[k * LDB + tx * 4];
            const float4 b1 = *(const float4*)&Bs[k * LDB + 64 + tx * 4];
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (a.bias) v += a.bias[n];
            if (a.epi == EPI_GELU) v = gelu_f(v);
            if (a.residual) v = a.residual[(size_t)m * a.ldy + n] + v;
            a.y[(size_t)m * a.ldy + n] = v;
        }
    }
}

// The same product for a handful of rows (a prompt being primed): SBM x 16 output tiles, so that
// a [32][768] x [768][2304] product still spreads over 144 CTAs instead of 18. Same arithmetic as
// the kernel above: d * q weights, one fused multiply-add per k in ascending order.
template <int SBM>
__global__ void __launch_bounds__(128) gemm_q8_fp32_skinny_kernel(GemmArgs a) {
    constexpr int SBN = 16, RM = SBM / 16, SLDA = SBM + 4, SLDB = SBN + 4;
    __shared__ __align__(16) float As[BK * SLDA];   // [k][m]
    __shared__ __align__(16) float Bs[BK * SLDB];   // [k][n]
    const int t = threadIdx.x;
    const int m0 = blockIdx.y * SBM, n0 = blockIdx.x * SBN;
    const int K = a.K, kb_per_row = K >> 5;
    const int tx = t & 7, ty = t >> 3;              // columns 2 tx, 2 tx + 1; rows ty * RM ...
    float acc[RM][2];
#pragma unroll
    for (int i = 0; i < RM; ++i) acc[i][0] = acc[i][1] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        __syncthreads();
        // activations: SBM rows x 32 k, eight float4 per row
#pragma unroll
        for (int i = 0; i < SBM * 8 / 128; ++i) {
            const int idx = t + 128 * i, row = idx >> 3, c4 = idx & 7, m = m0 + row;
            const float4 v = m < a.M ? ((const float4*)(a.x + (size_t)m * K + k0))[c4] : make_float4(0, 0, 0, 0);
            As[(4 * c4 + 0) * SLDA + row] = v.x; As[(4 * c4 + 1) * SLDA + row] = v.y;
            As[(4 * c4 + 2) * SLDA + row] = v.z; As[(4 * c4 + 3) * SLDA + row] = v.w;
        }
        // weights: 16 rows x 32 quants of one Q8_0 block column
        if (t < 32) {
            const int row = t >> 1, half = t & 1;
            const size_t n = (size_t)(n0 + row);     // < N_pad (zero rows past N)
            const uint4 wr = __ldg((const uint4*)(a.qu + n * K + k0) + half);
            const float wscale = __half2float(__ldg(a.d + n * kb_per_row + (k0 >> 5)));
            const uint32_t ws[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                Bs[(half * 16 + 4 * j + 0) * SLDB + row] = wscale * qb<0>(ws[j]);
                Bs[(half * 16 + 4 * j + 1) * SLDB + row] = wscale * qb<1>(ws[j]);
                Bs[(half * 16 + 4 * j + 2) * SLDB + row] = wscale * qb<2>(ws[j]);
                Bs[(half * 16 + 4 * j + 3) * SLDB + row] = wscale * qb<3>(ws[j]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float2 b = *(const float2*)&Bs[k * SLDB + tx * 2];
#pragma unroll
            for (int i = 0; i < RM; ++i) {
                const float av = As[k * SLDA + ty * RM + i];
                acc[i][0] = fmaf(av, b.x, acc[i][0]);
                acc[i][1] = fmaf(av, b.y, acc[i][1]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < RM; ++i) {
        const int m = m0 + ty * RM + i;
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int n = n0 + tx * 2 + j;
            if (n >= a.N) continue;
            float v = acc[i][j];
            if (a.bias) v += a.bias[n];
            if (a.epi == EPI_GELU) v = gelu_f(v);
            if (a.residual) v = a.residual[(size_t)m * a.ldy + n] + v;
            a.y[(size_t)m * a.ldy + n] = v;
        }
    }
}

int launch_gemm_q8_fp32(const QMat& w, const float* x, const float* bias, const float* residual, int epi,
                        float* y, int M, int ldy, cudaStream_t st) {
    GemmArgs a;
    a.qu = w.qu; a.d = w.d; a.N = w.N; a.K = w.K;
    a.x = x; a.bias = bias; a.residual = residual; a.epi = epi;
    a.y = y; a.M = M; a.ldy = ldy;
    if (M <= 64) {
        // few rows: small tiles so that every SM gets one
        dim3 grid((w.N + 15) / 16, 1);
        if (M <= 32) gemm_q8_fp32_skinny_kernel<32><<<grid, 128, 0, st>>>(a);
        else gemm_q8_fp32_skinny_kernel<64><<<grid, 128, 0, st>>>(a);
        FC_LAUNCHED();
        return FC_OK;
    }
    dim3 grid((w.N + BN - 1) / BN, (M + BM - 1) / BM);
    gemm_q8_fp32_kernel<<<grid, 256, 0, st>>>(a);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
