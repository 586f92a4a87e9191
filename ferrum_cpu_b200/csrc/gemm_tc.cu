// Q8_0 GEMM on the 5th-generation tensor cores (math mode FC_MATH_BF16X3):
//     Y[M][N] = X[M][K] · dequant(W[N][K])ᵀ + bias (+GELU) (+residual)
//
// Replaces ops::linear_forward (ferrum_core/src/ops.rs:233-256) for M >= 2 with the weight
// kept packed. The reference multiplies f32 by f32; tcgen05 has no f32 operand kind, so both
// operands are split into two bf16 terms (x = xh + xl, w = wh + wl, each exact to 2^-17
// relative) and every 128x128x16 step issues three kind::f16 MMAs into the same fp32 TMEM
// accumulator: xh·wh + xl·wh + xh·wl. The dropped xl·wl term is 2^-16 relative per product.
//
// Persistent kernel, one CTA per SM, 256 x 128 output tiles (two 128-row MMA tiles that share
// one dequantised weight tile) taken round-robin, N fastest, so that the CTAs running together
// share a few row panels of X in L2:
//   warp 16     TMA producer: the two bf16 planes of the X tile (256 rows x 64 k, 128-byte
//               swizzle) into the stage's A buffers, completing on the stage's mbarrier;
//   warps 8-15  dequantise the 128 x 64 Q8_0 weight tile: w = d * q exactly as
//               gguf::dequant_q8_0 (ferrum_core/src/gguf/dequant.rs:37-49), split into bf16
//               hi/lo and stored in the same swizzled K-major layout the tensor core reads;
//   warp 17     allocates all 512 TMEM columns (two buffers of two accumulators) and issues tcgen05.mma from one
//               thread; tcgen05.commit frees the stage and finally publishes the accumulator;
//   warps 0-7   epilogue of the previous tile while the next one is being multiplied, four warps (one per 32
//               TMEM lanes) for each 128-row half: tcgen05.ld their accumulator lanes, bias / GELU /
//               residual, then either f32 rows or the bf16 hi/lo planes the next GEMM consumes. (With four
//               warps for the whole tile the epilogue outlasted the MMAs of the next tile and held its buffer.)
// Every mbarrier wait is bounded by a cycle budget; when it runs out the kernel raises a
// status word, releases its TMEM and returns.
//
// Bound: tensor pipe. 2·M·N·K algorithmic FLOP (6·M·N·K executed).
#include <cuda.h>
#include <cuda_bf16.h>

#include "fc_common.cuh"

namespace fc {

namespace {

constexpr int BM = 256, BN = 128, BK = 64;            // a CTA tile is two 128-row MMA tiles sharing one weight tile
constexpr int STAGES = 2;
constexpr int TILE_BYTES = 128 * BK * 2;                // one 128-row bf16 operand tile: 16 KiB
constexpr int A_BYTES = 2 * TILE_BYTES;                 // one plane of the 256-row X tile
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * TILE_BYTES;   // A hi, A lo (256 rows each), B hi, B lo
constexpr int EPI_WARPS = 8, DQ_WARPS = 8;   // epilogue: four warps (one per 32 TMEM lanes) for each 128-row half of the tile
constexpr int TMA_WARP = EPI_WARPS + DQ_WARPS, MMA_WARP = TMA_WARP + 1;
constexpr int THREADS = (MMA_WARP + 1) * 32;
constexpr int TMEM_COLS = 512;                          // two buffers of two 128-column accumulators
// bf16 x bf16 -> f32, M = 128, N = 128, both operands K-major
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

struct Bars {
    unsigned long long full_a[STAGES];
    unsigned long long full_b[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    uint32_t tmem_base;
    volatile int abort;
};
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + (int)sizeof(Bars);

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
// A thread that finds the phase incomplete is suspended by the hardware for up to 2 us.
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(s32(b)), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (after raising the status word) when the budget runs out or
// another role of this CTA already gave up.
__device__ bool wait_bar(Bars* bars, unsigned long long* b, uint32_t parity, int* status, long long budget) {
    const long long t0 = clock64();
    while (!mbar_try_wait(b, parity)) {
        if (bars->abort) return false;
        if (clock64() - t0 > budget) {
            bars->abort = 1;
            atomicExch(status, FC_E_TIMEOUT);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(s32(dst)), "l"(map), "r"(x), "r"(y), "r"(s32(bar)) : "memory");
}
// K-major, 128-byte swizzle: 8-row atoms of 1024 bytes (SBO = 64 x 16 B), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)64 << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}

template <int B>
__device__ __forceinline__ float qb(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 + B)) - 8388736.0f;
}
// Two values -> packed bf16 hi pair and lo pair (element 0 in the low half).
__device__ __forceinline__ void split2(float w0, float w1, uint32_t* hi, uint32_t* lo) {
    const __nv_bfloat162 h = __float22bfloat162_rn(make_float2(w0, w1));
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __float22bfloat162_rn(make_float2(w0 - hf.x, w1 - hf.y));
    *hi = *(const uint32_t*)&h;
    *lo = *(const uint32_t*)&l;
}

// 256-bit global accesses: one full 32-byte sector per lane and instruction.
__device__ __forceinline__ void st256(void* p, const uint32_t* v) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]) : "memory");
}
__device__ __forceinline__ void ld256(const void* p, uint32_t* v) {
    asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "l"(p) : "memory");
}

struct TcArgs {
    const uint8_t* qu; const __half* d; int N, K;
    const float* bias; const float* residual; int epi;
    float* y;                 // f32 output rows, or null when the output goes to planes
    uint16_t *yhi, *ylo;      // bf16 hi / lo output planes [M][ldy]
    int M, ldy;
    int* status;
    // EPI_SCORE: per (row, N tile) softmax statistics instead of the product (see launch_gemm_q8_bf16x3_score)
    const int* targets;
    float4* stats;
    float* tlogit;
    long long wait_cycles;    // budget of every mbarrier wait
    int withhold;             // test hook: the TMA producer issues nothing, so the waits on its stages run out
};

}  // namespace

__global__ void __launch_bounds__(THREADS, 1)
gemm_q8_bf16x3_kernel(const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo, const TcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Bars* bars = (Bars*)(smem + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = a.K / BK;
    const int tiles_n = (a.N + BN - 1) / BN, tiles_m = (a.M + BM - 1) / BM;
    const int n_tiles = tiles_n * tiles_m;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bars->full_a[s], 1);
            mbar_init(&bars->full_b[s], DQ_WARPS);
            mbar_init(&bars->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->acc_full[b], 1);
            mbar_init(&bars->acc_empty[b], EPI_WARPS);
        }
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {   // the MMA warp owns the tensor memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&bars->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;

    if (warp == TMA_WARP) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && !a.withhold) {
            int it = 0;                                   // k-blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * BM;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_bar(bars, &bars->empty[s], ((it / STAGES) & 1) ^ 1, a.status, a.wait_cycles)) { tile = n_tiles; break; }
                    unsigned char* st = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&bars->full_a[s], 2 * A_BYTES);
                    tma_load_2d(st, &map_hi, kb * BK, m0, &bars->full_a[s]);
                    tma_load_2d(st + A_BYTES, &map_lo, kb * BK, m0, &bars->full_a[s]);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int it = 0, ti = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++ti) {
                const int buf = ti & 1;
                // the epilogue must have drained this accumulator (two tiles ago)
                ok = wait_bar(bars, &bars->acc_empty[buf], ((ti >> 1) & 1) ^ 1, a.status, a.wait_cycles);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem + (uint32_t)(buf * 2 * BN);     // rows 0..127 here, rows 128..255 at + BN
                for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t par = (it / STAGES) & 1;
                    ok = wait_bar(bars, &bars->full_a[s], par, a.status, a.wait_cycles) && wait_bar(bars, &bars->full_b[s], par, a.status, a.wait_cycles);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t base = s32(smem + s * STAGE_BYTES);
                    const uint64_t bh = smem_desc(base + 2 * A_BYTES), bl = smem_desc(base + 2 * A_BYTES + TILE_BYTES);
#pragma unroll
                    for (int hm = 0; hm < 2; ++hm) {                     // the two 128-row halves of the X tile
                        const uint64_t ah = smem_desc(base + hm * TILE_BYTES), al = smem_desc(base + A_BYTES + hm * TILE_BYTES);
#pragma unroll
                        for (int ks = 0; ks < BK / 16; ++ks) {
                            const uint64_t adv = (uint64_t)(ks * 2);    // 32 bytes per k-step of 16 bf16
                            umma(acc + hm * BN, ah + adv, bh + adv, (kb | ks) != 0);
                            umma(acc + hm * BN, al + adv, bh + adv, 1);
                            umma(acc + hm * BN, ah + adv, bl + adv, 1);
                        }
                    }
                    umma_commit(&bars->empty[s]);                    // frees the stage when the MMAs retire
                }
                if (ok) umma_commit(&bars->acc_full[buf]);
            }
        }
    } else if (warp >= EPI_WARPS) {
        // ---------------------------------------------------------------- weight dequantisers
        const int t = threadIdx.x - EPI_WARPS * 32;  // 0..255
        const int row = t >> 1, half = t & 1;        // weight row of the tile, 32-wide half of the k-block
        int it = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const int n0 = (tile % tiles_n) * BN;
            const size_t n = (size_t)(n0 + row);     // < N_pad (zero rows past N)
            const uint8_t* qrow = a.qu + n * a.K + half * 32;
            const __half* drow = a.d + n * (a.K >> 5) + half;
            // two k-blocks of quants are kept in flight ahead of the one being converted; they
            // rotate through named registers (an array indexed by kb & 1 would live in local memory)
            const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
            uint4 qa0 = z4, qc0 = z4, qa1 = z4, qc1 = z4;
            float sc0 = 0.0f, sc1 = 0.0f;
            if (0 < nkb) {
                qa0 = __ldg((const uint4*)qrow);
                qc0 = __ldg((const uint4*)qrow + 1);
                sc0 = __half2float(__ldg(drow));
            }
            if (1 < nkb) {
                qa1 = __ldg((const uint4*)(qrow + (size_t)BK));
                qc1 = __ldg((const uint4*)(qrow + (size_t)BK) + 1);
                sc1 = __half2float(__ldg(drow + 2));
            }
            for (int kb = 0; kb < nkb; ++kb, ++it) {
                const int s = it % STAGES;
                const uint4 c0 = qa0, c1 = qc0;
                const float scale = sc0;
                qa0 = qa1; qc0 = qc1; sc0 = sc1;
                if (kb + 2 < nkb) {
                    qa1 = __ldg((const uint4*)(qrow + (size_t)(kb + 2) * BK));
                    qc1 = __ldg((const uint4*)(qrow + (size_t)(kb + 2) * BK) + 1);
                    sc1 = __half2float(__ldg(drow + (kb + 2) * 2));
                }
                // the conversion runs before the stage is waited for: only the stores sit between
                // the stage becoming free and becoming full again
                const uint32_t ws[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                uint4 hi[4], lo[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {        // 16-byte chunk c of this half: 8 weights
                    split2(scale * qb<0>(ws[2 * c]), scale * qb<1>(ws[2 * c]), &hi[c].x, &lo[c].x);
                    split2(scale * qb<2>(ws[2 * c]), scale * qb<3>(ws[2 * c]), &hi[c].y, &lo[c].y);
                    split2(scale * qb<0>(ws[2 * c + 1]), scale * qb<1>(ws[2 * c + 1]), &hi[c].z, &lo[c].z);
                    split2(scale * qb<2>(ws[2 * c + 1]), scale * qb<3>(ws[2 * c + 1]), &hi[c].w, &lo[c].w);
                }
                if (!wait_bar(bars, &bars->empty[s], ((it / STAGES) & 1) ^ 1, a.status, a.wait_cycles)) { tile = n_tiles; break; }
                unsigned char* bhi = smem + s * STAGE_BYTES + 2 * A_BYTES + row * 128;
                unsigned char* blo = bhi + TILE_BYTES;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int chunk = ((half * 4 + c) ^ (row & 7)) * 16;   // 128-byte swizzle
                    *(uint4*)(bhi + chunk) = hi[c];
                    *(uint4*)(blo + chunk) = lo[c];
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->full_b[s]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 0-7)
        const bool vec_ok = (a.ldy & 3) == 0 && (((uintptr_t)a.y | (uintptr_t)a.residual) & 15) == 0;
        // rows of 32 columns start on 32-byte boundaries: whole-sector accesses
        const bool vec8_ok = (a.ldy & 7) == 0 && (((uintptr_t)a.y | (uintptr_t)a.residual) & 31) == 0;
        int ti = 0;
        // EPI_SCORE: running (largest logit, sum of exponentials relative to it, its first column) of this lane's row
        // over the four 32-column chunks of a tile, and the row's target
        float run_m = -INFINITY, run_s = 0.0f;
        int run_i = 0x7fffffff, tgt = -1;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++ti) {
            const int buf = ti & 1;
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            if (!wait_bar(bars, &bars->acc_full[buf], (ti >> 1) & 1, a.status, a.wait_cycles)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int hm = warp >> 2, quarter = warp & 3;                // 128-row half of the tile, 32-lane quarter of TMEM
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {                          // 32-column chunk
                const int m = m0 + hm * 128 + quarter * 32 + lane;
                uint32_t r[32];
                const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((buf * 2 + hm) * BN + c * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                      "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                      "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c == BN / 32 - 1) {
                    // this warp's part of the accumulator is in registers: hand the TMEM buffer back to the MMA warp
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
                }
                const int nb = n0 + c * 32;
                if (a.epi == EPI_SCORE) {
                    if (c == 0) {
                        run_m = -INFINITY; run_s = 0.0f; run_i = 0x7fffffff;
                        tgt = m < a.M ? __ldg(a.targets + m) : -1;
                    }
                    if (m < a.M && nb < a.N) {
                        // this chunk's largest logit and its first column (columns past N do not exist)
                        float cm = -INFINITY;
                        int ci = 0x7fffffff;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const float t = __uint_as_float(r[i]);
                            if (nb + i < a.N && t > cm) { cm = t; ci = nb + i; }
                        }
                        if (cm > run_m) {                      // strictly larger: an equal later column never replaces an earlier one
                            run_s *= expf(run_m - cm);          // run_m == -inf: run_s is 0 and stays 0
                            run_m = cm;
                            run_i = ci;
                        }
                        float e = 0.0f;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (nb + i < a.N) e += expf(__uint_as_float(r[i]) - run_m);
                        run_s += e;
                        if (tgt >= nb && tgt < nb + 32) {
                            float tl = 0.0f;
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (nb + i == tgt) tl = __uint_as_float(r[i]);
                            a.tlogit[m] = tl;
                        }
                    }
                    if (c == BN / 32 - 1 && m < a.M)
                        a.stats[(size_t)m * tiles_n + (tile % tiles_n)] = make_float4(run_m, run_s, __int_as_float(run_i), 0.0f);
                } else
                if (m < a.M && nb < a.N) {
                const bool full = nb + 32 <= a.N;
                float v[32];
                const size_t off = (size_t)m * a.ldy + nb;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float t = __uint_as_float(r[i]);
                    if (a.bias && (full || nb + i < a.N)) t += __ldg(a.bias + nb + i);
                    if (a.epi == EPI_GELU) t = gelu_f(t);
                    v[i] = t;
                }
                if (a.residual) {
                    if (full && vec8_ok) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t rr[8];
                            ld256(a.residual + off + 8 * i, rr);
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[8 * i + j] = __uint_as_float(rr[j]) + v[8 * i + j];
                        }
                    } else if (full && vec_ok) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 rr = *(const float4*)(a.residual + off + 4 * i);
                            v[4 * i] = rr.x + v[4 * i]; v[4 * i + 1] = rr.y + v[4 * i + 1];
                            v[4 * i + 2] = rr.z + v[4 * i + 2]; v[4 * i + 3] = rr.w + v[4 * i + 3];
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (nb + i < a.N) v[i] = a.residual[off + i] + v[i];
                    }
                }
                if (a.y) {
                    if (full && vec8_ok) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) w[j] = __float_as_uint(v[8 * i + j]);
                            st256(a.y + off + 8 * i, w);
                        }
                    } else if (full && vec_ok) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *(float4*)(a.y + off + 4 * i) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (nb + i < a.N) a.y[off + i] = v[i];
                    }
                } else {
                    if (a.epi == EPI_SWIGLU) {
                        // columns (2j, 2j + 1) are (gate_j, up_j) (llm.rs:417-428): 16 gated values, planes [M][N / 2]
                        uint32_t hi8[8], lo8[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float g0 = v[4 * i], g1 = v[4 * i + 2];
                            const float h0 = __fmul_rn(__fdiv_rn(g0, __fadd_rn(1.0f, expf(-g0))), v[4 * i + 1]);
                            const float h1 = __fmul_rn(__fdiv_rn(g1, __fadd_rn(1.0f, expf(-g1))), v[4 * i + 3]);
                            split2(h0, h1, &hi8[i], &lo8[i]);
                        }
                        const size_t o2 = (size_t)m * a.ldy + (nb >> 1);
                        if ((((uintptr_t)a.yhi | (uintptr_t)a.ylo) & 31) == 0 && (a.ldy & 15) == 0) {
                            st256(a.yhi + o2, hi8);
                            st256(a.ylo + o2, lo8);
                        } else {
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                *(uint4*)(a.yhi + o2 + 8 * i) = make_uint4(hi8[4 * i], hi8[4 * i + 1], hi8[4 * i + 2], hi8[4 * i + 3]);
                                *(uint4*)(a.ylo + o2 + 8 * i) = make_uint4(lo8[4 * i], lo8[4 * i + 1], lo8[4 * i + 2], lo8[4 * i + 3]);
                            }
                        }
                    } else {
                    // bf16 hi / lo planes for the next GEMM (ldy % 8 == 0, N % 32 == 0 for these outputs)
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) split2(v[2 * i], v[2 * i + 1], &hi[i], &lo[i]);
                    if ((((uintptr_t)a.yhi | (uintptr_t)a.ylo) & 31) == 0 && (a.ldy & 15) == 0) {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            st256(a.yhi + off + 16 * i, hi + 8 * i);
                            st256(a.ylo + off + 16 * i, lo + 8 * i);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            *(uint4*)(a.yhi + off + 8 * i) = make_uint4(hi[4 * i], hi[4 * i + 1], hi[4 * i + 2], hi[4 * i + 3]);
                            *(uint4*)(a.ylo + off + 8 * i) = make_uint4(lo[4 * i], lo[4 * i + 1], lo[4 * i + 2], lo[4 * i + 3]);
                        }
                    }
                    }
                }
                }
                __syncwarp();      // the next tcgen05.ld is warp-collective
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// x[n] -> bf16 hi, lo planes with x = hi + lo to 2^-17 relative.
__global__ void split_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo, size_t n4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = ((const float4*)x)[i];
        uint2 h, l;
        split2(v.x, v.y, &h.x, &l.x);
        split2(v.z, v.w, &h.y, &l.y);
        ((uint2*)hi)[i] = h;
        ((uint2*)lo)[i] = l;
    }
}

int launch_split_bf16(const float* x, void* hi, void* lo, size_t n, cudaStream_t st) {
    if (n % 4) return fail(FC_E_SHAPE, "split_bf16: element count %zu is not a multiple of 4", n);
    const size_t n4 = n / 4;
    const int blocks = (int)((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
    split_bf16_kernel<<<blocks > 0 ? blocks : 1, 256, 0, st>>>(x, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo, n4);
    FC_LAUNCHED();
    return FC_OK;
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_plane(CUtensorMap* map, const void* plane, int M, int K) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        FC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) return fail(FC_E_CUDA, "cuTensorMapEncodeTiled is not available");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};   // 64 x 256: two 128-row MMA tiles
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)plane, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FC_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for a [%d][%d] bf16 plane", (int)r, M, K);
    return FC_OK;
}
}  // namespace

// x_hi / x_lo: bf16 planes [M][K] (16-byte aligned). Output: f32 rows y (ldy floats apart), or, when
// y is null, bf16 planes y_hi / y_lo (N % 32 == 0, ldy % 8 == 0). status: device int, raised on timeout.
static int launch_tc(const QMat& w, const void* x_hi, const void* x_lo, TcArgs a, int M, cudaStream_t st) {
    static int sms[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev >= 64) return fail(FC_E_ARG, "device %d out of range", dev);
    if (!sms[dev]) {
        FC_CUDA(cudaFuncSetAttribute(gemm_q8_bf16x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        FC_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    }
    CUtensorMap mh, ml;
    FC_TRY(encode_plane(&mh, x_hi, M, w.K));
    FC_TRY(encode_plane(&ml, x_lo, M, w.K));
    a.qu = w.qu; a.d = w.d; a.N = w.N; a.K = w.K; a.M = M;
    a.wait_cycles = g_debug.wait_cycles; a.withhold = g_debug.withhold;
    const int n_tiles = ((w.N + BN - 1) / BN) * ((M + BM - 1) / BM);
    const int grid = n_tiles < sms[dev] ? n_tiles : sms[dev];
    gemm_q8_bf16x3_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(mh, ml, a);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_gemm_q8_bf16x3_ex(const QMat& w, const void* x_hi, const void* x_lo, const float* bias, const float* residual,
                             int epi, float* y, void* y_hi, void* y_lo, int M, int ldy, int* status, cudaStream_t st) {
    if (w.K % BK) return fail(FC_E_SHAPE, "the tensor-core GEMM needs K %% 64 == 0 (K = %d)", w.K);
    if (!y && (!y_hi || !y_lo || (w.N & 31) || (ldy & 7) || residual))
        return fail(FC_E_SHAPE, "plane output needs N %% 32 == 0, ldy %% 8 == 0 and no residual");
    if (epi == EPI_SWIGLU && (y || ldy < w.N / 2)) return fail(FC_E_SHAPE, "the SwiGLU epilogue writes planes [M][N / 2]");
    if (epi == EPI_SCORE) return fail(FC_E_ARG, "the scoring epilogue has its own entry");
    TcArgs a = {};
    a.bias = bias; a.residual = residual; a.epi = epi;
    a.y = y; a.yhi = (uint16_t*)y_hi; a.ylo = (uint16_t*)y_lo; a.ldy = ldy; a.status = status;
    return launch_tc(w, x_hi, x_lo, a, M, st);
}

int launch_gemm_q8_bf16x3_score(const QMat& w, const void* x_hi, const void* x_lo, const int* targets, void* stats, float* tlogit,
                                int M, int* status, cudaStream_t st) {
    if (w.K % BK) return fail(FC_E_SHAPE, "the tensor-core GEMM needs K %% 64 == 0 (K = %d)", w.K);
    if (!targets || !stats || !tlogit) return fail(FC_E_ARG, "the scoring epilogue needs targets, stats and tlogit");
    TcArgs a = {};
    a.epi = EPI_SCORE; a.targets = targets; a.stats = (float4*)stats; a.tlogit = tlogit; a.status = status;
    return launch_tc(w, x_hi, x_lo, a, M, st);
}

int launch_gemm_q8_bf16x3(const QMat& w, const void* x_hi, const void* x_lo, const float* bias, const float* residual,
                          int epi, float* y, int M, int ldy, int* status, cudaStream_t st) {
    return launch_gemm_q8_bf16x3_ex(w, x_hi, x_lo, bias, residual, epi, y, nullptr, nullptr, M, ldy, status, st);
}

// scoring.rs:175-181 from the per-tile records of the fused head: a warp per row folds the records in tile
// order (lane l takes tiles l, l + 32, ...; the lanes are then merged pairwise in a fixed pattern), p =
// exp(target logit - max) / sum in f32, clamp_prob (loss.rs:12-18), ln in f64; greedy = the first column of the
// largest logit is the target.
__global__ void __launch_bounds__(256) score_combine_kernel(const float4* __restrict__ stats, const float* __restrict__ tlogit,
                                                            const int* __restrict__ targets, int M, int n_tiles, int V,
                                                            double* __restrict__ logprob, uint8_t* __restrict__ is_greedy) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const int target = targets[row];
    if (target < 0 || target >= V) {
        if (lane == 0) { logprob[row] = 0.0; is_greedy[row] = 0; }
        return;
    }
    float m = -INFINITY, s = 0.0f;
    int idx = 0x7fffffff;
    auto merge = [&](float m2, float s2, int i2) {
        const float M2 = fmaxf(m, m2);
        const float f1 = m > -INFINITY ? expf(m - M2) : 0.0f, f2 = m2 > -INFINITY ? expf(m2 - M2) : 0.0f;
        s = s * f1 + s2 * f2;
        idx = m2 > m ? i2 : (m > m2 ? idx : min(idx, i2));
        m = M2;
    };
    const float4* rec = stats + (size_t)row * n_tiles;
    for (int t = lane; t < n_tiles; t += 32) {
        const float4 r = rec[t];
        merge(r.x, r.y, __float_as_int(r.z));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        // both lanes of a pair fold (lower lane, upper lane) in that order, so that they agree bit for bit
        if (lane & o) {
            const float m1 = m, s1 = s;
            const int i1 = idx;
            m = m2; s = s2; idx = i2;
            merge(m1, s1, i1);
        } else {
            merge(m2, s2, i2);
        }
    }
    if (lane == 0) {
        float p = expf(tlogit[row] - m) / s;
        if (p == p) p = fmaxf(p, 1e-12f);
        logprob[row] = log((double)p);
        is_greedy[row] = (uint8_t)(idx == target);
    }
}

int launch_score_combine(const void* stats, const float* tlogit, const int* targets, int M, int n_tiles, int V, double* logprob,
                         uint8_t* is_greedy, cudaStream_t st) {
    score_combine_kernel<<<(M + 7) / 8, 256, 0, st>>>((const float4*)stats, tlogit, targets, M, n_tiles, V, logprob, is_greedy);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc

// =====================================================================================
// The allocation-free variant of the tensor-core linear
// =====================================================================================
// fc_q8_0_linear_dev needs scratch in global memory (the two bf16 planes the activations are
// split into, and a status word) and grows it with cudaMalloc. Here the same scratch is a
// file-scope device array of fixed size, so the call allocates nothing at all.
namespace {
constexpr size_t kStaticPlaneElems = (size_t)4 << 20;   // activations per call: M * K <= 4 Mi
// [hi plane | lo plane], 16 MiB per GPU that loads the library, held until the process exits.
static __device__ __align__(256) uint16_t g_noalloc_planes[2 * kStaticPlaneElems];
static __device__ __align__(256) int g_noalloc_status;

// Device addresses of the two arrays above, looked up once per device. In host code the names
// g_noalloc_planes / g_noalloc_status are only handles for cudaGetSymbolAddress: passing
// them to a kernel directly would hand it a host address.
struct NoAllocScratch {
    uint16_t* planes = nullptr;
    int* status = nullptr;
};
NoAllocScratch g_noalloc_dev[64];
}  // namespace

extern "C" int fc_q8_0_linear_dev_noalloc(const fc_qweight* w, const float* x_dev, const float* bias_dev, float* y_dev,
                                          int M, void* cuda_stream, int* timed_out) {
    using namespace fc;
    if (!w || !x_dev || !y_dev) return fail(FC_E_ARG, "fc_q8_0_linear_dev_noalloc: null argument");
    if (!aligned16(x_dev) || !aligned16(y_dev) || !aligned16(bias_dev))
        return fail(FC_E_ARG, "fc_q8_0_linear_dev_noalloc: x_dev, y_dev and bias_dev must be 16-byte aligned");
    if (M <= 0) return fail(FC_E_SHAPE, "fc_q8_0_linear_dev_noalloc: M = %d", M);
    int device = 0;
    const QMat* mat = qweight_matrix(w, &device);
    if (mat->K % 64) return fail(FC_E_SHAPE, "fc_q8_0_linear_dev_noalloc: K = %d is not a multiple of 64", mat->K);
    if ((size_t)M * mat->K > kStaticPlaneElems)
        return fail(FC_E_SHAPE, "fc_q8_0_linear_dev_noalloc: M * K = %zu exceeds the fixed scratch of %zu activations; "
                    "split the rows over several calls or use fc_q8_0_linear_dev", (size_t)M * mat->K, kStaticPlaneElems);
    if (device < 0 || device >= 64) return fail(FC_E_ARG, "fc_q8_0_linear_dev_noalloc: device %d out of range", device);
    FC_CUDA(cudaSetDevice(device));
    NoAllocScratch& sc = g_noalloc_dev[device];
    if (!sc.planes) {
        // set-up, first call on this device: resolve the device addresses of the static arrays
        void *p = nullptr, *s = nullptr;
        FC_CUDA(cudaGetSymbolAddress(&p, g_noalloc_planes));
        FC_CUDA(cudaGetSymbolAddress(&s, g_noalloc_status));
        sc.planes = (uint16_t*)p;
        sc.status = (int*)s;
    }
    cudaStream_t st = (cudaStream_t)cuda_stream;
    // the status word keeps whatever the previous call left in it: start from zero
    FC_CUDA(cudaMemsetAsync(sc.status, 0, sizeof(int), st));
    uint16_t* hi = sc.planes;
    uint16_t* lo = sc.planes + kStaticPlaneElems;
    FC_TRY(launch_split_bf16(x_dev, hi, lo, (size_t)M * mat->K, st));
    FC_TRY(launch_gemm_q8_bf16x3(*mat, hi, lo, bias_dev, nullptr, EPI_NONE, y_dev, M, mat->N, sc.status, st));
    if (timed_out) {
        FC_CUDA(cudaMemcpyAsync(timed_out, sc.status, sizeof(int), cudaMemcpyDeviceToHost, st));
        FC_CUDA(cudaStreamSynchronize(st));
        if (*timed_out != 0) return fail(FC_E_TIMEOUT, "a bounded wait inside the tensor-core GEMM ran out (status %d)", *timed_out);
    }
    return FC_OK;
}
