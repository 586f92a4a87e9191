// Causal multi-head attention of a full window on the tcgen05 tensor cores (head_dim 64).
//
// Replaces the per-(window, head) loop of TransformerBlock::forward
// (ferrum_core/src/layer/transformer.rs:395-477): S = Q Kᵀ / sqrt(hd), entries j > i masked,
// row softmax, O = P V. The T x T probability matrix the reference keeps (`last_attention`,
// transformer.rs:458-478) is never formed: keys are visited in tiles of 64 with an online
// softmax. Both products run as bf16 3-term splits with fp32 accumulation (q = qh + ql,
// k = kh + kl: qh·kh + ql·kh + qh·kl; the same for P·V), so they reproduce f32 products to
// 2^-16 relative.
//
// Inputs are the bf16 hi / lo planes of the fused qkv rows [R][3d] written by the QKV GEMM;
// the output is the pair of planes [R][d] the out-projection GEMM reads.
//
// One CTA owns 128 query rows of one (window, head); two CTAs fit on an SM, so one's
// softmax overlaps the other's MMAs.
//   warps 0-3   one query row per thread: tcgen05.ld the score tile, scale, mask, running
//               max / sum, write P (bf16 hi / lo, 128-byte swizzle) to shared memory, then
//               fold the P·V tile into the row's output registers;
//   warp 4      TMA: Q once, then a K tile and a V tile (64 keys) per step;
//   warp 5      tcgen05.mma issue: 12 MMAs for the score tile, 12 for P·V (V is consumed
//               MN-major, exactly as TMA lays out its [keys][hd] rows).
// Every mbarrier wait is bounded; on a timeout the status word is raised and the CTA leaves.
//
// Bound: tensor pipe / MUFU. 4·hd·T(T+1)/2 algorithmic FLOP per (window, head).
#include <cuda.h>
#include <cuda_bf16.h>

#include "fc_common.cuh"

namespace fc {

namespace {

constexpr int HD = 64;                 // head dimension
constexpr int QT = 128;                // query rows per CTA
constexpr int KT = 64;                 // keys per step
constexpr int Q_BYTES = QT * HD * 2;   // one bf16 plane of the Q tile: 16 KiB
constexpr int KV_BYTES = KT * HD * 2;  // one bf16 plane of a K or V tile: 8 KiB
constexpr int P_BYTES = QT * KT * 2;   // one bf16 plane of the P tile: 16 KiB
constexpr int OFF_Q = 0, OFF_K = OFF_Q + 2 * Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + 2 * KV_BYTES;
constexpr int OFF_BARS = OFF_P + 2 * P_BYTES;
constexpr int SOFTMAX_WARPS = 4, TMA_WARP = 4, MMA_WARP = 5, THREADS = 6 * 32;
constexpr int TMEM_COLS = 128;         // score tile: columns 0..63, P·V tile: columns 64..127
constexpr long long WAIT_CYCLES = 4000000000LL;
// bf16 x bf16 -> f32, M = 128, N = 64; B K-major for Q·Kᵀ, MN-major (bit 16) for P·V
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KT >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);
constexpr uint32_t IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(QT >> 4) << 24);

struct Bars {
    unsigned long long q_full, k_full, v_full, k_empty, v_empty;
    unsigned long long s_full, s_empty, p_full, o_full, o_empty;
    uint32_t tmem_base;
    volatile int abort;
};
constexpr int SMEM_BYTES = OFF_BARS + 1024 /* alignment slack */ + (int)sizeof(Bars);

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 2^x on the special-function unit (2 ulp); 2^-inf = 0
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
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
__device__ bool wait_bar(Bars* bars, unsigned long long* b, uint32_t parity, int* status) {
    const long long t0 = clock64();
    while (!mbar_try_wait(b, parity)) {
        if (bars->abort) return false;
        if (clock64() - t0 > WAIT_CYCLES) {
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
// 128-byte swizzle, 8-row atoms of 1024 bytes (SBO = 64 x 16 B), descriptor version 1. The same
// encoding serves K-major tiles (rows = M or N index) and the MN-major V tile (rows = keys).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)64 << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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
}
__device__ __forceinline__ void split2(float w0, float w1, uint32_t* hi, uint32_t* lo) {
    const __nv_bfloat162 h = __float22bfloat162_rn(make_float2(w0, w1));
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __float22bfloat162_rn(make_float2(w0 - hf.x, w1 - hf.y));
    *hi = *(const uint32_t*)&h;
    *lo = *(const uint32_t*)&l;
}

struct AttnArgs {
    int T;
    int k_col, v_col;            // first column of the key / value heads in the fused q | k | v planes
    int group;                   // query heads per key / value head (1: multi-head attention)
    int ldo;                     // row stride of the output planes (= query heads x 64)
    uint16_t *out_hi, *out_lo;   // [R][ldo] bf16 planes
    int* status;
};

}  // namespace

__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_hi, const __grid_constant__ CUtensorMap q_lo,
                       const __grid_constant__ CUtensorMap kv_hi, const __grid_constant__ CUtensorMap kv_lo, const AttnArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Bars* bars = (Bars*)(smem + OFF_BARS);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = (gridDim.x - 1) - blockIdx.x;          // long (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int row0 = b * a.T;                             // first row of the window in [R]
    const int q0 = qt * QT;                               // first query of the tile inside the window
    const int last_q = min(a.T, q0 + QT) - 1;             // last valid query
    const int n_kt = last_q / KT + 1;                     // key tiles 0..n_kt-1 cover keys 0..last_q

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        mbar_init(&bars->k_full, 1); mbar_init(&bars->v_full, 1);
        mbar_init(&bars->k_empty, 1); mbar_init(&bars->v_empty, 1);
        mbar_init(&bars->s_full, 1); mbar_init(&bars->s_empty, SOFTMAX_WARPS);
        mbar_init(&bars->p_full, SOFTMAX_WARPS);
        mbar_init(&bars->o_full, 1); mbar_init(&bars->o_empty, SOFTMAX_WARPS);
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&bars->tmem_base)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars->tmem_base;

    if (warp == TMA_WARP) {
        if (lane == 0) {
            mbar_expect_tx(&bars->q_full, 2 * Q_BYTES);
            tma_load_2d(smem + OFF_Q, &q_hi, h * HD, row0 + q0, &bars->q_full);
            tma_load_2d(smem + OFF_Q + Q_BYTES, &q_lo, h * HD, row0 + q0, &bars->q_full);
            for (int kt = 0; kt < n_kt; ++kt) {
                const uint32_t par = (kt & 1) ^ 1;
                if (!wait_bar(bars, &bars->k_empty, par, a.status)) break;
                mbar_expect_tx(&bars->k_full, 2 * KV_BYTES);
                tma_load_2d(smem + OFF_K, &kv_hi, a.k_col + (h / a.group) * HD, row0 + kt * KT, &bars->k_full);
                tma_load_2d(smem + OFF_K + KV_BYTES, &kv_lo, a.k_col + (h / a.group) * HD, row0 + kt * KT, &bars->k_full);
                if (!wait_bar(bars, &bars->v_empty, par, a.status)) break;
                mbar_expect_tx(&bars->v_full, 2 * KV_BYTES);
                tma_load_2d(smem + OFF_V, &kv_hi, a.v_col + (h / a.group) * HD, row0 + kt * KT, &bars->v_full);
                tma_load_2d(smem + OFF_V + KV_BYTES, &kv_lo, a.v_col + (h / a.group) * HD, row0 + kt * KT, &bars->v_full);
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            const uint32_t sb = s32(smem);
            const uint64_t qh = smem_desc(sb + OFF_Q), ql = smem_desc(sb + OFF_Q + Q_BYTES);
            const uint64_t kh = smem_desc(sb + OFF_K), kl = smem_desc(sb + OFF_K + KV_BYTES);
            const uint64_t vh = smem_desc(sb + OFF_V), vl = smem_desc(sb + OFF_V + KV_BYTES);
            const uint64_t ph = smem_desc(sb + OFF_P), pl = smem_desc(sb + OFF_P + P_BYTES);
            bool ok = wait_bar(bars, &bars->q_full, 0, a.status);
            // score tile kt: its keys have landed and the softmax warps have read the previous one out of TMEM
            auto issue_scores = [&](int kt) -> bool {
                const uint32_t par = kt & 1;
                if (!(wait_bar(bars, &bars->k_full, par, a.status) && wait_bar(bars, &bars->s_empty, par ^ 1, a.status))) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks) {
                    const uint64_t adv = (uint64_t)(ks * 2);                 // 32 bytes along hd
                    umma(tmem, qh + adv, kh + adv, IDESC_S, ks != 0);
                    umma(tmem, ql + adv, kh + adv, IDESC_S, 1);
                    umma(tmem, qh + adv, kl + adv, IDESC_S, 1);
                }
                umma_commit(&bars->s_full);
                umma_commit(&bars->k_empty);
                return true;
            };
            ok = ok && issue_scores(0);
            for (int kt = 0; kt < n_kt && ok; ++kt) {
                const uint32_t par = kt & 1;
                // the next score tile is issued ahead of this tile's P·V: its MMAs run while the softmax warps are
                // still turning this tile's scores into P, and its scores are ready when they come back
                if (kt + 1 < n_kt) {
                    ok = issue_scores(kt + 1);
                    if (!ok) break;
                }
                // P·V tile: P is in shared memory, the previous P·V tile has been folded in
                ok = wait_bar(bars, &bars->v_full, par, a.status) && wait_bar(bars, &bars->p_full, par, a.status) &&
                     wait_bar(bars, &bars->o_empty, par ^ 1, a.status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int ks = 0; ks < KT / 16; ++ks) {
                    const uint64_t pa = (uint64_t)(ks * 2);                  // 32 bytes along the keys of a P row
                    const uint64_t va = (uint64_t)(ks * 128);                // 16 key rows of 128 bytes
                    umma(tmem + HD, ph + pa, vh + va, IDESC_O, ks != 0);
                    umma(tmem + HD, pl + pa, vh + va, IDESC_O, 1);
                    umma(tmem + HD, ph + pa, vl + va, IDESC_O, 1);
                }
                umma_commit(&bars->o_full);
                umma_commit(&bars->v_empty);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps
        const int r = warp * 32 + lane;               // query row inside the tile
        const int qi = q0 + r;                        // query index inside the window
        const float c2 = 0.125f * 1.4426950408889634f;   // 1 / sqrt(64) times log2(e)
        float o[HD];
#pragma unroll
        for (int c = 0; c < HD; ++c) o[c] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        unsigned char* prow_hi = smem + OFF_P + r * 128;
        unsigned char* prow_lo = prow_hi + P_BYTES;
        const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
        bool ok = true;
        for (int kt = 0; kt < n_kt && ok; ++kt) {
            const uint32_t par = kt & 1;
            ok = wait_bar(bars, &bars->s_full, par, a.status);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t s0[32], s1[32];
            tmem_ld32(lane_addr, s0);
            tmem_ld32(lane_addr + 32, s1);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->s_empty);
            // causal mask (key j > query i has weight exactly 0) and running max on the raw scores; the scale
            // 1 / sqrt(hd) and log2(e) go into one constant of the exponent: p = 2^((s - max) * scale * log2 e)
            const int k0 = kt * KT;
            float sv[KT];
            float tmax = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                sv[j] = (k0 + j <= qi) ? __uint_as_float(s0[j]) : -INFINITY;
                sv[32 + j] = (k0 + 32 + j <= qi) ? __uint_as_float(s1[j]) : -INFINITY;
                tmax = fmaxf(tmax, fmaxf(sv[j], sv[32 + j]));
            }
            const float mn = fmaxf(m, tmax);          // finite from the first tile on (key 0 <= every query)
            const float corr = exp2f((m - mn) * c2);
            const float off2 = -mn * c2;
            float psum = 0.0f;
#pragma unroll
            for (int c = 0; c < KT / 8; ++c) {        // 16-byte chunk c of the P row: 8 keys
                uint4 hi, lo;
                float p[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) { p[e] = ex2_approx(fmaf(sv[8 * c + e], c2, off2)); psum += p[e]; }
                split2(p[0], p[1], &hi.x, &lo.x);
                split2(p[2], p[3], &hi.y, &lo.y);
                split2(p[4], p[5], &hi.z, &lo.z);
                split2(p[6], p[7], &hi.w, &lo.w);
                const int chunk = (c ^ (r & 7)) * 16;  // 128-byte swizzle
                *(uint4*)(prow_hi + chunk) = hi;
                *(uint4*)(prow_lo + chunk) = lo;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_full);
            l = fmaf(l, corr, psum);
            m = mn;
            if (__any_sync(0xffffffffu, corr != 1.0f)) {   // the running max moves in the first tiles and rarely after
#pragma unroll
                for (int c = 0; c < HD; ++c) o[c] *= corr;
            }
            // fold in this tile's P·V
            ok = wait_bar(bars, &bars->o_full, par, a.status);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tmem_ld32(lane_addr + HD, s0);
            tmem_ld32(lane_addr + HD + 32, s1);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->o_empty);
#pragma unroll
            for (int c = 0; c < 32; ++c) { o[c] += __uint_as_float(s0[c]); o[32 + c] += __uint_as_float(s1[c]); }
        }
        if (ok && qi < a.T) {
            const float inv = 1.0f / l;
            const size_t off = (size_t)(row0 + qi) * a.ldo + (size_t)h * HD;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                uint4 hi, lo;
                split2(o[8 * c] * inv, o[8 * c + 1] * inv, &hi.x, &lo.x);
                split2(o[8 * c + 2] * inv, o[8 * c + 3] * inv, &hi.y, &lo.y);
                split2(o[8 * c + 4] * inv, o[8 * c + 5] * inv, &hi.z, &lo.z);
                split2(o[8 * c + 6] * inv, o[8 * c + 7] * inv, &hi.w, &lo.w);
                *(uint4*)(a.out_hi + off + 8 * c) = hi;
                *(uint4*)(a.out_lo + off + 8 * c) = lo;
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

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A [rows][cols] bf16 plane viewed through boxes of 64 columns x box_rows rows, 128-byte swizzle.
int encode(CUtensorMap* map, const void* plane, size_t rows, size_t cols, int box_rows) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        FC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) return fail(FC_E_CUDA, "cuTensorMapEncodeTiled is not available");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)plane, dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FC_E_CUDA, "cuTensorMapEncodeTiled failed (%d) for a [%zu][%zu] bf16 plane", (int)r, rows, cols);
    return FC_OK;
}
}  // namespace

// qkv_hi / qkv_lo: bf16 planes [B*T][H*64 + 2*KV*64] (q heads | k heads | v heads per row);
// out_hi / out_lo: planes [B*T][H*64]. Query head h reads key / value head h / (H / KV).
int launch_attn_prefill_tc_gqa(const void* qkv_hi, const void* qkv_lo, int B, int T, int H, int KV, void* out_hi, void* out_lo,
                               int* status, cudaStream_t st) {
    if (KV <= 0 || H % KV) return fail(FC_E_DIM, "n_heads %d must be a multiple of n_kv_heads %d", H, KV);
    static bool attr_set[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        FC_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set[dev] = true;
    }
    const size_t R = (size_t)B * T, ld = (size_t)(H + 2 * KV) * HD;
    CUtensorMap qh, ql, kh, kl;
    FC_TRY(encode(&qh, qkv_hi, R, ld, QT));
    FC_TRY(encode(&ql, qkv_lo, R, ld, QT));
    FC_TRY(encode(&kh, qkv_hi, R, ld, KT));
    FC_TRY(encode(&kl, qkv_lo, R, ld, KT));
    AttnArgs a;
    a.T = T; a.k_col = H * HD; a.v_col = (H + KV) * HD; a.group = H / KV; a.ldo = H * HD;
    a.out_hi = (uint16_t*)out_hi; a.out_lo = (uint16_t*)out_lo; a.status = status;
    dim3 grid((T + QT - 1) / QT, H, B);
    attn_prefill_tc_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(qh, ql, kh, kl, a);
    FC_LAUNCHED();
    return FC_OK;
}

// The multi-head form: planes [B*T][3d] in, [B*T][d] out.
int launch_attn_prefill_tc(const void* qkv_hi, const void* qkv_lo, int B, int T, int d, int H, void* out_hi, void* out_lo,
                           int* status, cudaStream_t st) {
    if (d != H * HD) return fail(FC_E_SHAPE, "tensor-core attention needs head_dim 64 (d = %d, H = %d)", d, H);
    return launch_attn_prefill_tc_gqa(qkv_hi, qkv_lo, B, T, H, H, out_hi, out_lo, status, st);
}

}  // namespace fc
