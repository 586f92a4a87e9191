// Lock-step decode of many streams: the kernels of one KV-cached step for S streams at once.
//
// Replaces S independent runs of CachedTransformer::feed (ferrum_core/src/slm/cached.rs:100-125)
// -> TransformerBlock::forward_with_cache (layer/transformer.rs:221-294): every stream has its
// own KV caches and window, all streams sit at the same position, and each Q8_0 matrix is read
// from HBM ONCE per step for all of them.
//
// The linear layers are skinny products Y[S][N] = X[S][K] · Wᵀ with S <= 64 rows. They run on the
// warp-level tensor-core path (mma.sync m16n8k16, f16 operands, f32 accumulate) arranged so that
// the result is as exact as the reference's f32 arithmetic:
//   * the A operand is the int8 quant level itself (|q| <= 127 is exact in f16), 16 weight rows
//     per warp; the f16 block scale multiplies the f32 sum of each 32-wide Q8_0 block afterwards,
//     so no rounding of d*q ever happens (gguf/dequant.rs:37-49 forms d*q in f32; here the same
//     real product is distributed over the sum);
//   * the B operand holds every activation as two f16 terms x = hi + lo (22 significant bits),
//     in two adjacent columns, so one accumulator pair per stream sums to the f32-equivalent dot
//     product;
//   * the weights are read from a fragment-major copy made at upload: per (16 rows, 32-wide block)
//     512 contiguous bytes in lane order plus 32 bytes of scales — Q8_0's own 34 B per 32 weights,
//     every warp load a full 512-byte line.
// A CTA owns 16 or 32 output rows; its warps split K and add their partial sums through shared memory
// in warp order (deterministic). Attention reads each stream's f32 cache rows once; the greedy
// pick is token_stream.rs:134 + sampling.rs:96-104 per stream. More than 16 streams run as groups of 16
// whose kernel chains are parallel branches of the step's CUDA graph (the caller's side).
//
// Bound: HBM. Per step: every Q8_0 matrix once + per stream the f32 K/V rows of positions 0..pos.
#include <cuda_fp16.h>

#include <algorithm>

#include "fc_common.cuh"

namespace fc {

namespace {

constexpr int RED_LD = 33;

// Programmatic dependent launch: every kernel of the step is launched as a dependent of the one
// ahead of it. It may start (and fetch what no kernel writes: weights) while that kernel still
// runs; pdl_wait_prior() returns once the kernel ahead has completed and its writes are visible.
// Every kernel executes the wait on every path before it touches step data, so completion stays
// transitive along the chain. Both calls are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// bytes (b0, b1) of w (biased quants q + 128) -> two exact f16 values (q0, q1): 0x6400 | b is
// 1024 + b, and 1152 = 1024 + 128 is subtracted.
template <int HI>
__device__ __forceinline__ uint32_t q2h(uint32_t w) {
    const uint32_t r = __byte_perm(w, 0x64646464u, HI ? 0x4342 : 0x4140);
    const __half2 h = __hsub2(*(const __half2*)&r, __halves2half2(__ushort_as_half((unsigned short)0x6480), __ushort_as_half((unsigned short)0x6480)));
    return *(const uint32_t*)&h;
}
__device__ __forceinline__ void mma16816(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

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

struct SkArgs {
    const uint4* wq;        // fragment-major quants: [row group][k-block][32 lanes] x 16 B
    const __half2* wd;      // scales: [row group][k-block][8] pairs (row g, row g + 8)
    int N, K, S;
    int depth;              // ring slots per warp (k-blocks in flight), <= SK_DEPTH
    // ---- input: f16 hi / lo rows [cols][K] (row 2s = hi, 2s + 1 = lo of stream s)
    const uint4* xp;
    // ---- output
    const float* bias;      // [N] or null
    int epi;                // EPI_NONE / EPI_GELU
    const float* residual;  // [S][ldy] or null: y = residual + (product + bias); may be y itself
    float* y;               // f32 rows [S][ldy], or null
    int ldy;
    __half* yp;             // f16 hi / lo rows [cols][ldp], or null
    int ldp;
    float* part_out;        // raw sums of this CTA's K range [gridDim.z][S][N] (no bias), or null
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Waits until at most n (< 16) of this thread's cp.async groups are still in flight.
__device__ __forceinline__ void cp_async_wait_n(int n) {
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<5>(); break;
        case 6: cp_async_wait<6>(); break;
        case 7: cp_async_wait<7>(); break;
        case 8: cp_async_wait<8>(); break;
        case 9: cp_async_wait<9>(); break;
        case 10: cp_async_wait<10>(); break;
        case 11: cp_async_wait<11>(); break;
        case 12: cp_async_wait<12>(); break;
        case 13: cp_async_wait<13>(); break;
        case 14: cp_async_wait<14>(); break;
        default: cp_async_wait<15>(); break;
    }
}

constexpr int SK_DEPTH = 16;       // most k-blocks of weights a warp keeps in flight
constexpr int SK_MAX_SPLITS = 8;

// NT: 8-column MMA tiles (4 streams each) per warp; RG: 16-row groups per warp. blockIdx.x picks the rows,
// blockIdx.y the group of 8 * NT activation columns, blockIdx.z the K range (products whose K ranges are split over
// CTAs leave partial sums that the consumer adds in range order).
//
// Weights never depend on the kernel ahead, so every warp requests the first blocks of its K slice
// (its own ring in shared memory, cp.async) before it waits for that kernel (programmatic dependent
// launch): the weight stream of one product overlaps the tail of the kernel before it, and HBM sees
// RG * 544 B * depth per warp in flight instead of one block at a time.
// MAXT: the largest block the instance is launched with (512, or 1024 for the narrow tiles whose registers allow it).
template <int NT, int RG, int MAXT = 512>
__global__ void __launch_bounds__(MAXT) skinny_q8_kernel(const SkArgs a) {
    extern __shared__ __align__(16) unsigned char sk_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nwarps = blockDim.x >> 5;
    constexpr int SLOT = RG * 544;                     // per 16-row group: 512 B quants + 32 B scales
    const int depth = a.depth;
    unsigned char* ring = sk_smem + (size_t)warp * depth * SLOT;
    float* red = (float*)(sk_smem + (size_t)nwarps * depth * SLOT);   // [warps][4 * NT streams][RED_LD]
    const int nkb = a.K >> 5, k8 = a.K >> 3;
    const int kbA = (int)((long long)blockIdx.z * nkb / gridDim.z), kbB = (int)((long long)(blockIdx.z + 1) * nkb / gridDim.z);
    const int kb0 = kbA + (int)((long long)warp * (kbB - kbA) / nwarps), kb1 = kbA + (int)((long long)(warp + 1) * (kbB - kbA) / nwarps);
    const int rg0 = blockIdx.x * RG;
    const int col0 = blockIdx.y * (8 * NT);           // first activation column of this CTA
    const uint4* wq = a.wq + ((size_t)rg0 * nkb) * 32 + lane;
    const uint4* wd4 = (const uint4*)(a.wd + ((size_t)rg0 * nkb) * 8);   // 32 B of scales per (row group, k-block)
    int slot_w = 0;                                    // ring slot the next request fills
    auto request = [&](int kb) {
        unsigned char* slot = ring + (size_t)slot_w * SLOT;
#pragma unroll
        for (int r = 0; r < RG; ++r) {
            cp_async16(slot + r * 544 + lane * 16, wq + ((size_t)r * nkb + kb) * 32);
            if (lane < 2) cp_async16(slot + r * 544 + 512 + lane * 16, wd4 + ((size_t)r * nkb + kb) * 2 + lane);
        }
        slot_w = slot_w + 1 == depth ? 0 : slot_w + 1;
    };
#pragma unroll 1
    for (int i = 0; i < depth; ++i) {                  // one group per block, empty ones included: block i is group i
        if (kb0 + i < kb1) request(kb0 + i);
        cp_async_commit();
    }
    pdl_wait_prior();                                  // the activations come from the kernel ahead
    pdl_launch_next();                                 // the kernel behind may start fetching its own weights

    // bias and residual of the output this thread finishes first are requested now, so that they have arrived when
    // the K loop ends
    constexpr int ROWS = 16 * RG;
    const int n_base = blockIdx.x * ROWS, s_base = col0 >> 1;
    const int s_here = min(4 * NT, a.S - s_base);
    float bias0 = 0.0f, res0 = 0.0f;
    {
        const int sl = threadIdx.x / ROWS, n = n_base + (threadIdx.x - sl * ROWS);
        if (sl < s_here && n < a.N && !a.part_out) {
            if (a.bias) bias0 = __ldg(a.bias + n);
            if (a.residual) res0 = a.residual[(size_t)(s_base + sl) * a.ldy + n];
        }
    }
    float acc[RG][NT][2];
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int j = 0; j < NT; ++j) acc[r][j][0] = acc[r][j][1] = 0.0f;
    const uint4* xb = a.xp + (size_t)(col0 + g) * k8 + t;
    auto fetch_x = [&](uint4 (&xv)[NT], int kb) {
#pragma unroll
        for (int j = 0; j < NT; ++j) xv[j] = __ldg(xb + (size_t)(8 * j) * k8 + 4 * kb);
    };
    auto fetch_w = [&](uint4 (&w)[RG], float2 (&sc)[RG], const unsigned char* slot) {
#pragma unroll
        for (int r = 0; r < RG; ++r) {
            w[r] = *(const uint4*)(slot + r * 544 + lane * 16);
            sc[r] = __half22float2(*(const __half2*)(slot + r * 544 + 512 + g * 4));
        }
    };
    // one k-block: 32 k of RG * 16 rows against 4 * NT streams
    auto block_math = [&](const uint4 (&xv)[NT], const uint4 (&w)[RG], const float2 (&sc)[RG]) {
        // lane (g, t) holds k = 8t .. 8t+7 of rows g (x, y) and g + 8 (z, w): k-step 0 takes the
        // first four, k-step 1 the last four, on both operands alike
        uint32_t A[RG][2][4];
#pragma unroll
        for (int r = 0; r < RG; ++r) {
            A[r][0][0] = q2h<0>(w[r].x); A[r][0][2] = q2h<1>(w[r].x); A[r][0][1] = q2h<0>(w[r].z); A[r][0][3] = q2h<1>(w[r].z);
            A[r][1][0] = q2h<0>(w[r].y); A[r][1][2] = q2h<1>(w[r].y); A[r][1][1] = q2h<0>(w[r].w); A[r][1][3] = q2h<1>(w[r].w);
        }
        // the MMAs of up to four column tiles are issued back to back (independent accumulators), and only then are
        // their block sums scaled and added: the tensor pipe's latency is covered by the MMAs behind, not waited for
        constexpr int JB = NT < 4 ? NT : 4;
#pragma unroll
        for (int j0 = 0; j0 < NT; j0 += JB) {
            float d[JB][RG][4];
#pragma unroll
            for (int jj = 0; jj < JB; ++jj)
#pragma unroll
                for (int r = 0; r < RG; ++r) {
                    d[jj][r][0] = d[jj][r][1] = d[jj][r][2] = d[jj][r][3] = 0.0f;
                    mma16816(d[jj][r], A[r][0][0], A[r][0][1], A[r][0][2], A[r][0][3], xv[j0 + jj].x, xv[j0 + jj].y);
                }
#pragma unroll
            for (int jj = 0; jj < JB; ++jj)
#pragma unroll
                for (int r = 0; r < RG; ++r)
                    mma16816(d[jj][r], A[r][1][0], A[r][1][1], A[r][1][2], A[r][1][3], xv[j0 + jj].z, xv[j0 + jj].w);
#pragma unroll
            for (int jj = 0; jj < JB; ++jj)
#pragma unroll
                for (int r = 0; r < RG; ++r) {
                    acc[r][j0 + jj][0] = fmaf(sc[r].x, d[jj][r][0] + d[jj][r][1], acc[r][j0 + jj][0]);
                    acc[r][j0 + jj][1] = fmaf(sc[r].y, d[jj][r][2] + d[jj][r][3], acc[r][j0 + jj][1]);
                }
        }
    };
    if (kb1 - kb0 <= depth) {
        // The whole K slice of the warp is in its ring (every shape of the models here): one wait for all of it, and
        // then a loop without waits or refills, which the compiler is free to overlap across k-blocks. (A wait on
        // the copy groups also holds back until the loads issued before it have returned, activation fragments
        // included: per k-block it costs an L2 round trip.)
        cp_async_wait<0>();
        __syncwarp();
#pragma unroll 2
        for (int i = 0; i < kb1 - kb0; ++i) {
            uint4 xv[NT], w[RG];
            float2 sc[RG];
            fetch_x(xv, kb0 + i);
            fetch_w(w, sc, ring + (size_t)i * SLOT);
            block_math(xv, w, sc);
        }
    } else {
        int slot_r = 0;
        for (int kb = kb0; kb < kb1; ++kb) {
            uint4 xv[NT], w[RG];
            float2 sc[RG];
            fetch_x(xv, kb);
            cp_async_wait_n(depth - 1);                // block kb has landed: depth + i groups committed, the first i + 1 complete
            __syncwarp();
            fetch_w(w, sc, ring + (size_t)slot_r * SLOT);
            slot_r = slot_r + 1 == depth ? 0 : slot_r + 1;
            __syncwarp();                              // every lane has read the slot before it is refilled
            if (kb + depth < kb1) request(kb + depth);
            cp_async_commit();
            block_math(xv, w, sc);
        }
    }
    cp_async_wait<0>();
    // partial sums of this warp's K slice: red[warp][stream][row]
    float* mine = red + (size_t)warp * (4 * NT) * RED_LD;
    static_assert(ROWS <= RED_LD, "reduction rows");
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        float* col = mine + (4 * j + t) * RED_LD;
#pragma unroll
        for (int r = 0; r < RG; ++r) { col[16 * r + g] = acc[r][j][0]; col[16 * r + g + 8] = acc[r][j][1]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < s_here * ROWS; idx += blockDim.x) {
        const int sl = idx / ROWS, r = idx - sl * ROWS, n = n_base + r, s = s_base + sl;
        if (n >= a.N) continue;
        float v = 0.0f;
        for (int w = 0; w < nwarps; ++w) v += red[((size_t)w * (4 * NT) + sl) * RED_LD + r];   // K slices in order
        if (a.part_out) {
            a.part_out[((size_t)blockIdx.z * a.S + s) * a.N + n] = v;
            continue;
        }
        const bool first = idx == (int)threadIdx.x;
        if (a.bias) v += first ? bias0 : a.bias[n];
        if (a.epi == EPI_GELU) v = gelu_f(v);
        if (a.residual) v = (first ? res0 : a.residual[(size_t)s * a.ldy + n]) + v;
        if (a.y) a.y[(size_t)s * a.ldy + n] = v;
        if (a.yp) {
            const __half h = __float2half_rn(v);
            a.yp[(size_t)(2 * s) * a.ldp + n] = h;
            a.yp[(size_t)(2 * s + 1) * a.ldp + n] = __float2half_rn(v - __half2float(h));
        }
    }
}

// Fragment-major copy of one matrix: thread = (row group, k-block, lane).
__global__ void repack_frag_kernel(const uint8_t* __restrict__ qu, const __half* __restrict__ d, int N_pad, int K,
                                   uint4* __restrict__ fq, __half2* __restrict__ fd) {
    const int nkb = K >> 5;
    const size_t total = (size_t)(N_pad >> 4) * nkb * 32;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int lane = (int)(i & 31), g = lane >> 2, t = lane & 3;
        const size_t blk = i >> 5, rg = blk / nkb;
        const int kb = (int)(blk - rg * nkb);
        const size_t r0 = rg * 16 + g, r1 = r0 + 8;
        const uint2 lo = *(const uint2*)(qu + r0 * K + (size_t)kb * 32 + 8 * t);
        const uint2 hi = *(const uint2*)(qu + r1 * K + (size_t)kb * 32 + 8 * t);
        fq[i] = make_uint4(lo.x, lo.y, hi.x, hi.y);
        if (t == 0) fd[blk * 8 + g] = __halves2half2(d[r0 * nkb + kb], d[r1 * nkb + kb]);
    }
}

// Fixed-order block reductions; `red` has >= 33 floats.
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

// layer/embedding.rs:70-90 for S streams at one position: x[s] = tok[cur[s]] + pos[*pos].
__global__ void embed_batch_kernel(QMat tok, const float* __restrict__ pos_emb, const int* __restrict__ cur, const int* __restrict__ pos,
                                   float* __restrict__ x) {
    pdl_wait_prior();
    pdl_launch_next();
    const int s = blockIdx.x, p = *pos;
    const int id = min(max(cur[s], 0), tok.N - 1);   // the pick only hands on ids below the vocabulary size; never index outside the table
    const int d = tok.K;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float dq = __half2float(tok.d[(size_t)id * (d >> 5) + (c >> 5)]);
        const int q = (int)tok.qu[(size_t)id * d + c] - 128;
        x[(size_t)s * d + c] = dq * (float)q + pos_emb[(size_t)p * d + c];
    }
}

// layer/norm.rs:46-82 per stream row, written as the f16 hi / lo rows the skinny product reads. When
// the product ahead left K-split partial sums, the row is first completed: x_new = x + (sum of the
// n_part partials in order + part_bias), stored to x_out (the residual add of transformer.rs:272,293).
template <int PER>
__global__ void ln_rows_f16_kernel(const float* __restrict__ x, const float* __restrict__ part, int n_part, int S,
                                   const float* __restrict__ part_bias, float* __restrict__ x_out, const float* __restrict__ g,
                                   const float* __restrict__ b, int d, __half* __restrict__ xp) {
    __shared__ float red[33];
    // gain, bias and the pending product's bias do not depend on the kernel ahead: they are on their way while this
    // kernel waits for it
    float gv[PER], bv[PER], pbv[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        gv[i] = __ldg(g + min(c, d - 1));
        bv[i] = __ldg(b + min(c, d - 1));
        pbv[i] = (n_part > 0 && part_bias) ? __ldg(part_bias + min(c, d - 1)) : 0.0f;
    }
    pdl_wait_prior();
    pdl_launch_next();
    const int s = blockIdx.x;
    const float* xr = x + (size_t)s * d;
    // Loads are clamped, not guarded: a guarded load per iteration puts a branch between the loads and they go out one
    // L2 round trip at a time; unguarded they are all in flight together.
    float v[PER];
    float sum = 0.0f;
    if (n_part > 0) {
        constexpr int CH = PER < 4 ? PER : 4;      // columns per thread whose loads are in flight together
#pragma unroll
        for (int i0 = 0; i0 < PER; i0 += CH) {
            float pp[CH][SK_MAX_SPLITS];
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int c = min((int)(threadIdx.x + (i0 + k) * blockDim.x), d - 1);
                v[i0 + k] = xr[c];
#pragma unroll
                for (int p = 0; p < SK_MAX_SPLITS; ++p) pp[k][p] = part[((size_t)min(p, n_part - 1) * S + s) * d + c];
            }
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int i = i0 + k, c = threadIdx.x + i * blockDim.x;
                float pv = pp[k][0];               // the partials are added in order
#pragma unroll
                for (int p = 1; p < SK_MAX_SPLITS; ++p) pv = p < n_part ? pv + pp[k][p] : pv;
                if (part_bias) pv += pbv[i];
                const float xv = c < d ? v[i] + pv : 0.0f;
                if (c < d && x_out) x_out[(size_t)s * d + c] = xv;
                v[i] = xv;
                sum += xv;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) v[i] = xr[min((int)(threadIdx.x + i * blockDim.x), d - 1)];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            if ((int)(threadIdx.x + i * blockDim.x) >= d) v[i] = 0.0f;
            sum += v[i];
        }
    }
    const float mean = block_sum(sum, red) / (float)d;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        const float t = v[i] - mean;
        q += c < d ? t * t : 0.0f;
    }
    const float sd = sqrtf(block_sum(q, red) / (float)d + 1e-5f);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < d) {
            const float y = ((v[i] - mean) / sd) * gv[i] + bv[i];
            const __half h = __float2half_rn(y);
            xp[(size_t)(2 * s) * d + c] = h;
            xp[(size_t)(2 * s + 1) * d + c] = __float2half_rn(y - __half2float(h));
        }
    }
}

// layer/transformer.rs:246-283 for (head h, stream s): the step's k and v rows are appended to
// the stream's cache at *pos, scores over the pos + 1 cached rows (dot ascending over hd, times
// 1/sqrt(hd)), softmax (max, exp, sum), out = sum_j (e_j / sum) v_j. hd <= 64, hd % 4 == 0.
// Output: f16 hi / lo rows of the attention output for the out-projection.
__global__ void __launch_bounds__(256) attn_decode_batch_kernel(const float* __restrict__ qkv, float* const* __restrict__ kcs,
                                                                float* const* __restrict__ vcs, size_t layer_off, int d, int hd,
                                                                const int* __restrict__ pos, __half* __restrict__ ap) {
    extern __shared__ float sm[];   // scores[len] | red[64] | part[16][64]
    // The position and the cached rows of earlier steps were written at least two kernels ago (a kernel is only
    // launched once the one ahead of it has passed its own dependency wait), so they can be touched before this
    // kernel's wait: the head's slices of the cached k and v rows are asked into L2 while the QKV product runs.
    const int h = blockIdx.x, s = blockIdx.y, hs = h * hd;
    const int p = *pos, len = p + 1;
    float* kc = kcs[s] + layer_off;
    float* vc = vcs[s] + layer_off;
    for (int i = threadIdx.x; i < 4 * p; i += blockDim.x) {   // 128 B lines: two per row slice of up to 64 floats, k and v
        const int j = i >> 2, part_i = i & 3;
        const float* base = (part_i & 2 ? vc : kc) + (size_t)j * d + hs + (part_i & 1) * 32;
        if ((part_i & 1) * 32 < hd) asm volatile("prefetch.global.L2 [%0];" ::"l"(base));
    }
    pdl_wait_prior();
    pdl_launch_next();
    float* sc = sm;
    float* red = sm + ((len + 3) & ~3);
    float* part = red + 64;
    const float* row = qkv + (size_t)s * 3 * d;
    // the step's own k and v rows go to the cache; this kernel reads them from the QKV product's output instead
    if (threadIdx.x < hd) {
        kc[(size_t)p * d + hs + threadIdx.x] = row[d + hs + threadIdx.x];
        vc[(size_t)p * d + hs + threadIdx.x] = row[2 * d + hs + threadIdx.x];
    }
    const int hw = threadIdx.x >> 4, li = threadIdx.x & 15;
    const bool has = 4 * li < hd;
    const int lic = has ? li : 0;                  // a lane past the head width reads lane 0's columns and drops them
    const float4 z4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float4 q = has ? *(const float4*)(row + hs + 4 * li) : z4;
    const float scale = 1.0f / sqrtf((float)hd);
    float mx = -INFINITY;
    // a half warp per cached row: lane li owns dimensions 4 li .. 4 li + 3, eight rows in flight. The two halves of
    // a warp may run different numbers of rows, so the shuffles name only the lanes of their own half.
    const unsigned hmask = 0xFFFFu << (threadIdx.x & 16);
    constexpr int UK = 8;
    for (int j0 = hw; j0 < len; j0 += 16 * UK) {
        float dot[UK];
        float4 kq[UK];
#pragma unroll
        for (int u = 0; u < UK; ++u) {
            const int j = j0 + 16 * u;
            const int jc = min(j, len - 1);            // clamped, not guarded: all eight loads are in flight together
            const float* kr = jc == p ? row + d : kc + (size_t)jc * d;
            kq[u] = *(const float4*)(kr + hs + 4 * lic);
        }
#pragma unroll
        for (int u = 0; u < UK; ++u) {
            const float4 kk = (j0 + 16 * u < len && has) ? kq[u] : z4;
            dot[u] = fmaf(q.w, kk.w, fmaf(q.z, kk.z, fmaf(q.y, kk.y, q.x * kk.x)));
        }
#pragma unroll
        for (int sh = 8; sh > 0; sh >>= 1)
#pragma unroll
            for (int u = 0; u < UK; ++u) dot[u] += __shfl_xor_sync(hmask, dot[u], sh);
#pragma unroll
        for (int u = 0; u < UK; ++u) {
            const int j = j0 + 16 * u;
            if (j < len) {
                const float v = dot[u] * scale;
                if (li == 0) sc[j] = v;
                mx = fmaxf(mx, v);
            }
        }
    }
    mx = block_max(mx, red);
    float e = 0.0f;
    for (int j = threadIdx.x; j < len; j += blockDim.x) {
        const float t = expf(sc[j] - mx);
        sc[j] = t;
        e += t;
    }
    const float sum = block_sum(e, red);
    // out: every half warp adds up its own rows (lane li: dimensions 4 li .. 4 li + 3, four rows in
    // flight), then the 16 partial rows are added in half-warp order
    float4 o = z4;
    for (int j0 = hw; j0 < len; j0 += 64) {
        float4 vv[4];
        float pj[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + 16 * u;
            const int jc = min(j, len - 1);
            const float* vr = jc == p ? row + 2 * d : vc + (size_t)jc * d;
            vv[u] = *(const float4*)(vr + hs + 4 * lic);
            pj[u] = (j < len && has) ? sc[jc] / sum : 0.0f;   // rows past the end and lanes past the head weigh 0
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            o.x = fmaf(pj[u], vv[u].x, o.x); o.y = fmaf(pj[u], vv[u].y, o.y);
            o.z = fmaf(pj[u], vv[u].z, o.z); o.w = fmaf(pj[u], vv[u].w, o.w);
        }
    }
    if (has) *(float4*)(part + hw * 64 + 4 * li) = o;
    __syncthreads();
    if (threadIdx.x < hd) {
        float acc = 0.0f;
#pragma unroll
        for (int gg = 0; gg < 16; ++gg) acc += part[gg * 64 + threadIdx.x];
        const __half hi = __float2half_rn(acc);
        ap[(size_t)(2 * s) * d + hs + threadIdx.x] = hi;
        ap[(size_t)(2 * s + 1) * d + hs + threadIdx.x] = __float2half_rn(acc - __half2float(hi));
    }
}

struct ArgPair { float v; int i; };
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;   // first index on ties
}

// ops.rs:478-502 softmax of each stream's logits, then token_stream.rs:134 + sampling.rs:96-104:
// the first index of the largest ln(max(p, 1e-12)). The pick becomes the stream's next input and
// is appended to its output row, unless it is `eos` (the stream is then done: nothing more is
// appended for it) . Block 0 advances the shared position.
__global__ void __launch_bounds__(1024) pick_batch_kernel(const float* __restrict__ logits, int ldl, int V, int eos, int* __restrict__ cur,
                                                          int* __restrict__ done, int* __restrict__ n_out, int* __restrict__ out, int out_cap,
                                                          int* pos, int advance) {
    __shared__ float red[33];
    __shared__ ArgPair pred[32];
    pdl_wait_prior();
    pdl_launch_next();
    const int s = blockIdx.x;
    const float* row = logits + (size_t)s * ldl;
    const float4* row4 = (const float4*)row;           // ldl % 4 == 0: rows start on 16-byte boundaries
    const int V4 = V >> 2;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
        const float4 v = row4[i];
        mx = fmaxf(mx, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
    for (int i = 4 * V4 + threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float e = 0.0f;
    for (int i = threadIdx.x; i < V4; i += blockDim.x) {
        const float4 v = row4[i];
        e += (expf(v.x - mx) + expf(v.y - mx)) + (expf(v.z - mx) + expf(v.w - mx));
    }
    for (int i = 4 * V4 + threadIdx.x; i < V; i += blockDim.x) e += expf(row[i] - mx);
    const float sum = block_sum(e, red);
    // Only a logit within rounding distance of the largest one can tie its probability after the
    // f32 exp and division; everything more than 0.01 below it has a strictly smaller probability
    // (the largest probability is at least 1 / V, far above the 1e-12 floor), so the full formula
    // is evaluated for those candidates only.
    ArgPair best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = row[i];
        if (l >= mx - 0.01f) best = better(best, ArgPair{logf(fmaxf(expf(l - mx) / sum, 1e-12f)), i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = better(best, ArgPair{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) pred[wid] = best;
    __syncthreads();
    if (wid == 0) {
        best = lane < (int)(blockDim.x >> 5) ? pred[lane] : ArgPair{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) best = better(best, ArgPair{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
        if (lane == 0) {
            if (!done[s]) {
                if (best.i < 0 || best.i >= V) {
                    done[s] = 2;                       // no finite logit: reported as an error by the host, nothing is emitted
                } else if (best.i == eos) {
                    done[s] = 1;
                } else {
                    if (n_out[s] < out_cap) out[(size_t)s * out_cap + n_out[s]] = best.i;
                    n_out[s] += 1;
                    cur[s] = best.i;
                }
            }
            if (s == 0 && advance) *pos += 1;
        }
    }
}

// After the prime: token 1 of every stream (the prime's pick, at queue[prompt_len]) becomes the
// stream's current input and first output; a stream whose prime picked eos starts out done.
__global__ void gather_first_kernel(int* const* __restrict__ queues, StepState* const* __restrict__ states, int prompt_len, int S,
                                    int* cur, int* done, int* n_out, int* out, int out_cap, int* pos) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < kBatchMaxStreams) pos[s] = prompt_len;       // one position word per group of the step
    if (s >= S) return;
    const StepState* st = states[s];
    const bool fin = st->done != 0 || st->tail <= prompt_len;
    done[s] = fin ? 1 : 0;
    n_out[s] = fin ? 0 : 1;
    const int tok = fin ? 0 : queues[s][prompt_len];
    cur[s] = tok;
    if (!fin && out_cap > 0) out[(size_t)s * out_cap] = tok;
}

template <class... KArgs, class... Args>
cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Rows of a window forward into the streams' caches: row r = (stream r / n, position r % n) of
// qkv [S * n][3d] -> k and v rows of that stream at that position.
__global__ void scatter_kv_kernel(const float* __restrict__ qkv, float* const* __restrict__ kcs, float* const* __restrict__ vcs,
                                  size_t layer_off, int n, int d) {
    const int r = blockIdx.x, s = r / n, t = r - s * n;
    const float4* src = (const float4*)(qkv + (size_t)r * 3 * d);
    float4* kd = (float4*)(kcs[s] + layer_off + (size_t)t * d);
    float4* vd = (float4*)(vcs[s] + layer_off + (size_t)t * d);
    const int d4 = d >> 2;
    for (int c = threadIdx.x; c < d4; c += blockDim.x) { kd[c] = src[d4 + c]; vd[c] = src[2 * d4 + c]; }
}

// The last row of each of S windows of n rows: x [S * n][d] -> out [S][d].
__global__ void gather_last_rows_kernel(const float* __restrict__ x, int n, int d, float* __restrict__ out) {
    const int s = blockIdx.x;
    const float* src = x + ((size_t)s * n + n - 1) * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) out[(size_t)s * d + c] = src[c];
}

__global__ void batch_init_kernel(int S, int pos0, int* done, int* n_out, int* cur, int* pos) {
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < kBatchMaxStreams) pos[s] = pos0;             // one position word per group of the step
    if (s < S) { done[s] = 0; n_out[s] = 0; cur[s] = 0; }
}

template <int NT, int RG, int MAXT = 512>
int launch_skinny_nt(const SkArgs& a, int warps, int col_groups, int splits, cudaStream_t st) {
    auto bytes = [](int w, int depth) {
        return (size_t)w * (depth * RG * 544 + 4 * NT * RED_LD * sizeof(float));
    };
    constexpr size_t kSmemCap = 200 * 1024;
    static bool attr[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr[dev]) {
        FC_CUDA(cudaFuncSetAttribute(skinny_q8_kernel<NT, RG, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemCap));
        attr[dev] = true;
    }
    SkArgs b = a;
    while (b.depth > 1 && bytes(warps, b.depth) > kSmemCap) --b.depth;   // a shallower ring when the slots are large
    if (bytes(warps, b.depth) > kSmemCap) return fail(FC_E_SHAPE, "the lock-step product does not fit shared memory");
    FC_CUDA(launch_dep(skinny_q8_kernel<NT, RG, MAXT>, dim3((a.N + 16 * RG - 1) / (16 * RG), col_groups, splits), dim3(warps * 32),
                       bytes(warps, b.depth), st, b));
    ++g_launches;
    return FC_OK;
}

}  // namespace

size_t frag_quant_bytes(const QMat& w) { return (size_t)w.N_pad * w.K; }
size_t frag_scale_bytes(const QMat& w) { return (size_t)w.N_pad * (w.K >> 5) * sizeof(__half); }

int launch_repack_frag(const QMat& w, void* fq, void* fd, cudaStream_t st) {
    if (w.N_pad % 32 || w.K % 32) return fail(FC_E_SHAPE, "fragment-major copy needs N_pad %% 32 == 0 and K %% 32 == 0");
    const size_t total = (size_t)(w.N_pad >> 4) * (w.K >> 5) * 32;
    const size_t want = (total + 255) / 256;
    repack_frag_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, st>>>(w.qu, w.d, w.N_pad, w.K, (uint4*)fq, (__half2*)fd);
    FC_LAUNCHED();
    return FC_OK;
}

int batch_cols(int S) { return S <= 8 ? 16 : S <= 16 ? 32 : S <= 32 ? 64 : 128; }

int skinny_max_splits() { return SK_MAX_SPLITS; }

int launch_skinny_q8(const QFrag& w, int S, const void* xp, const float* bias, int epi, const SkinnyOut& out, int* splits_used,
                     cudaStream_t st) {
    if (S < 1 || S > kBatchMaxStreams) return fail(FC_E_SHAPE, "the lock-step product takes 1..%d streams (got %d)", kBatchMaxStreams, S);
    SkArgs a;
    a.wq = (const uint4*)w.q; a.wd = (const __half2*)w.d; a.xp = (const uint4*)xp;
    a.N = w.N; a.K = w.K; a.S = S;
    a.bias = bias; a.epi = epi; a.residual = out.residual;
    a.y = out.y; a.ldy = out.ldy; a.yp = (__half*)out.planes; a.ldp = out.ldp; a.part_out = out.part;
    const int nkb = w.K >> 5, cols = batch_cols(S);
    // products that leave partial sums split K over CTAs as well: ranges of at least 8 blocks
    int splits = 1;
    if (out.part) splits = std::max(1, std::min(SK_MAX_SPLITS, nkb / 8));
    if (splits_used) *splits_used = splits;
    const int kb_cta = (nkb + splits - 1) / splits;
    // warps split a CTA's K range: at least two 32-wide blocks each
    // A warp's K slice is a chain of dependent steps (block landed -> fragments -> MMAs -> scaled add), about 0.3 us
    // per k-block whatever the width: the slices are kept to two or three blocks by using up to 16 warps.
    int warps = std::min(out.max_warps, kb_cta >= 32 ? 16 : kb_cta >= 16 ? 8 : kb_cta >= 8 ? 4 : kb_cta >= 4 ? 2 : 1);
    // at most 16 streams and a long K (the down-projection): 32 warps (three or four blocks each) on the 16-row tile, in
    // a chain on its own and with two chains side by side (two groups of 16 on the 24-block shape: 31.6 k -> 34.0 k
    // tokens/s; with four groups 48.9 k -> 48.3 k, so not there)
    const bool wide_block = out.long_k_block && cols <= 32 && kb_cta >= 96 && (w.N + 31) / 32 * splits < 2 * 148;
    if (wide_block) warps = 32;
    a.depth = std::max(1, std::min(SK_DEPTH, (kb_cta + warps - 1) / warps));
    if (cols <= 32) {
        // few streams: a chain on its own is bound by latency and takes 32 rows per CTA only when that still leaves
        // every SM several CTAs; chains that share the GPU are bound by throughput, and 32 rows halve the activation
        // fragments read from L2 per weight
        const bool wide = (w.N + 31) / 32 * splits >= 2 * 148 || out.max_warps < 16;
        if (wide_block) return cols == 16 ? launch_skinny_nt<2, 1, 1024>(a, warps, 1, splits, st) : launch_skinny_nt<4, 1, 1024>(a, warps, 1, splits, st);
        if (cols == 16) return wide ? launch_skinny_nt<2, 2>(a, warps, 1, splits, st) : launch_skinny_nt<2, 1>(a, warps, 1, splits, st);
        return wide ? launch_skinny_nt<4, 2>(a, warps, 1, splits, st) : launch_skinny_nt<4, 1>(a, warps, 1, splits, st);
    }
    // 17..64 streams: CTAs of 64 columns (one or two per row range), 32 rows each
    return launch_skinny_nt<8, 2>(a, warps, cols / 64, splits, st);
}

int launch_embed_batch(const QMat& tok, const float* pos_emb, const int* cur, const int* pos, int S, float* x, cudaStream_t st) {
    FC_CUDA(launch_dep(embed_batch_kernel, dim3(S), dim3(256), 0, st, tok, pos_emb, cur, pos, x));
    ++g_launches;
    return FC_OK;
}

int launch_ln_rows_f16(const float* x, const float* part, int n_part, const float* part_bias, float* x_out, const float* g,
                       const float* b, int S, int d, void* xp, cudaStream_t st) {
    const int threads = 256, per = (d + threads - 1) / threads;
    if (!part) n_part = 0;
    if (per <= 4) FC_CUDA(launch_dep(ln_rows_f16_kernel<4>, dim3(S), dim3(threads), 0, st, x, part, n_part, S, part_bias, x_out, g, b, d, (__half*)xp));
    else if (per <= 16) FC_CUDA(launch_dep(ln_rows_f16_kernel<16>, dim3(S), dim3(threads), 0, st, x, part, n_part, S, part_bias, x_out, g, b, d, (__half*)xp));
    else return fail(FC_E_SHAPE, "LayerNorm width %d exceeds 4096", d);
    ++g_launches;
    return FC_OK;
}

int launch_attn_decode_batch(const float* qkv, float* const* kcs, float* const* vcs, size_t layer_off, int d, int H, int ctx,
                             const int* pos, int S, void* ap, cudaStream_t st) {
    const int hd = d / H;
    if (hd > 64 || hd % 4) return fail(FC_E_SHAPE, "head_dim %d is not supported by the lock-step attention", hd);
    const size_t smem = (size_t)(((ctx + 3) & ~3) + 64 + 16 * 64) * sizeof(float);
    if (smem > 48 * 1024) return fail(FC_E_SHAPE, "context %d exceeds what the lock-step attention holds in shared memory", ctx);
    FC_CUDA(launch_dep(attn_decode_batch_kernel, dim3(H, S), dim3(256), smem, st, qkv, kcs, vcs, layer_off, d, hd, pos, (__half*)ap));
    ++g_launches;
    return FC_OK;
}

int launch_pick_batch(const float* logits, int ldl, int V, int S, int eos, int* cur, int* done, int* n_out, int* out, int out_cap,
                      int* pos, int advance, cudaStream_t st) {
    if (ldl % 4) return fail(FC_E_SHAPE, "pick: logit rows must start on 16-byte boundaries");
    FC_CUDA(launch_dep(pick_batch_kernel, dim3(S), dim3(1024), 0, st, logits, ldl, V, eos, cur, done, n_out, out, out_cap, pos, advance));
    ++g_launches;
    return FC_OK;
}

int launch_gather_first(int* const* queues, StepState* const* states, int prompt_len, int S, int* cur, int* done, int* n_out,
                        int* out, int out_cap, int* pos, cudaStream_t st) {
    gather_first_kernel<<<(S + 63) / 64, 64, 0, st>>>(queues, states, prompt_len, S, cur, done, n_out, out, out_cap, pos);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_scatter_kv(const float* qkv, float* const* kcs, float* const* vcs, size_t layer_off, int S, int n, int d, cudaStream_t st) {
    if (d % 4) return fail(FC_E_SHAPE, "scatter_kv: d %% 4 != 0");
    scatter_kv_kernel<<<S * n, 128, 0, st>>>(qkv, kcs, vcs, layer_off, n, d);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_gather_last_rows(const float* x, int S, int n, int d, float* out, cudaStream_t st) {
    gather_last_rows_kernel<<<S, 256, 0, st>>>(x, n, d, out);
    FC_LAUNCHED();
    return FC_OK;
}

int launch_batch_init(int S, int pos0, int* done, int* n_out, int* cur, int* pos, cudaStream_t st) {
    batch_init_kernel<<<(S + 63) / 64, 64, 0, st>>>(S, pos0, done, n_out, cur, pos);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
