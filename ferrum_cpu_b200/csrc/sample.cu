// Token sampler on the device: repetition penalty -> temperature softmax -> top-k -> top-p ->
// renormalise -> inverse-CDF draw, the pipeline of sample_with_params
// (ferrum_core/src/slm/sampling.rs:124-210) on the log-probabilities stream_next builds
// (slm/token_stream.rs:134: ln(max(p, 1e-12))), with Ferrum's xorshift64* generator
// (rng.rs:29-40) advanced on the device.
//
// One CTA, the row staged in shared memory. Differences from the sequential reference, all at
// rounding level: sums are block reductions (a different association than index order), the
// running mass of the draw is a block scan + a sequential walk inside one thread's chunk, and
// probabilities that tie exactly at the top-p cut are all kept (the reference's unstable sort
// keeps an unspecified subset of them). A draw can therefore differ from the reference only
// when r falls within rounding of a cumulative boundary.
//
// Bound: latency (one row of V floats, ~70 block-wide passes out of shared memory).
#include <climits>

#include "fc_common.cuh"

namespace fc {

namespace {
constexpr int ST = 1024;   // threads

__device__ float bsum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int w = 0; w < ST / 32; ++w) t += red[w];
    return t;
}
__device__ float bmax(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = -INFINITY;
#pragma unroll
    for (int w = 0; w < ST / 32; ++w) t = fmaxf(t, red[w]);
    return t;
}
__device__ int bsum_int(int v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = __int_as_float(v);
    __syncthreads();
    int t = 0;
#pragma unroll
    for (int w = 0; w < ST / 32; ++w) t += __float_as_int(red[w]);
    return t;
}
// rng.rs:29-35
__device__ unsigned long long next_u64(unsigned long long* state) {
    unsigned long long x = *state;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *state = x;
    return x * 0x2545F4914F6CDD1DULL;
}
// total order of slm/sampling.rs:96-104 (f32::total_cmp) as a signed key
__device__ __forceinline__ int order_key(float f) {
    const int b = __float_as_int(f);
    return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}
}  // namespace

// logits_or_probs: V values; from_probs != 0: they are probabilities and the logits are
// ln(max(p, 1e-12)). recent[0 .. n_recent): the ids of the current window. The drawn id goes
// to *token_out and, when `state` is given, through the EOS check into queue[tail].
__global__ void __launch_bounds__(ST, 1)
sample_kernel(const float* __restrict__ in, int V, int from_probs, fc_sampling prm, const int* __restrict__ recent,
              int n_recent_fixed, unsigned long long* rng_state, int* queue, int queue_cap, StepState* state, int* token_out) {
    extern __shared__ __align__(16) float w[];       // [V]
    __shared__ float red[ST / 32];
    __shared__ int found;
    __shared__ float r_draw;
    const int tid = threadIdx.x;
    if (state && (state->done | state->error)) return;
    const int n_recent = state ? state->tail : n_recent_fixed;

    for (int i = tid; i < V; i += ST) w[i] = from_probs ? logf(fmaxf(in[i], 1e-12f)) : in[i];
    __syncthreads();
    // 1. repetition penalty, once per occurrence: the thread that holds the first occurrence of
    // an id applies it as many times as the id occurs
    const float rp = prm.repetition_penalty;
    if (fabsf(rp - 1.0f) > 1.1920929e-7f && rp > 0.0f) {
        for (int j = tid; j < n_recent; j += ST) {
            const int tok = recent[j];
            if (tok < 0 || tok >= V) continue;
            bool first = true;
            for (int q = 0; q < j && first; ++q) first = recent[q] != tok;
            if (!first) continue;
            int count = 0;
            for (int q = j; q < n_recent; ++q) count += recent[q] == tok;
            float l = w[tok];
            for (int c = 0; c < count; ++c) l = l > 0.0f ? l / rp : l * rp;
            w[tok] = l;
        }
        __syncthreads();
    }
    int token = 0;
    if (prm.temperature <= 0.0f) {
        // argmax_first over the penalised logits; no draw
        int bk = INT_MIN, bi = 0x7fffffff;
        for (int i = tid; i < V; i += ST) {
            const int kx = order_key(w[i]);
            if (kx > bk) { bk = kx; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const int ok = __shfl_xor_sync(0xffffffffu, bk, o), oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ok > bk || (ok == bk && oi < bi)) { bk = ok; bi = oi; }
        }
        __shared__ int kk[ST / 32], ii[ST / 32];
        if ((tid & 31) == 0) { kk[tid >> 5] = bk; ii[tid >> 5] = bi; }
        __syncthreads();
        bk = kk[0]; bi = ii[0];
        for (int q = 1; q < ST / 32; ++q)
            if (kk[q] > bk || (kk[q] == bk && ii[q] < bi)) { bk = kk[q]; bi = ii[q]; }
        token = V > 0 && bi < V ? bi : 0;
    } else {
        const float t = fmaxf(prm.temperature, 0.01f);
        // 2. temperature softmax
        float mx = -INFINITY;
        for (int i = tid; i < V; i += ST) mx = fmaxf(mx, w[i]);
        mx = bmax(mx, red);
        float s = 0.0f;
        for (int i = tid; i < V; i += ST) {
            const float e = expf((w[i] - mx) / t);
            w[i] = e;
            s += e;
        }
        const float sum = bsum(s, red);
        if (!(sum > 1e-10f)) {
            // degenerate mass: uniform fallback (sampling.rs:160-167)
            if (tid == 0) found = (int)(next_u64(rng_state) % (unsigned long long)V);
            __syncthreads();
            token = found;
        } else {
            for (int i = tid; i < V; i += ST) w[i] /= sum;
            __syncthreads();
            // 3. top-k: the k-th largest probability by bisection on its bit pattern
            if (prm.top_k > 0 && prm.top_k < V) {
                unsigned T = 0;
                for (int bit = 30; bit >= 0; --bit) {
                    const unsigned cand = T | (1u << bit);
                    int c = 0;
                    for (int i = tid; i < V; i += ST) c += __float_as_uint(w[i]) >= cand;
                    if (bsum_int(c, red) >= prm.top_k) T = cand;
                }
                const float threshold = __uint_as_float(T);
                for (int i = tid; i < V; i += ST)
                    if (w[i] < threshold) w[i] = 0.0f;
                __syncthreads();
            }
            // 4. top-p: the largest cut whose kept mass still reaches top_p
            if (prm.top_p < 1.0f) {
                unsigned T = 0;
                for (int bit = 30; bit >= 0; --bit) {
                    const unsigned cand = T | (1u << bit);
                    float m = 0.0f;
                    for (int i = tid; i < V; i += ST) m += __float_as_uint(w[i]) >= cand ? w[i] : 0.0f;
                    const float kept = bsum(m, red);
                    if (kept >= prm.top_p && kept > 0.0f) T = cand;   // kept > 0: the cut never passes the top token
                }
                // the top token always stays (T never exceeds the maximum that carries mass)
                const float cut = __uint_as_float(T);
                for (int i = tid; i < V; i += ST)
                    if (w[i] < cut) w[i] = 0.0f;
                __syncthreads();
            }
            // 5. renormalise and draw
            float s2 = 0.0f;
            for (int i = tid; i < V; i += ST) s2 += w[i];
            const float sum2 = bsum(s2, red);
            for (int i = tid; i < V; i += ST) w[i] /= sum2;
            if (tid == 0) {
                r_draw = (float)(next_u64(rng_state) >> 40) / 16777216.0f;   // rng.rs:37-40
                found = 0x7fffffff;
            }
            __syncthreads();
            // pick_by_mass (sampling.rs:106-121): thread t owns indices [t*chunk, (t+1)*chunk)
            const int chunk = (V + ST - 1) / ST, i0 = min(tid * chunk, V), i1 = min(i0 + chunk, V);
            float local = 0.0f;
            int last = -1;
            for (int i = i0; i < i1; ++i)
                if (w[i] > 0.0f) { local += w[i]; last = i; }
            // exclusive scan of the chunk masses over the threads
            float incl = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float v = __shfl_up_sync(0xffffffffu, incl, o);
                if ((tid & 31) >= o) incl += v;
            }
            if ((tid & 31) == 31) red[tid >> 5] = incl;
            __syncthreads();
            float base = incl - local;
            for (int q = 0; q < (tid >> 5); ++q) base += red[q];
            const float r = r_draw;
            float cum = base;
            for (int i = i0; i < i1; ++i)
                if (w[i] > 0.0f) {
                    cum += w[i];
                    if (r <= cum) { atomicMin(&found, i); break; }
                }
            __syncthreads();
            if (found == 0x7fffffff) {
                // rounding left the total a hair under r: the last index that has any mass
                __shared__ int lasts[ST / 32];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
                if ((tid & 31) == 0) lasts[tid >> 5] = last;
                __syncthreads();
                int l = 0;
                for (int q = 0; q < ST / 32; ++q) l = max(l, lasts[q]);
                token = l;
            } else {
                token = found;
            }
        }
    }
    if (tid == 0) {
        if (token_out) *token_out = token;
        if (state) {
            if (token == state->eos) {
                state->done = 1;
            } else if (state->tail < queue_cap) {
                queue[state->tail] = token;
                state->tail += 1;
            } else {
                state->error = FC_E_DIM;
            }
        }
    }
}

int launch_sample(const float* in, int V, int from_probs, const fc_sampling& prm, const int* recent, int n_recent,
                  unsigned long long* rng_state, int* queue, int queue_cap, StepState* state, int* token_out, cudaStream_t st) {
    const size_t smem = (size_t)V * sizeof(float);
    if (V <= 0 || smem > 200 * 1024) return fail(FC_E_SHAPE, "the device sampler holds a row of at most 51200 logits in shared memory (V = %d)", V);
    static bool attr_set[64] = {};
    int dev = 0;
    FC_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        FC_CUDA(cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[dev] = true;
    }
    sample_kernel<<<1, ST, smem, st>>>(in, V, from_probs, prm, recent, n_recent, rng_state, queue, queue_cap, state, token_out);
    FC_LAUNCHED();
    return FC_OK;
}

}  // namespace fc
