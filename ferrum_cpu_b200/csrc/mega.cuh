// Parameters of the persistent decode kernel (decode_mega.cu) and the work split shared by
// the kernel and the host code that packs its per-CTA parameter blocks.
#pragma once
#include "fc_common.cuh"

namespace fc {

// Rows of an [N][K] Q8_0 matrix owned by CTA c of G. Ranges are multiples of g rows so that
// the scale-plane offset r0 * K/16 bytes stays 16-byte aligned (bulk copies need it).
__host__ __device__ inline int mega_row_gran(int K) {
    int g = 1;
    while ((g * K) & 255) g <<= 1;     // K % 32 == 0 -> g in {1,2,4,8}
    return g;
}
__host__ __device__ inline void mega_cta_rows(int N, int K, int c, int G, int* r0, int* r1) {
    const int g = mega_row_gran(K);
    const int units = (N + g - 1) / g;
    const int u0 = (int)((long long)c * units / G), u1 = (int)((long long)(c + 1) * units / G);
    *r0 = u0 * g;
    *r1 = (u1 * g < N) ? u1 * g : N;
}

// The LM head is read from a second, tile-major copy made at upload: rows are grouped into
// strips of 8, and a strip is K/32 tiles of 272 bytes, each holding the 8 x 32 signed quants of
// one Q8_0 block column (row-major, 256 B) followed by the 8 f16 scales (16 B). A tile is
// exactly the B operand of one m16n8k32 integer MMA plus its scales, a strip is contiguous (one
// bulk copy), and the density is Q8_0's own 34 bytes per 32 weights.
constexpr int kMegaStripRows = 8;
constexpr int kMegaTileBytes = 272;
struct QTile {
    const unsigned char* t = nullptr;
    int N = 0, K = 0;
};
__host__ __device__ inline int mega_strip_bytes(int K) { return (K >> 5) * kMegaTileBytes; }
__host__ __device__ inline int mega_strips(int N) { return (N + kMegaStripRows - 1) / kMegaStripRows; }
// Strips of an N-row matrix owned by CTA c of G.
__host__ __device__ inline void mega_cta_strips(int N, int c, int G, int* s0, int* s1) {
    const int units = mega_strips(N);
    *s0 = (int)((long long)c * units / G);
    *s1 = (int)((long long)(c + 1) * units / G);
}

constexpr int kMegaBiasPackMax = 640;   // most floats of bias one CTA can own in a block (smaller grids own more rows)
constexpr int kMegaMaxLayers = 32;

// Offsets (floats) of the four bias slices of one CTA inside its pack; each slice starts on a
// multiple of 4. Returns the pack length used.
__host__ __device__ inline int mega_bias_offsets(int d, int F, int c, int G, int off[4]) {
    const int N[4] = {3 * d, d, F, d}, K[4] = {d, d, d, F};
    int o = 0;
    for (int i = 0; i < 4; ++i) {
        int r0, r1;
        mega_cta_rows(N[i], K[i], c, G, &r0, &r1);
        off[i] = o;
        o += (r1 - r0 + 3) & ~3;
    }
    return o;
}

struct MegaLayer {
    QMat qkv, out, up, down;
    const float* lnpack;     // [4d]: ln1 gain, ln1 bias, ln2 gain, ln2 bias
    const float* biaspack;   // [G][bias_pack]: per-CTA slices of the qkv, out, up, down biases
};

struct MegaParams {
    int L, d, H, F, T, V;
    QMat tok;                  // embedding rows (row-major planes)
    QTile head;                // LM head, tile-major
    const float* pos;
    const float* lnfpack;      // [4d]: final LayerNorm gain, bias (rest unused)
    const MegaLayer* layers;   // device array [L], built for this launch's grid size
    int bias_pack;             // floats per CTA in the bias packs (multiple of 4, <= kMegaBiasPackMax)
    float *kc, *vc;            // f32 KV caches [L][T][d]
    // exchange buffers in global memory (written by some CTAs, read by all after a barrier)
    float* qg;                 // [d] query row
    float* attg;               // [d] attention output (contexts short enough for one CTA per head)
    float* partg;              // [H * attn_splits][hd + 2] attention partials (max, sum, out)
    float *x1g, *xg;           // [d] residual stream after attention / after the MLP
    float* hidg;               // [F] GELU output
    float* logits;             // [V]
    float* statg;              // [grid][4] per-CTA softmax statistics and best candidate
    float* probs;              // [V] or null: probabilities of the last step
    int* queue;                // token window (token_stream.rs `window`)
    int queue_cap;
    StepState* state;
    unsigned* bar;             // grid barrier counter, zeroed before every launch
    int* status;               // 0, or FC_E_TIMEOUT when a bounded wait ran out
    int n_steps;               // tokens fed by this launch
    int head_from;             // steps before this index skip the LM head
    int select;                // head steps pick the next token greedily and append it
    int attn_splits;           // CTAs per head in the attention phase
    // Optional phase timeline (tracing): when non-null, every CTA stores the global nanosecond
    // timer at every phase boundary of the launch's last step in its row [trace_cap] of the
    // buffer; entry 0 is the step start.
    unsigned long long* trace;
    int trace_cap;
    long long wait_cycles;     // budget of every bounded wait (mbarrier, grid barrier)
    int withhold;              // test hook: the producer warps copy nothing
};

size_t mega_smem_bytes();
int mega_head_rows_max();   // most LM-head rows one CTA can own
int mega_threads();
int mega_supported(const fc_config& c);
int mega_max_grid(int* grid);
int launch_decode_mega(const MegaParams& p, int grid, cudaStream_t st);
// Tile-major copy of w (rows up to w.N_pad, a multiple of 8) into out
// [w.N_pad / 8 strips][mega_strip_bytes(K)].
int launch_repack_tiles(const QMat& w, unsigned char* out, cudaStream_t st);

}  // namespace fc
