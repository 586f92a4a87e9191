// rowq_oracle — CPU restatement of Ferrum's in-memory quantised weight and its linear
// (ferrum_core/src/quant.rs:122-263 QWeight, ops.rs:268-377 qlinear), linked into
// libferrum_oracle.so.
//
// TEST INFRASTRUCTURE ONLY: the checker the CUDA path is compared against.
//
// Parity status: pinned on the reference's own unit tests — round trips bounded by half a step
// (quant.rs:597-637), packed sizes (quant.rs:639-648,680-685), nibble sign extension
// (quant.rs:650-656), qlinear against the dequantised serial sum (ops.rs:877-949) and against
// the f32 linear within the reference's drift bounds (ops.rs:836-930); the Q4_0 / Q5_0 block
// decoders on the reference's Q5 known-answer block (gguf/dequant.rs:371-393).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

int row_bytes(int cols, int kind) { return kind == 1 ? (cols + 1) / 2 : cols; }

// quant.rs:221-223 nibble_to_i8.
int nibble_to_i8(uint8_t nib) { return (int)(int8_t)(uint8_t)(nib << 4) >> 4; }

// quant.rs:164-212 QWeight::from_f32.
void from_f32(const float* data, int rows, int cols, int kind, float* scales, uint8_t* q) {
    const int half = (cols + 1) / 2, rb = row_bytes(cols, kind);
    std::memset(q, 0, (size_t)rows * rb);
    for (int r = 0; r < rows; ++r) {
        const float* row = data + (size_t)r * cols;
        float amax = 0.0f;
        for (int c = 0; c < cols; ++c) amax = std::max(amax, std::fabs(row[c]));
        const float qmax = kind == 1 ? 7.0f : 127.0f;
        const float scale = amax / qmax;
        scales[r] = scale;
        const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
        uint8_t* dst = q + (size_t)r * rb;
        for (int c = 0; c < cols; ++c) {
            float lv = std::round(row[c] * inv);
            if (lv < -qmax) lv = -qmax;
            if (lv > qmax) lv = qmax;
            const int qi = lv == lv ? (int)lv : 0;
            if (kind == 0) dst[c] = (uint8_t)(int8_t)qi;
            else if (c < half) dst[c] = (uint8_t)((dst[c] & 0xF0) | (qi & 0x0F));
            else dst[c - half] = (uint8_t)((dst[c - half] & 0x0F) | ((qi & 0x0F) << 4));
        }
    }
}

int level_at(const uint8_t* q, int cols, int kind, int r, int c) {
    const int half = (cols + 1) / 2, rb = row_bytes(cols, kind);
    const uint8_t* src = q + (size_t)r * rb;
    if (kind == 0) return (int8_t)src[c];
    return nibble_to_i8(c < half ? (src[c] & 0x0F) : (uint8_t)(src[c - half] >> 4));
}

}  // namespace

extern "C" {

float fo_f16_to_f32(uint16_t h);   // ferrum_oracle.cpp

// gguf/dequant.rs:66-83 dequant_q4_0: blocks of [f16 d][16 bytes]; low nibble -> element j, high
// nibble -> element j + 16, value d * (nibble - 8).
void fo_dequant_q4_0(const uint8_t* raw, size_t n, float* out) {
    for (size_t b = 0; b < n / 32; ++b, raw += 18) {
        const float d = fo_f16_to_f32((uint16_t)(raw[0] | (raw[1] << 8)));
        for (int j = 0; j < 16; ++j) {
            out[b * 32 + j] = d * (float)((int)(raw[2 + j] & 0x0F) - 8);
            out[b * 32 + j + 16] = d * (float)((int)(raw[2 + j] >> 4) - 8);
        }
    }
}
// gguf/dequant.rs:105-130 dequant_q5 without a minimum (Q5_0): [f16 d][u32 qh][16 bytes];
// value d * ((nibble | fifth bit << 4) - 16).
void fo_dequant_q5_0(const uint8_t* raw, size_t n, float* out) {
    for (size_t b = 0; b < n / 32; ++b, raw += 22) {
        const float d = fo_f16_to_f32((uint16_t)(raw[0] | (raw[1] << 8)));
        const uint32_t qh = (uint32_t)raw[2] | ((uint32_t)raw[3] << 8) | ((uint32_t)raw[4] << 16) | ((uint32_t)raw[5] << 24);
        for (int j = 0; j < 16; ++j) {
            const int x0 = (int)((raw[6 + j] & 0x0F) | (((qh >> j) & 1u) << 4));
            const int x1 = (int)((raw[6 + j] >> 4) | (((qh >> (j + 16)) & 1u) << 4));
            out[b * 32 + j] = d * (float)(x0 - 16);
            out[b * 32 + j + 16] = d * (float)(x1 - 16);
        }
    }
}

int fo_nibble_to_i8(int nib) { return nibble_to_i8((uint8_t)nib); }
size_t fo_rowq_packed_len(int rows, int cols, int kind) { return (size_t)rows * row_bytes(cols, kind); }
void fo_rowq_from_f32(const float* data, int rows, int cols, int kind, float* scales, uint8_t* q) {
    from_f32(data, rows, cols, kind, scales, q);
}
// quant.rs:226-263 dequant_row / to_f32.
void fo_rowq_to_f32(const uint8_t* q, const float* scales, int rows, int cols, int kind, float* out) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) out[(size_t)r * cols + c] = (float)level_at(q, cols, kind, r, c) * scales[r];
}
// ops.rs:316-377 qlinear with qaccum_cols (ops.rs:268-306): the scale is folded into the
// activations, the output starts at the bias and the rows are added in ascending p.
void fo_rowq_linear(const float* x, const uint8_t* q, const float* scales, int kind, const float* bias, int m, int k, int n, float* y) {
    std::vector<float> a((size_t)m * k);
    for (int i = 0; i < m; ++i)
        for (int p = 0; p < k; ++p) a[(size_t)i * k + p] = x[(size_t)i * k + p] * scales[p];
    for (int i = 0; i < m; ++i) {
        float* out = y + (size_t)i * n;
        for (int j = 0; j < n; ++j) out[j] = bias[j];
        for (int p = 0; p < k; ++p) {
            const float ap = a[(size_t)i * k + p];
            for (int j = 0; j < n; ++j) out[j] += ap * (float)level_at(q, n, kind, p, j);
        }
    }
}

}  // extern "C"
