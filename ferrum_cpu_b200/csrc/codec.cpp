// Host-side load-time codecs of libferrum_cuda: IEEE half conversion, the Q8_0 block
// encoder/decoder and Ferrum's xorshift64* generator. None of this runs in the forward
// pass; a ferrum_cuda wrapper uses it to re-encode the f32 layers the (untouched) GGUF
// loader produces, and the benchmark uses it to synthesise seeded weights.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/ferrum_cuda.h"

namespace {

inline uint32_t bits_of(float f) { uint32_t u; std::memcpy(&u, &f, sizeof u); return u; }
inline float float_of(uint32_t u) { float f; std::memcpy(&f, &u, sizeof f); return f; }

// Round-to-nearest-even right shift of `v` by `s` bits (1 <= s <= 31).
inline uint32_t rne_shift(uint32_t v, unsigned s) {
    const uint32_t kept = v >> s;
    const uint32_t rest = v & ((1u << s) - 1u);
    const uint32_t tie = 1u << (s - 1);
    return kept + ((rest > tie || (rest == tie && (kept & 1u))) ? 1u : 0u);
}

}  // namespace

extern "C" {

// gguf_write/blocks.rs:12-61: RNE, overflow -> Inf, gradual underflow, NaN -> sign|0x7E00.
uint16_t fc_f32_to_f16(float v) {
    const uint32_t u = bits_of(v);
    const uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t e = (u >> 23) & 0xFFu;
    const uint32_t m = u & 0x7FFFFFu;
    if (e == 0xFFu) return (uint16_t)(s | (m ? 0x7E00u : 0x7C00u));
    const int he = (int)e - 112;                 // half exponent field before rounding
    if (he >= 31) return (uint16_t)(s | 0x7C00u);
    if (he <= 0) {
        if (he < -10) return s;                  // below half of the smallest subnormal
        return (uint16_t)(s | rne_shift(m | 0x800000u, (unsigned)(14 - he)));
    }
    // A mantissa carry walks into the exponent field, which is the right answer; an
    // exponent that reaches 31 this way is exactly Inf (0x7C00).
    return (uint16_t)(s | (((uint32_t)he << 10) + rne_shift(m, 13)));
}

// gguf/dequant.rs:7-35.
float fc_f16_to_f32(uint16_t h) {
    const uint32_t s = (uint32_t)(h >> 15) << 31;
    const uint32_t e = (h >> 10) & 31u;
    const uint32_t m = h & 1023u;
    if (e == 31u) return float_of(s | 0x7F800000u | (m << 13));
    if (e) return float_of(s | ((e + 112u) << 23) | (m << 13));
    // subnormal: m * 2^-24 is exact in f32
    const float mag = (float)m * 5.9604644775390625e-8f;
    return float_of(s | bits_of(mag));
}

// quant.rs:271-280 + gguf_write/blocks.rs:132-140.
int fc_q8_0_quantize(const float* x, size_t n, void* out) {
    if (!x || !out || n % 32) return FC_E_FORMAT;
    uint8_t* o = (uint8_t*)out;
    for (size_t b = 0; b < n / 32; ++b, x += 32, o += 34) {
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) {
            const float a = fabsf(x[i]);
            amax = (a > amax) ? a : amax;
        }
        const float d = amax / 127.0f;
        const float inv = (d != 0.0f) ? 1.0f / d : 0.0f;
        const uint16_t d16 = fc_f32_to_f16(d);
        o[0] = (uint8_t)d16;
        o[1] = (uint8_t)(d16 >> 8);
        for (int i = 0; i < 32; ++i) {
            float r = roundf(x[i] * inv);        // ties away from zero
            if (!(r == r)) r = 0.0f;             // Rust `as i8`: NaN -> 0, saturating
            r = r > 127.0f ? 127.0f : (r < -128.0f ? -128.0f : r);
            o[2 + i] = (uint8_t)(int8_t)(int)r;
        }
    }
    return FC_OK;
}

// gguf/dequant.rs:37-49.
int fc_q8_0_dequantize(const void* raw, size_t n, float* out) {
    if (!raw || !out || n % 32) return FC_E_FORMAT;
    const uint8_t* p = (const uint8_t*)raw;
    for (size_t b = 0; b < n / 32; ++b, p += 34, out += 32) {
        const float d = fc_f16_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
        for (int i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)p[2 + i];
    }
    return FC_OK;
}

// rng.rs:9-48.
uint64_t fc_rng_seed(uint64_t seed) { return seed ? seed : 0x9E3779B97F4A7C15ull; }

static inline uint64_t rng_next(uint64_t* s) {
    uint64_t x = *s;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    *s = x;
    return x * 0x2545F4914F6CDD1Dull;
}
static inline float rng_unit(uint64_t* s) { return (float)(rng_next(s) >> 40) * (1.0f / 16777216.0f); }

void fc_rng_fill_normal(uint64_t* state, float scale, size_t n, float* out) {
    uint64_t s = *state;
    for (size_t i = 0; i < n; ++i) {
        float u1 = rng_unit(&s);
        u1 = u1 > 1e-7f ? u1 : 1e-7f;
        const float u2 = rng_unit(&s);
        const float z = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
        out[i] = z * scale;
    }
    *state = s;
}

void fc_rng_fill_ids(uint64_t* state, int32_t vocab, size_t n, int32_t* out) {
    uint64_t s = *state;
    for (size_t i = 0; i < n; ++i) out[i] = (int32_t)(rng_next(&s) % (uint64_t)vocab);
    *state = s;
}


// ---- per-row-scale int8 / int4 (quant.rs:122-263) -------------------------------------------
size_t fc_rowq_packed_len(int rows, int cols, int kind) {
    if (rows <= 0 || cols <= 0) return 0;
    return (size_t)rows * (size_t)(kind == FC_Q_INT4 ? (cols + 1) / 2 : cols);
}

// QWeight::from_f32: scale = max|v| / 127 (int8_scale, quant.rs:17-19) or / 7 (quant.rs:189-190);
// level = round_half_away(v / scale) clamped to the symmetric range; a zero row has scale 0.
int fc_rowq_from_f32(const float* data, int rows, int cols, int kind, float* scales, uint8_t* q) {
    if (!data || !scales || !q) return FC_E_ARG;
    if (rows <= 0 || cols <= 0 || (kind != FC_Q_INT8 && kind != FC_Q_INT4)) return FC_E_SHAPE;
    const float qmax = kind == FC_Q_INT8 ? 127.0f : 7.0f;
    const int half = (cols + 1) / 2;
    const size_t rb = kind == FC_Q_INT8 ? (size_t)cols : (size_t)half;
    std::memset(q, 0, (size_t)rows * rb);
    for (int r = 0; r < rows; ++r) {
        const float* row = data + (size_t)r * cols;
        float amax = 0.0f;
        for (int c = 0; c < cols; ++c) amax = std::fmax(amax, std::fabs(row[c]));
        const float scale = amax / qmax;
        scales[r] = scale;
        const float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
        uint8_t* dst = q + (size_t)r * rb;
        for (int c = 0; c < cols; ++c) {
            float lv = std::round(row[c] * inv);
            lv = lv < -qmax ? -qmax : (lv > qmax ? qmax : lv);
            if (!(lv == lv)) lv = 0.0f;                         // `NaN as i8` is 0 in Rust
            const int qi = (int)lv;
            if (kind == FC_Q_INT8) dst[c] = (uint8_t)(int8_t)qi;
            else if (c < half) dst[c] = (uint8_t)((dst[c] & 0xF0) | (qi & 0x0F));
            else dst[c - half] = (uint8_t)((dst[c - half] & 0x0F) | ((qi & 0x0F) << 4));
        }
    }
    return FC_OK;
}

int fc_rowq_to_f32(const uint8_t* q, const float* scales, int rows, int cols, int kind, float* out) {
    if (!q || !scales || !out) return FC_E_ARG;
    if (rows <= 0 || cols <= 0 || (kind != FC_Q_INT8 && kind != FC_Q_INT4)) return FC_E_SHAPE;
    const int half = (cols + 1) / 2;
    const size_t rb = kind == FC_Q_INT8 ? (size_t)cols : (size_t)half;
    for (int r = 0; r < rows; ++r) {
        const uint8_t* src = q + (size_t)r * rb;
        for (int c = 0; c < cols; ++c) {
            int lv;
            if (kind == FC_Q_INT8) lv = (int8_t)src[c];
            else {
                const uint8_t nib = c < half ? (src[c] & 0x0F) : (src[c - half] >> 4);
                lv = (int8_t)(nib << 4) >> 4;                   // nibble_to_i8, quant.rs:221-223
            }
            out[(size_t)r * cols + c] = (float)lv * scales[r];
        }
    }
    return FC_OK;
}


// ---- exact re-blocking of integer-level GGML formats to Q8_0 ---------------------------------
size_t fc_ggml_block_bytes(int ggml_type) {
    switch (ggml_type) {
        case FC_GGML_Q4_0: return 18;   // f16 d + 16 bytes of nibbles (gguf/format.rs:116)
        case FC_GGML_Q5_0: return 22;   // f16 d + 4 bytes of high bits + 16 bytes of nibbles (gguf/format.rs:118)
        case FC_GGML_Q8_0: return 34;
        default: return 0;
    }
}

int fc_ggml_to_q8_0(int ggml_type, const void* raw, size_t n, void* out) {
    if (!raw || !out) return FC_E_ARG;
    const size_t bb = fc_ggml_block_bytes(ggml_type);
    if (!bb || n % 32) return FC_E_FORMAT;
    const uint8_t* src = (const uint8_t*)raw;
    uint8_t* dst = (uint8_t*)out;
    for (size_t b = 0; b < n / 32; ++b, src += bb, dst += 34) {
        dst[0] = src[0]; dst[1] = src[1];                       // the f16 scale, untouched
        int8_t* q = (int8_t*)(dst + 2);
        if (ggml_type == FC_GGML_Q8_0) {
            std::memcpy(q, src + 2, 32);
        } else if (ggml_type == FC_GGML_Q4_0) {
            // low nibble -> element j, high nibble -> element j + 16, centred at 8 (dequant.rs:73-80)
            for (int j = 0; j < 16; ++j) {
                q[j] = (int8_t)((src[2 + j] & 0x0F) - 8);
                q[j + 16] = (int8_t)((src[2 + j] >> 4) - 8);
            }
        } else {
            // the fifth bit of element j is bit j of qh, of element j + 16 bit j + 16 (dequant.rs:112-126)
            uint32_t qh;
            std::memcpy(&qh, src + 2, 4);
            for (int j = 0; j < 16; ++j) {
                const int x0 = (src[6 + j] & 0x0F) | (int)(((qh >> j) & 1u) << 4);
                const int x1 = (src[6 + j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
                q[j] = (int8_t)(x0 - 16);
                q[j + 16] = (int8_t)(x1 - 16);
            }
        }
    }
    return FC_OK;
}


// ---- every GGML block format the reference's importer reads (gguf/dequant.rs:37-315), to f32 ---------------
// Sizes of gguf/format.rs:107-130: values per block and bytes per block.
static bool ggml_block(int t, size_t* vals, size_t* bytes) {
    switch (t) {
        case FC_GGML_F32: *vals = 1; *bytes = 4; return true;
        case FC_GGML_F16: *vals = 1; *bytes = 2; return true;
        case FC_GGML_Q4_0: *vals = 32; *bytes = 18; return true;
        case FC_GGML_Q4_1: *vals = 32; *bytes = 20; return true;
        case FC_GGML_Q5_0: *vals = 32; *bytes = 22; return true;
        case FC_GGML_Q5_1: *vals = 32; *bytes = 24; return true;
        case FC_GGML_Q8_0: *vals = 32; *bytes = 34; return true;
        case FC_GGML_Q8_1: *vals = 32; *bytes = 36; return true;
        case FC_GGML_Q2_K: *vals = 256; *bytes = 84; return true;
        case FC_GGML_Q3_K: *vals = 256; *bytes = 110; return true;
        case FC_GGML_Q4_K: *vals = 256; *bytes = 144; return true;
        case FC_GGML_Q5_K: *vals = 256; *bytes = 176; return true;
        case FC_GGML_Q6_K: *vals = 256; *bytes = 210; return true;
        default: return false;
    }
}

size_t fc_ggml_type_bytes(int ggml_type, size_t n) {
    size_t vals = 0, bytes = 0;
    if (!ggml_block(ggml_type, &vals, &bytes) || n % vals) return 0;
    return n / vals * bytes;
}

}  // extern "C"

namespace {
inline float half_at(const uint8_t* p) { return fc_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }

// The 6-bit (scale, min) pair of sub-block j of a Q4_K / Q5_K super-block (gguf/dequant.rs:133-141): the first
// four pairs sit in the low six bits of bytes j and j + 4; the last four keep their low nibbles in byte j + 4
// and their top two bits in the spare bits of bytes j - 4 and j.
inline void k4_scale_min(int j, const uint8_t* q, int* sc, int* mn) {
    if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
    else { *sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4); *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// One block of `t` at `b` into out[0 .. values per block). Products are formed exactly as the reference forms them
// (which factor is rounded first), so the f32 results agree bit for bit.
void dequant_block(int t, const uint8_t* b, float* out) {
    switch (t) {
        case FC_GGML_F32: std::memcpy(out, b, 4); break;
        case FC_GGML_F16: out[0] = half_at(b); break;
        case FC_GGML_Q8_0: case FC_GGML_Q8_1: {           // dequant.rs:37-64 (Q8_1 carries an unused block sum)
            const float d = half_at(b);
            const int8_t* q = (const int8_t*)(b + (t == FC_GGML_Q8_0 ? 2 : 4));
            for (int j = 0; j < 32; ++j) out[j] = d * (float)q[j];
            break;
        }
        case FC_GGML_Q4_0: {                               // dequant.rs:66-83
            const float d = half_at(b);
            for (int j = 0; j < 16; ++j) {
                out[j] = d * (float)((int)(b[2 + j] & 0x0F) - 8);
                out[j + 16] = d * (float)((int)(b[2 + j] >> 4) - 8);
            }
            break;
        }
        case FC_GGML_Q4_1: {                               // dequant.rs:85-101: d * nibble + m
            const float d = half_at(b), m = half_at(b + 2);
            for (int j = 0; j < 16; ++j) {
                out[j] = d * (float)(b[4 + j] & 0x0F) + m;
                out[j + 16] = d * (float)(b[4 + j] >> 4) + m;
            }
            break;
        }
        case FC_GGML_Q5_0: case FC_GGML_Q5_1: {           // dequant.rs:105-130
            const bool with_min = t == FC_GGML_Q5_1;
            const float d = half_at(b), m = with_min ? half_at(b + 2) : 0.0f;
            const uint8_t* hb = b + (with_min ? 4 : 2);
            const uint32_t qh = (uint32_t)hb[0] | ((uint32_t)hb[1] << 8) | ((uint32_t)hb[2] << 16) | ((uint32_t)hb[3] << 24);
            const uint8_t* qs = hb + 4;
            for (int j = 0; j < 16; ++j) {
                const int x0 = (qs[j] & 0x0F) | (int)(((qh >> j) & 1u) << 4);
                const int x1 = (qs[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
                out[j] = with_min ? d * (float)x0 + m : d * (float)(x0 - 16);
                out[j + 16] = with_min ? d * (float)x1 + m : d * (float)(x1 - 16);
            }
            break;
        }
        case FC_GGML_Q4_K: case FC_GGML_Q5_K: {           // dequant.rs:143-206: (d * sc) * q - (dmin * m)
            const bool five = t == FC_GGML_Q5_K;
            const float d = half_at(b), dmin = half_at(b + 2);
            const uint8_t* scales = b + 4;
            const uint8_t* qh = b + 16;                     // Q5_K only: 32 bytes, bit 2g / 2g + 1 of byte l for pair g
            const uint8_t* qs = b + (five ? 48 : 16);
            for (int g = 0; g < 4; ++g) {                  // 64 values: low nibbles, then high nibbles, of 32 bytes
                int s1, m1, s2, m2;
                k4_scale_min(2 * g, scales, &s1, &m1);
                k4_scale_min(2 * g + 1, scales, &s2, &m2);
                const float d1 = d * (float)s1, n1 = dmin * (float)m1, d2 = d * (float)s2, n2 = dmin * (float)m2;
                for (int l = 0; l < 32; ++l) {
                    const int h1 = five && (qh[l] & (1u << (2 * g))) ? 16 : 0;
                    const int h2 = five && (qh[l] & (2u << (2 * g))) ? 16 : 0;
                    out[64 * g + l] = d1 * (float)((qs[32 * g + l] & 0x0F) + h1) - n1;
                    out[64 * g + 32 + l] = d2 * (float)((qs[32 * g + l] >> 4) + h2) - n2;
                }
            }
            break;
        }
        case FC_GGML_Q6_K: {                               // dequant.rs:208-241: (d * scale) * (6-bit value - 32)
            const uint8_t *ql = b, *qh = b + 128;
            const int8_t* sc = (const int8_t*)(b + 192);
            const float d = half_at(b + 208);
            for (int half = 0; half < 2; ++half)
                for (int l = 0; l < 32; ++l) {
                    const int is = l / 16;
                    const uint8_t h = qh[32 * half + l];
                    const int q1 = ((ql[64 * half + l] & 0x0F) | ((h & 3) << 4)) - 32;
                    const int q2 = ((ql[64 * half + l + 32] & 0x0F) | (((h >> 2) & 3) << 4)) - 32;
                    const int q3 = ((ql[64 * half + l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
                    const int q4 = ((ql[64 * half + l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
                    float* o = out + 128 * half + l;
                    o[0] = d * (float)sc[8 * half + is] * (float)q1;
                    o[32] = d * (float)sc[8 * half + is + 2] * (float)q2;
                    o[64] = d * (float)sc[8 * half + is + 4] * (float)q3;
                    o[96] = d * (float)sc[8 * half + is + 6] * (float)q4;
                }
            break;
        }
        case FC_GGML_Q2_K: {                               // dequant.rs:243-276: (d * sc) * q - (dmin * m), 16 runs of 16
            const uint8_t *scales = b, *qs = b + 16;
            const float d = half_at(b + 80), dmin = half_at(b + 82);
            int run = 0;
            for (int half = 0; half < 2; ++half)
                for (int shift = 0; shift < 8; shift += 2)
                    for (int r = 0; r < 2; ++r, ++run) {
                        const float dl = d * (float)(scales[run] & 0x0F), ml = dmin * (float)(scales[run] >> 4);
                        for (int l = 0; l < 16; ++l) out[16 * run + l] = dl * (float)((qs[32 * half + 16 * r + l] >> shift) & 3) - ml;
                    }
            break;
        }
        case FC_GGML_Q3_K: {                               // dequant.rs:278-324: d * (scale - 32) * (low2 - (high bit ? 0 : 4))
            const uint8_t *hmask = b, *qs = b + 32, *sc = b + 96;
            const float d = half_at(b + 108);
            int scales[16];
            for (int j = 0; j < 8; ++j) { scales[j] = sc[j] & 0x0F; scales[j + 8] = sc[j] >> 4; }
            for (int j = 0; j < 16; ++j) scales[j] |= ((sc[8 + j / 4] >> (2 * (j % 4))) & 3) << 4;
            int run = 0;
            unsigned m = 1;
            for (int half = 0; half < 2; ++half)
                for (int shift = 0; shift < 8; shift += 2, m <<= 1)
                    for (int r = 0; r < 2; ++r, ++run) {
                        const float dl = d * (float)((int)(int8_t)scales[run] - 32);
                        for (int l = 16 * r; l < 16 * r + 16; ++l) {
                            const int low = (qs[32 * half + l] >> shift) & 3;
                            out[16 * run + (l - 16 * r)] = dl * (float)(low - ((hmask[l] & m) ? 0 : 4));
                        }
                    }
            break;
        }
    }
}
}  // namespace

extern "C" {

int fc_ggml_dequantize(int ggml_type, const void* raw, size_t nbytes, size_t n, float* out) {
    if (!raw || !out) return FC_E_ARG;
    size_t vals = 0, bytes = 0;
    if (!ggml_block(ggml_type, &vals, &bytes) || n % vals) return FC_E_FORMAT;
    if (nbytes < n / vals * bytes) return FC_E_FORMAT;       // data shorter than the element count (dequant.rs:541-547)
    const uint8_t* src = (const uint8_t*)raw;
    for (size_t i = 0; i < n / vals; ++i) dequant_block(ggml_type, src + i * bytes, out + i * vals);
    return FC_OK;
}

int fc_ggml_requantize_q8_0(int ggml_type, const void* raw, size_t nbytes, size_t n, void* out) {
    if (!raw || !out) return FC_E_ARG;
    if (n % 32) return FC_E_FORMAT;
    if (fc_ggml_block_bytes(ggml_type)) {                      // integer levels under one f16 scale: exact
        if (nbytes < n / 32 * fc_ggml_block_bytes(ggml_type)) return FC_E_FORMAT;
        return fc_ggml_to_q8_0(ggml_type, raw, n, out);
    }
    size_t vals = 0, bytes = 0;
    if (!ggml_block(ggml_type, &vals, &bytes) || n % vals || nbytes < n / vals * bytes) return FC_E_FORMAT;
    // formats with minima or sub-block scales: to f32 and through the Q8_0 encoder, 256 values at a time
    const uint8_t* src = (const uint8_t*)raw;
    uint8_t* dst = (uint8_t*)out;
    float buf[256];
    const size_t step = vals < 32 ? 32 : vals;                 // f32 / f16 values go 32 at a time
    for (size_t i = 0; i < n; i += step) {
        for (size_t k = 0; k < step / vals; ++k) dequant_block(ggml_type, src + (i / vals + k) * bytes, buf + k * vals);
        const int rc = fc_q8_0_quantize(buf, step, dst + i / 32 * 34);
        if (rc != FC_OK) return rc;
    }
    return FC_OK;
}

}  // extern "C"
