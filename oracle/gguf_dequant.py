"""CPU restatement of the reference's GGML block decoders (ferrum_core/src/gguf/dequant.rs:37-315). TEST
INFRASTRUCTURE: only tests/ may import this file; the shipped library has its own decoders (csrc/codec.cpp), which
the tests hold to these bit for bit.

Plain loops over numpy scalars: every product is formed in f32 in the order the reference forms it
(`d * sc` first, then `* q`, then `- min`), so the results are the reference's f32 values exactly. Parity is pinned
on the reference's own known-answer blocks (dequant.rs:337-547), restated in tests/test_ggml_formats.py.
"""
import numpy as np

F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 0, 1, 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14
# gguf/format.rs:107-130: (values per block, bytes per block)
BLOCK = {F32: (1, 4), F16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_0: (32, 34),
         Q8_1: (32, 36), Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}

f32 = np.float32


def type_nbytes(t, n):
    """gguf/format.rs:107-130; None where the reference returns an error."""
    if t not in BLOCK or n % BLOCK[t][0]:
        return None
    return n // BLOCK[t][0] * BLOCK[t][1]


def _half(b, at):
    return f32(np.frombuffer(bytes(b[at:at + 2]), dtype=np.float16)[0])   # dequant.rs:7-35 (IEEE half, exact in f32)


def scale_min_k4(j, q):
    """dequant.rs:133-141."""
    if j < 4:
        return int(q[j]) & 63, int(q[j + 4]) & 63
    return (int(q[j + 4]) & 0x0F) | ((int(q[j - 4]) >> 6) << 4), (int(q[j + 4]) >> 4) | ((int(q[j]) >> 6) << 4)


def _block(t, b):
    b = [int(x) for x in b]
    if t == F32:
        return [f32(np.frombuffer(bytes(b), dtype=np.float32)[0])]
    if t == F16:
        return [_half(b, 0)]
    if t in (Q8_0, Q8_1):                                   # dequant.rs:37-64
        d, off = _half(b, 0), 2 if t == Q8_0 else 4
        return [d * f32(q - 256 if q > 127 else q) for q in b[off:off + 32]]
    if t == Q4_0:                                           # dequant.rs:66-83
        d, out = _half(b, 0), [f32(0)] * 32
        for j in range(16):
            out[j] = d * f32((b[2 + j] & 15) - 8)
            out[j + 16] = d * f32((b[2 + j] >> 4) - 8)
        return out
    if t == Q4_1:                                           # dequant.rs:85-101
        d, m, out = _half(b, 0), _half(b, 2), [f32(0)] * 32
        for j in range(16):
            out[j] = d * f32(b[4 + j] & 15) + m
            out[j + 16] = d * f32(b[4 + j] >> 4) + m
        return out
    if t in (Q5_0, Q5_1):                                   # dequant.rs:105-130
        with_min = t == Q5_1
        d = _half(b, 0)
        m = _half(b, 2) if with_min else f32(0)
        at = 4 if with_min else 2
        qh = b[at] | (b[at + 1] << 8) | (b[at + 2] << 16) | (b[at + 3] << 24)
        qs, out = b[at + 4:at + 20], [f32(0)] * 32
        for j in range(16):
            x0 = (qs[j] & 15) | (((qh >> j) & 1) << 4)
            x1 = (qs[j] >> 4) | (((qh >> (j + 16)) & 1) << 4)
            out[j] = d * f32(x0) + m if with_min else d * f32(x0 - 16)
            out[j + 16] = d * f32(x1) + m if with_min else d * f32(x1 - 16)
        return out
    if t in (Q4_K, Q5_K):                                   # dequant.rs:143-206
        five = t == Q5_K
        d, dmin, scales = _half(b, 0), _half(b, 2), b[4:16]
        qh = b[16:48] if five else None
        qs = b[48:176] if five else b[16:144]
        out = [f32(0)] * 256
        for g in range(4):
            s1, m1 = scale_min_k4(2 * g, scales)
            s2, m2 = scale_min_k4(2 * g + 1, scales)
            d1, n1, d2, n2 = d * f32(s1), dmin * f32(m1), d * f32(s2), dmin * f32(m2)
            for l in range(32):
                h1 = 16 if five and qh[l] & (1 << (2 * g)) else 0
                h2 = 16 if five and qh[l] & (2 << (2 * g)) else 0
                out[64 * g + l] = d1 * f32((qs[32 * g + l] & 15) + h1) - n1
                out[64 * g + 32 + l] = d2 * f32((qs[32 * g + l] >> 4) + h2) - n2
        return out
    if t == Q6_K:                                           # dequant.rs:208-241
        ql, qh, sc, d = b[0:128], b[128:192], [x - 256 if x > 127 else x for x in b[192:208]], _half(b, 208)
        out = [f32(0)] * 256
        for half in range(2):
            for l in range(32):
                i, h = l // 16, qh[32 * half + l]
                q1 = ((ql[64 * half + l] & 15) | ((h & 3) << 4)) - 32
                q2 = ((ql[64 * half + l + 32] & 15) | (((h >> 2) & 3) << 4)) - 32
                q3 = ((ql[64 * half + l] >> 4) | (((h >> 4) & 3) << 4)) - 32
                q4 = ((ql[64 * half + l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32
                o = 128 * half + l
                out[o] = d * f32(sc[8 * half + i]) * f32(q1)
                out[o + 32] = d * f32(sc[8 * half + i + 2]) * f32(q2)
                out[o + 64] = d * f32(sc[8 * half + i + 4]) * f32(q3)
                out[o + 96] = d * f32(sc[8 * half + i + 6]) * f32(q4)
        return out
    if t == Q2_K:                                           # dequant.rs:243-276
        scales, qs, d, dmin = b[0:16], b[16:80], _half(b, 80), _half(b, 82)
        out, run = [], 0
        for half in range(2):
            for shift in (0, 2, 4, 6):
                for r in range(2):
                    dl, ml = d * f32(scales[run] & 15), dmin * f32(scales[run] >> 4)
                    run += 1
                    out += [dl * f32((q >> shift) & 3) - ml for q in qs[32 * half + 16 * r:32 * half + 16 * r + 16]]
        return out
    if t == Q3_K:                                           # dequant.rs:278-324
        hmask, qs, sc, d = b[0:32], b[32:96], b[96:108], _half(b, 108)
        scales = [0] * 16
        for j in range(8):
            scales[j], scales[j + 8] = sc[j] & 15, sc[j] >> 4
        for j in range(16):
            scales[j] |= ((sc[8 + j // 4] >> (2 * (j % 4))) & 3) << 4
        out, run, m = [], 0, 1
        for half in range(2):
            for shift in (0, 2, 4, 6):
                for r in range(2):
                    dl = d * f32(scales[run] - 32)
                    run += 1
                    for l in range(16 * r, 16 * r + 16):
                        low = (qs[32 * half + l] >> shift) & 3
                        out.append(dl * f32(low - (0 if hmask[l] & m else 4)))
                m <<= 1
        return out
    raise ValueError(f"ggml type {t}")


def dequantize(t, raw, n):
    """n values of type t from raw bytes; ValueError where the reference returns an error (unknown type, n not a whole
    number of blocks, data shorter than n values)."""
    nb = type_nbytes(t, n)
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    if nb is None or raw.size < nb:
        raise ValueError("bad size")
    vals, bb = BLOCK[t]
    out = []
    with np.errstate(all="ignore"):
        for i in range(n // vals):
            out += _block(t, raw[i * bb:(i + 1) * bb])
    return np.array(out, dtype=np.float32)
