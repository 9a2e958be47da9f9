// tsb_oracle — CPU restatement of the TurboSpark reference's algorithms for the
// speculative-decoding verify path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Nothing in the shipped
// library (libtsb) links, loads or calls it.  Only the test-suite, the smoke
// check and the benchmark's CPU-baseline leg load it, and only as the checker
// or the timed CPU baseline.
//
// The reference is a Rust workspace; no Rust toolchain exists where this is
// built, so every function below restates the published behaviour of the
// reference function it cites (path within the reference project, line range).
// Pinning: the restatement is checked against the reference's own golden
// vectors and known-answer tests (hand-packed Q4_K superblock, ggml-generated
// MXFP4 bytes/floats/codebook/exponent table, residual worked examples,
// select==draw identity, tree fixtures); see tests/golden/.
//
// Arithmetic notes
//  * f32 sums are sequential in index order, as Rust's `iter().sum()` is.
//  * Built with -ffp-contract=off so `a*b-c` rounds twice, as the Rust does.
//  * f64 exp/pow and f32 exp/sin/cos/ln come from glibc, which is what Rust's
//    std lowers to on Linux.
//  * f16 <-> f32 follows the `half` crate 2.7.1 (IEEE round-to-nearest-even).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#define TSO_API extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------
// binary16 / bfloat16 conversions
// ---------------------------------------------------------------------------

// half 2.7.1 `f16::to_f32` (crates/compute/src/quant_1bit.rs:73-77 call site).
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            // subnormal: normalise
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// half 2.7.1 `f16::from_f32`: round-to-nearest-even, overflow to infinity,
// NaN keeps a quiet payload (crates/compute/src/quant_1bit.rs:80-84 call site).
static inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 255) {
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7C00u | 0x0200u | (man >> 13));
    }
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;  // rounds to zero
        man |= 0x800000u;
        int shift = 14 - e;  // 14..24
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1))) half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t half_man = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_man);
    if (rem > 0x1000u || (rem == 0x1000u && (half_man & 1))) out++;  // carry may roll into exp / inf
    return out;
}

// crates/compute/src/quant.rs:14-16
static inline float bf16_to_f32(uint16_t b) {
    uint32_t bits = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// crates/compute/src/quant.rs:29-40
static inline uint16_t f32_to_bf16(float f) {
    uint32_t bits;
    std::memcpy(&bits, &f, 4);
    if (std::isnan(f)) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t lsb = (bits >> 16) & 1u;
    uint32_t bias = 0x7FFFu + lsb;
    return (uint16_t)((bits + bias) >> 16);
}

TSO_API float tso_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
TSO_API uint16_t tso_f32_to_f16(float f) { return f32_to_f16(f); }
TSO_API float tso_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
TSO_API uint16_t tso_f32_to_bf16(float f) { return f32_to_bf16(f); }
TSO_API void tso_f32_to_f16_n(const float* x, uint16_t* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f32_to_f16(x[i]);
}
TSO_API void tso_f16_to_f32_n(const uint16_t* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f16_to_f32(x[i]);
}

// ---------------------------------------------------------------------------
// Q4_K  (crates/compute/src/quant_gguf/q4_k.rs)
// ---------------------------------------------------------------------------

static const int Q4K_ELEMS = 256, Q4K_SUB = 32, Q4K_BYTES = 144, Q4K_SUBS = 8;

// q4_k.rs:43-54 — the 6-bit scale/min of sub-block j out of the 12 packed bytes.
static inline void q4k_scale_min(int j, const uint8_t* p, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = p[j] & 63;
        *m = p[j + 4] & 63;
    } else {
        *sc = (uint8_t)((p[j + 4] & 0xF) | ((p[j - 4] >> 6) << 4));
        *m = (uint8_t)((p[j + 4] >> 4) | ((p[j] >> 6) << 4));
    }
}

// q4_k.rs:67-108
static void dequantize_q4k(const uint8_t* blocks, int64_t n, float* out) {
    int64_t nb = n / Q4K_ELEMS;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t* blk = blocks + b * Q4K_BYTES;
        float d = f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t* packed = blk + 4;
        const uint8_t* qs = blk + 16;
        for (int g = 0; g < Q4K_SUBS / 2; g++) {
            uint8_t sc_lo, m_lo, sc_hi, m_hi;
            q4k_scale_min(2 * g, packed, &sc_lo, &m_lo);
            q4k_scale_min(2 * g + 1, packed, &sc_hi, &m_hi);
            float d_lo = d * (float)sc_lo, min_lo = dmin * (float)m_lo;
            float d_hi = d * (float)sc_hi, min_hi = dmin * (float)m_hi;
            const uint8_t* group = qs + g * Q4K_SUB;
            int64_t at = b * Q4K_ELEMS + g * 2 * Q4K_SUB;
            for (int l = 0; l < Q4K_SUB; l++) {
                uint8_t byte = group[l];
                out[at + l] = d_lo * (float)(byte & 0xF) - min_lo;
                out[at + Q4K_SUB + l] = d_hi * (float)(byte >> 4) - min_hi;
            }
        }
    }
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

// q4_k.rs:126-204 — min/max fit per sub-block; NOT ggml's search.
static void quantize_q4k(const float* row, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / Q4K_ELEMS; b++) {
        const float* block = row + b * Q4K_ELEMS;
        float scales[8], mins[8];
        for (int j = 0; j < 8; j++) {
            const float* sub = block + j * Q4K_SUB;
            float lo = 0.f;
            for (int i = 0; i < Q4K_SUB; i++) lo = std::fmin(lo, sub[i]);
            float hi = lo;
            for (int i = 0; i < Q4K_SUB; i++) hi = std::fmax(hi, sub[i]);
            scales[j] = (hi - lo) / 15.0f;
            mins[j] = -lo;
        }
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; j++) {
            max_scale = std::fmax(max_scale, scales[j]);
            max_min = std::fmax(max_min, mins[j]);
        }
        float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        uint8_t packed[12] = {0};
        for (int j = 0; j < 8; j++) {
            uint8_t ls = (uint8_t)clampf(std::round(scales[j] * inv_scale), 0.f, 63.f);
            uint8_t lm = (uint8_t)clampf(std::round(mins[j] * inv_min), 0.f, 63.f);
            if (j < 4) {
                packed[j] |= ls;
                packed[j + 4] |= lm;
            } else {
                packed[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                packed[j - 4] |= (uint8_t)((ls >> 4) << 6);
                packed[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        uint16_t d = f32_to_f16(max_scale / 63.0f);
        uint16_t dmin = f32_to_f16(max_min / 63.0f);
        uint8_t quants[Q4K_ELEMS] = {0};
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(j, packed, &sc, &m);
            float step = f16_to_f32(d) * (float)sc;
            if (step == 0.f) continue;
            float bias = f16_to_f32(dmin) * (float)m;
            for (int i = 0; i < Q4K_SUB; i++) {
                float w = block[j * Q4K_SUB + i];
                quants[j * Q4K_SUB + i] = (uint8_t)clampf(std::round((w + bias) / step), 0.f, 15.f);
            }
        }
        uint8_t* o = out + b * Q4K_BYTES;
        o[0] = (uint8_t)(d & 0xFF);
        o[1] = (uint8_t)(d >> 8);
        o[2] = (uint8_t)(dmin & 0xFF);
        o[3] = (uint8_t)(dmin >> 8);
        std::memcpy(o + 4, packed, 12);
        for (int g = 0; g < 4; g++) {
            int at = g * 2 * Q4K_SUB;
            for (int l = 0; l < Q4K_SUB; l++)
                o[16 + g * Q4K_SUB + l] = (uint8_t)(quants[at + l] | (quants[at + Q4K_SUB + l] << 4));
        }
    }
}

TSO_API void tso_q4k_scale_min(int j, const uint8_t* packed, uint8_t* sc, uint8_t* m) {
    q4k_scale_min(j, packed, sc, m);
}
TSO_API void tso_dequantize_q4k(const uint8_t* blocks, int64_t n, float* out) { dequantize_q4k(blocks, n, out); }
TSO_API void tso_quantize_q4k(const float* row, int64_t n, uint8_t* out) { quantize_q4k(row, n, out); }

// ---------------------------------------------------------------------------
// Q6_K  (crates/compute/src/quant_gguf/q6_k.rs)
// ---------------------------------------------------------------------------

static const int Q6K_ELEMS = 256, Q6K_BYTES = 210;

// q6_k.rs:52-95
static void dequantize_q6k(const uint8_t* blocks, int64_t n, float* out) {
    for (int64_t b = 0; b < n / Q6K_ELEMS; b++) {
        const uint8_t* base = blocks + b * Q6K_BYTES;
        float d = f16_to_f32((uint16_t)(base[208] | (base[209] << 8)));
        for (int h = 0; h < 2; h++) {
            const uint8_t* ql = base + h * 64;
            const uint8_t* qh = base + 128 + h * 32;
            const int8_t* sc = (const int8_t*)(base + 192 + h * 8);
            int64_t at = b * Q6K_ELEMS + h * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int q[4] = {
                    (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32,
                    (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32,
                    (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32,
                    (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32,
                };
                for (int k = 0; k < 4; k++) out[at + l + k * 32] = d * (float)sc[is + k * 2] * (float)q[k];
            }
        }
    }
}

// q6_k.rs:102-176
static void quantize_q6k(const float* row, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / Q6K_ELEMS; b++) {
        const float* block = row + b * Q6K_ELEMS;
        float scales[16];
        float max_scale = 0.f;
        for (int j = 0; j < 16; j++) {
            float extreme = 0.f;
            for (int i = 0; i < 16; i++) {
                float v = block[j * 16 + i];
                if (std::fabs(v) > std::fabs(extreme)) extreme = v;
            }
            scales[j] = -extreme / 32.0f;
            if (std::fabs(scales[j]) > std::fabs(max_scale)) max_scale = scales[j];
        }
        int8_t sc[16] = {0};
        uint16_t d;
        if (max_scale == 0.f) {
            d = f32_to_f16(0.f);
        } else {
            float iscale = -128.0f / max_scale;
            for (int j = 0; j < 16; j++) {
                float r = std::round(iscale * scales[j]);
                int v = (int)r;
                sc[j] = (int8_t)std::min(127, std::max(-128, v));
            }
            d = f32_to_f16(1.0f / iscale);
        }
        float d_f32 = f16_to_f32(d);
        uint8_t levels[Q6K_ELEMS];
        for (int i = 0; i < Q6K_ELEMS; i++) levels[i] = 32;
        for (int j = 0; j < 16; j++) {
            float step = d_f32 * (float)sc[j];
            if (step == 0.f) continue;
            for (int i = 0; i < 16; i++) {
                float w = block[j * 16 + i];
                int q = (int)clampf(std::round(w / step), -32.f, 31.f);
                levels[j * 16 + i] = (uint8_t)(q + 32);
            }
        }
        uint8_t* o = out + b * Q6K_BYTES;
        uint8_t* ql = o;
        uint8_t* qh = o + 128;
        for (int h = 0; h < 2; h++) {
            int at = h * 128;
            for (int l = 0; l < 32; l++) {
                uint8_t v[4] = {levels[at + l], levels[at + l + 32], levels[at + l + 64], levels[at + l + 96]};
                ql[h * 64 + l] = (uint8_t)((v[0] & 0xF) | ((v[2] & 0xF) << 4));
                ql[h * 64 + l + 32] = (uint8_t)((v[1] & 0xF) | ((v[3] & 0xF) << 4));
                qh[h * 32 + l] =
                    (uint8_t)((v[0] >> 4) | ((v[1] >> 4) << 2) | ((v[2] >> 4) << 4) | ((v[3] >> 4) << 6));
            }
        }
        for (int j = 0; j < 16; j++) o[192 + j] = (uint8_t)sc[j];
        o[208] = (uint8_t)(d & 0xFF);
        o[209] = (uint8_t)(d >> 8);
    }
}

TSO_API void tso_dequantize_q6k(const uint8_t* blocks, int64_t n, float* out) { dequantize_q6k(blocks, n, out); }
TSO_API void tso_quantize_q6k(const float* row, int64_t n, uint8_t* out) { quantize_q6k(row, n, out); }

// ---------------------------------------------------------------------------
// MXFP4  (crates/compute/src/quant_gguf_mxfp4.rs)
// ---------------------------------------------------------------------------

static const int MX_ELEMS = 32, MX_BYTES = 17;
// quant_gguf_mxfp4.rs:76-78 — index 8 is +0.
static const float MXFP4_VALUES[16] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f,
                                       0.f, -1.f, -2.f, -3.f, -4.f, -6.f, -8.f, -12.f};

// quant_gguf_mxfp4.rs:95-102
static inline float mxfp4_scale(uint8_t e) {
    uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// quant_gguf_mxfp4.rs:114-141
static void dequantize_mxfp4(const uint8_t* blocks, int64_t n, float* out) {
    int64_t nb = (n + MX_ELEMS - 1) / MX_ELEMS;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t* base = blocks + b * MX_BYTES;
        float d = mxfp4_scale(base[0]);
        for (int j = 0; j < 16; j++) {
            uint8_t byte = base[1 + j];
            int64_t lo = b * MX_ELEMS + j, hi = lo + 16;
            if (lo < n) out[lo] = MXFP4_VALUES[byte & 0xF] * d;
            if (hi < n) out[hi] = MXFP4_VALUES[byte >> 4] * d;
        }
    }
}

// The reference ships no MXFP4 encoder (quant_gguf_mxfp4.rs:40-48).  This one
// is this project's own, used only to make synthetic weights: per 32-element
// block the smallest shared exponent e with 12*2^(e-128) >= max|w|, then each
// code is the index of the nearest codebook value to w / 2^(e-128), ties to the
// lower index.
static void quantize_mxfp4(const float* row, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / MX_ELEMS; b++) {
        const float* blk = row + b * MX_ELEMS;
        float amax = 0.f;
        for (int i = 0; i < MX_ELEMS; i++) amax = std::fmax(amax, std::fabs(blk[i]));
        int e = 0;
        if (amax > 0.f) {
            e = 128 + (int)std::ceil(std::log2((double)amax / 12.0));
            e = std::min(255, std::max(0, e));
            while (e < 255 && 12.0f * mxfp4_scale((uint8_t)e) < amax) e++;
        }
        float d = mxfp4_scale((uint8_t)e);
        uint8_t codes[MX_ELEMS];
        for (int i = 0; i < MX_ELEMS; i++) {
            float t = blk[i] / d;
            int best = 0;
            float bd = std::fabs(t - MXFP4_VALUES[0]);
            for (int c = 1; c < 16; c++) {
                float dd = std::fabs(t - MXFP4_VALUES[c]);
                if (dd < bd) {
                    bd = dd;
                    best = c;
                }
            }
            codes[i] = (uint8_t)best;
        }
        uint8_t* o = out + b * MX_BYTES;
        o[0] = (uint8_t)e;
        for (int j = 0; j < 16; j++) o[1 + j] = (uint8_t)(codes[j] | (codes[j + 16] << 4));
    }
}

TSO_API float tso_mxfp4_scale(uint8_t e) { return mxfp4_scale(e); }
TSO_API float tso_mxfp4_value(int i) { return MXFP4_VALUES[i & 15]; }
TSO_API void tso_dequantize_mxfp4(const uint8_t* blocks, int64_t n, float* out) { dequantize_mxfp4(blocks, n, out); }
TSO_API void tso_quantize_mxfp4(const float* row, int64_t n, uint8_t* out) { quantize_mxfp4(row, n, out); }

// ---------------------------------------------------------------------------
// Q5_K  (crates/compute/src/quant_gguf/q5_k.rs) and Q8_0 (crates/compute/src/quant_gguf/q8_0.rs)
// ---------------------------------------------------------------------------

static const int Q5K_ELEMS = 256, Q5K_BYTES = 176, Q5K_QH_AT = 16, Q5K_QL_AT = 48;
static const int Q80_ELEMS = 32, Q80_BYTES = 34;

// q5_k.rs:43-100 — Q4_K's scales and mins; the fifth bit of element (group g, half h, byte l) is bit 2g+h of qh[l].
static void dequantize_q5k(const uint8_t* blocks, int64_t n, float* out) {
    for (int64_t b = 0; b < n / Q5K_ELEMS; b++) {
        const uint8_t* blk = blocks + b * Q5K_BYTES;
        float d = f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t* packed = blk + 4;
        const uint8_t* qh = blk + Q5K_QH_AT;
        const uint8_t* ql = blk + Q5K_QL_AT;
        for (int g = 0; g < 4; g++) {
            uint8_t sc_lo, m_lo, sc_hi, m_hi;
            q4k_scale_min(2 * g, packed, &sc_lo, &m_lo);
            q4k_scale_min(2 * g + 1, packed, &sc_hi, &m_hi);
            float d_lo = d * (float)sc_lo, min_lo = dmin * (float)m_lo;
            float d_hi = d * (float)sc_hi, min_hi = dmin * (float)m_hi;
            int64_t at = b * Q5K_ELEMS + g * 64;
            for (int l = 0; l < 32; l++) {
                uint8_t byte = ql[g * 32 + l], hb = qh[l];
                int q_lo = (byte & 0xF) + (((hb >> (2 * g)) & 1) << 4);
                int q_hi = (byte >> 4) + (((hb >> (2 * g + 1)) & 1) << 4);
                out[at + l] = d_lo * (float)q_lo - min_lo;
                out[at + 32 + l] = d_hi * (float)q_hi - min_hi;
            }
        }
    }
}

// The reference carries no Q5_K encoder (its bytes always arrive quantized).  This one exists so tests have
// arbitrary weights in the format: the Q4_K min/max fit above with 31 steps per sub-block instead of 15.
static void quantize_q5k(const float* row, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / Q5K_ELEMS; b++) {
        const float* block = row + b * Q5K_ELEMS;
        float scales[8], mins[8];
        for (int j = 0; j < 8; j++) {
            const float* sub = block + j * 32;
            float lo = 0.f;
            for (int i = 0; i < 32; i++) lo = std::fmin(lo, sub[i]);
            float hi = lo;
            for (int i = 0; i < 32; i++) hi = std::fmax(hi, sub[i]);
            scales[j] = (hi - lo) / 31.0f;
            mins[j] = -lo;
        }
        float max_scale = 0.f, max_min = 0.f;
        for (int j = 0; j < 8; j++) {
            max_scale = std::fmax(max_scale, scales[j]);
            max_min = std::fmax(max_min, mins[j]);
        }
        float inv_scale = max_scale > 0.f ? 63.0f / max_scale : 0.f;
        float inv_min = max_min > 0.f ? 63.0f / max_min : 0.f;
        uint8_t packed[12] = {0};
        for (int j = 0; j < 8; j++) {
            uint8_t ls = (uint8_t)clampf(std::round(scales[j] * inv_scale), 0.f, 63.f);
            uint8_t lm = (uint8_t)clampf(std::round(mins[j] * inv_min), 0.f, 63.f);
            if (j < 4) {
                packed[j] |= ls;
                packed[j + 4] |= lm;
            } else {
                packed[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
                packed[j - 4] |= (uint8_t)((ls >> 4) << 6);
                packed[j] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        uint16_t d = f32_to_f16(max_scale / 63.0f);
        uint16_t dmin = f32_to_f16(max_min / 63.0f);
        uint8_t* o = out + b * Q5K_BYTES;
        std::memset(o, 0, Q5K_BYTES);
        o[0] = (uint8_t)(d & 0xFF), o[1] = (uint8_t)(d >> 8), o[2] = (uint8_t)(dmin & 0xFF), o[3] = (uint8_t)(dmin >> 8);
        std::memcpy(o + 4, packed, 12);
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(j, packed, &sc, &m);
            float step = f16_to_f32(d) * (float)sc;
            if (step == 0.f) continue;
            float bias = f16_to_f32(dmin) * (float)m;
            const int g = j >> 1, h = j & 1;
            for (int l = 0; l < 32; l++) {
                int q = (int)clampf(std::round((block[j * 32 + l] + bias) / step), 0.f, 31.f);
                o[Q5K_QL_AT + g * 32 + l] |= (uint8_t)((q & 0xF) << (4 * h));
                o[Q5K_QH_AT + l] |= (uint8_t)((q >> 4) << (2 * g + h));
            }
        }
    }
}

// q8_0.rs:20-47 — f16 scale, 32 SIGNED weights; out = q * d.
static void dequantize_q8_0(const uint8_t* blocks, int64_t n, float* out) {
    for (int64_t b = 0; b < n / Q80_ELEMS; b++) {
        const uint8_t* blk = blocks + b * Q80_BYTES;
        float d = f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int k = 0; k < Q80_ELEMS; k++) out[b * Q80_ELEMS + k] = (float)(int8_t)blk[2 + k] * d;
    }
}

// q8_0.rs:56-79 — the scale is rounded through f16 before the weights are quantized against it.
static void quantize_q8_0(const float* row, int64_t n, uint8_t* out) {
    for (int64_t b = 0; b < n / Q80_ELEMS; b++) {
        const float* block = row + b * Q80_ELEMS;
        float amax = 0.f;
        for (int k = 0; k < Q80_ELEMS; k++) amax = std::fmax(amax, std::fabs(block[k]));
        uint16_t d = f32_to_f16(amax / 127.0f);
        float df = f16_to_f32(d);
        float inv = df == 0.f ? 0.f : 1.0f / df;
        uint8_t* o = out + b * Q80_BYTES;
        o[0] = (uint8_t)(d & 0xFF), o[1] = (uint8_t)(d >> 8);
        for (int k = 0; k < Q80_ELEMS; k++) {
            int q = (int)std::round(block[k] * inv);  // round half away from zero, as f32::round
            q = q < -127 ? -127 : (q > 127 ? 127 : q);
            o[2 + k] = (uint8_t)(int8_t)q;
        }
    }
}

TSO_API void tso_dequantize_q5k(const uint8_t* blocks, int64_t n, float* out) { dequantize_q5k(blocks, n, out); }
TSO_API void tso_quantize_q5k(const float* row, int64_t n, uint8_t* out) { quantize_q5k(row, n, out); }
TSO_API void tso_dequantize_q8_0(const uint8_t* blocks, int64_t n, float* out) { dequantize_q8_0(blocks, n, out); }
TSO_API void tso_quantize_q8_0(const float* row, int64_t n, uint8_t* out) { quantize_q8_0(row, n, out); }

// ---------------------------------------------------------------------------
// GEMV / small-M GEMM over quantized rows
// q4_k.rs:207-220, q6_k.rs:183-198, quant_gguf_mxfp4.rs:149-162:
// y[r] = sum over the dequantized row times x, sequential f32 in index order.
// kind: 0 = Q4_K, 1 = Q6_K, 2 = MXFP4, 3 = Q5_K, 4 = Q8_0 (q5_k.rs:104-118, q8_0.rs:82-96).
// ---------------------------------------------------------------------------

static int64_t row_bytes_of(int kind, int64_t cols) {
    switch (kind) {
        case 0: return cols / Q4K_ELEMS * Q4K_BYTES;
        case 1: return cols / Q6K_ELEMS * Q6K_BYTES;
        case 3: return cols / Q5K_ELEMS * Q5K_BYTES;
        case 4: return cols / Q80_ELEMS * Q80_BYTES;
        default: return (cols + MX_ELEMS - 1) / MX_ELEMS * MX_BYTES;
    }
}

static void dequant_row(int kind, const uint8_t* row, int64_t cols, float* out) {
    switch (kind) {
        case 0: dequantize_q4k(row, cols, out); break;
        case 1: dequantize_q6k(row, cols, out); break;
        case 3: dequantize_q5k(row, cols, out); break;
        case 4: dequantize_q8_0(row, cols, out); break;
        default: dequantize_mxfp4(row, cols, out); break;
    }
}

TSO_API int64_t tso_row_bytes(int kind, int64_t cols) { return row_bytes_of(kind, cols); }

static void parallel_for(int64_t n, int threads, const std::function<void(int64_t, int64_t)>& fn) {
    if (threads <= 1 || n < 2) {
        fn(0, n);
        return;
    }
    std::vector<std::thread> pool;
    int64_t per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; t++) {
        int64_t lo = t * per, hi = std::min(n, lo + per);
        if (lo >= hi) break;
        pool.emplace_back([=, &fn] { fn(lo, hi); });
    }
    for (auto& th : pool) th.join();
}

// x is [tokens, cols] f32, y is [tokens, rows] f32 (token-major, as the
// reference's batched kernels lay activations out:
// crates/gpu/src/dequant_kquant_gemm_batch.rs:96-126).  Each (token,row) is the
// GEMV formula, so a token's result never depends on the other tokens.
TSO_API void tso_gemm_quant(int kind, const uint8_t* w, int64_t rows, int64_t cols, const float* x, int64_t tokens,
                            float* y, int threads) {
    int64_t rb = row_bytes_of(kind, cols);
    parallel_for(rows, threads, [&](int64_t lo, int64_t hi) {
        std::vector<float> deq((size_t)cols);
        for (int64_t r = lo; r < hi; r++) {
            dequant_row(kind, w + r * rb, cols, deq.data());
            for (int64_t t = 0; t < tokens; t++) {
                const float* xv = x + t * cols;
                float acc = 0.f;
                for (int64_t c = 0; c < cols; c++) acc += deq[c] * xv[c];
                y[t * rows + r] = acc;
            }
        }
    });
}

// ---------------------------------------------------------------------------
// Mixture of experts: routing and the routed feed-forward
// ---------------------------------------------------------------------------
// router_topk_gemma4 (crates/runtime/src/real_forward_dispatch.rs:1135-1158): order by logit descending
// (total_cmp), ties to the lower index; softmax over the selected logits only; times the per-expert scale.
// The weights are what the host then uploads as f16 (crates/runtime/src/families/llama/moe.rs:118-127).
TSO_API void tso_moe_route(const float* logits, int64_t tokens, int64_t n_experts, int64_t k, const float* scale,
                           int32_t* ids, uint16_t* weights_f16) {
    for (int64_t t = 0; t < tokens; t++) {
        const float* row = logits + t * n_experts;
        std::vector<int64_t> order((size_t)n_experts);
        for (int64_t e = 0; e < n_experts; e++) order[(size_t)e] = e;
        std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return row[a] > row[b]; });
        const float mx = row[order[0]];
        std::vector<float> ex((size_t)k);
        float sum = 0.f;
        for (int64_t r = 0; r < k; r++) {
            ex[(size_t)r] = expf(row[order[(size_t)r]] - mx);
            sum += ex[(size_t)r];
        }
        for (int64_t r = 0; r < k; r++) {
            const int64_t e = order[(size_t)r];
            ids[t * k + r] = (int32_t)e;
            weights_f16[t * k + r] = f32_to_f16(ex[(size_t)r] / sum * (scale ? scale[e] : 1.0f));
        }
    }
}

// moe_phase1_gate_up_act_* and moe_phase2_down_reduce_k8_* (crates/gpu/src/shaders/moe_gguf.metal:561-678):
//   acts[slot][f] = half(silu(gate . x) * (up . x));   y[d] = half(float(residual[d]) + sum_slot float(w[slot]) * (down[d] . acts[slot]))
// with the slot sum taken in slot order.  gate_up: per expert [2F rows: gate then up][D cols]; down: per expert [D][F].
TSO_API void tso_moe_ffn(int kind, const uint8_t* gate_up, const uint8_t* down, int64_t n_experts, int64_t d_model, int64_t ffn,
                         const uint16_t* x_f16, const uint16_t* residual_f16, const int32_t* ids, const uint16_t* weights_f16,
                         int64_t tokens, int64_t k, uint16_t* y_f16, int threads) {
    (void)n_experts;
    const int64_t gu_rb = row_bytes_of(kind, d_model), dn_rb = row_bytes_of(kind, ffn);
    parallel_for(tokens, threads, [&](int64_t lo, int64_t hi) {
        std::vector<float> x((size_t)d_model), deq((size_t)std::max(d_model, ffn)), acts((size_t)ffn), partial((size_t)(k * d_model));
        for (int64_t t = lo; t < hi; t++) {
            for (int64_t c = 0; c < d_model; c++) x[(size_t)c] = f16_to_f32(x_f16[t * d_model + c]);
            for (int64_t s = 0; s < k; s++) {
                const int64_t e = ids[t * k + s];
                const uint8_t* gw = gate_up + e * 2 * ffn * gu_rb;
                for (int64_t f = 0; f < ffn; f++) {
                    float g = 0.f, u = 0.f;
                    dequant_row(kind, gw + f * gu_rb, d_model, deq.data());
                    for (int64_t c = 0; c < d_model; c++) g += deq[(size_t)c] * x[(size_t)c];
                    dequant_row(kind, gw + (ffn + f) * gu_rb, d_model, deq.data());
                    for (int64_t c = 0; c < d_model; c++) u += deq[(size_t)c] * x[(size_t)c];
                    const float a = (g / (1.0f + expf(-g))) * u;
                    acts[(size_t)f] = f16_to_f32(f32_to_f16(a));
                }
                const uint8_t* dw = down + e * d_model * dn_rb;
                const float w = f16_to_f32(weights_f16[t * k + s]);
                for (int64_t d = 0; d < d_model; d++) {
                    dequant_row(kind, dw + d * dn_rb, ffn, deq.data());
                    float v = 0.f;
                    for (int64_t f = 0; f < ffn; f++) v += deq[(size_t)f] * acts[(size_t)f];
                    partial[(size_t)(s * d_model + d)] = w * v;
                }
            }
            for (int64_t d = 0; d < d_model; d++) {
                float acc = f16_to_f32(residual_f16[t * d_model + d]);
                for (int64_t s = 0; s < k; s++) acc += partial[(size_t)(s * d_model + d)];
                y_f16[t * d_model + d] = f32_to_f16(acc);
            }
        }
    });
}

// ---------------------------------------------------------------------------
// Row operators with the reference's rounding points
// ---------------------------------------------------------------------------

// crates/compute/src/rms_norm.rs:5-14
TSO_API void tso_rms_norm(const float* x, const float* w, int64_t d, float eps, float* out) {
    float sum_sq = 0.f;
    for (int64_t i = 0; i < d; i++) sum_sq += x[i] * x[i];
    float inv_rms = 1.0f / std::sqrt(sum_sq / (float)d + eps);
    for (int64_t i = 0; i < d; i++) out[i] = x[i] * w[i] * inv_rms;
}

// crates/compute/src/rope.rs:208-255 — NeoX pairing (i, head_dim/2 + i), one
// position for all tokens of the call.
TSO_API void tso_rope_neox(const float* input, int64_t num_tokens, int64_t num_heads, int64_t head_dim,
                           int64_t rotated_pairs, int64_t position, float theta, float* out) {
    int64_t half = head_dim / 2;
    float log_theta = std::log(theta);
    float position_f = (float)position;
    std::vector<float> c((size_t)rotated_pairs), s((size_t)rotated_pairs);
    for (int64_t i = 0; i < rotated_pairs; i++) {
        float exponent = -((float)(2 * i)) / (float)head_dim;
        float angle = position_f * std::exp(exponent * log_theta);
        c[i] = std::cos(angle);
        s[i] = std::sin(angle);
    }
    std::memcpy(out, input, sizeof(float) * (size_t)(num_tokens * num_heads * head_dim));
    for (int64_t t = 0; t < num_tokens; t++)
        for (int64_t h = 0; h < num_heads; h++) {
            int64_t base = (t * num_heads + h) * head_dim;
            for (int64_t i = 0; i < rotated_pairs; i++) {
                float x0 = input[base + i], x1 = input[base + half + i];
                out[base + i] = x0 * c[i] - x1 * s[i];
                out[base + half + i] = x0 * s[i] + x1 * c[i];
            }
        }
}

// crates/gpu/src/shaders/utility.metal:41-52 — (g / (1 + exp(-g))) * u in f32.
TSO_API void tso_silu_mul(const float* gate, const float* up, int64_t n, float* out) {
    for (int64_t i = 0; i < n; i++) out[i] = (gate[i] / (1.0f + std::exp(-gate[i]))) * up[i];
}

// crates/compute/src/attention.rs:53-137 (no sinks), window = None.
// q [nq, hd], k/v [seq, nkv, hd]; out [nq, hd].
static void causal_attention(const float* q, const float* k, const float* v, int64_t hd, int64_t nq, int64_t nkv,
                             int64_t seq_len, float scale, float* out) {
    int64_t group = nq / nkv;
    std::vector<float> scores((size_t)seq_len);
    for (int64_t qh = 0; qh < nq; qh++) {
        int64_t kvh = qh / group;
        const float* qv = q + qh * hd;
        for (int64_t p = 0; p < seq_len; p++) {
            const float* kv = k + (p * nkv + kvh) * hd;
            float dot = 0.f;
            for (int64_t i = 0; i < hd; i++) dot += qv[i] * kv[i];
            scores[p] = dot * scale;
        }
        float mx = -std::numeric_limits<float>::infinity();
        for (int64_t p = 0; p < seq_len; p++) mx = std::fmax(mx, scores[p]);
        for (int64_t p = 0; p < seq_len; p++) scores[p] = std::exp(scores[p] - mx);
        float sum = 0.f;
        for (int64_t p = 0; p < seq_len; p++) sum += scores[p];
        float inv = 1.0f / sum;
        for (int64_t p = 0; p < seq_len; p++) scores[p] *= inv;
        int64_t stride = nkv * hd;
        for (int64_t d = 0; d < hd; d++) {
            const float* col = v + kvh * hd + d;
            float acc = 0.f;
            for (int64_t p = 0; p < seq_len; p++) acc += scores[p] * col[p * stride];
            out[qh * hd + d] = acc;
        }
    }
}

TSO_API void tso_causal_attention(const float* q, const float* k, const float* v, int64_t hd, int64_t nq, int64_t nkv,
                                  int64_t seq_len, float scale, float* out) {
    causal_attention(q, k, v, hd, nq, nkv, seq_len, scale, out);
}

// crates/compute/src/attention.rs:159-197 — attention over the selected rows
// only, in the order given (a tree row = committed prefix then its root path).
TSO_API void tso_indexed_attention(const float* q, const float* k, const float* v, const int64_t* positions,
                                   int64_t npos, int64_t hd, int64_t nq, int64_t nkv, float scale, float* out) {
    int64_t row = nkv * hd;
    std::vector<float> ks((size_t)(npos * row)), vs((size_t)(npos * row));
    for (int64_t i = 0; i < npos; i++) {
        std::memcpy(&ks[i * row], k + positions[i] * row, sizeof(float) * row);
        std::memcpy(&vs[i * row], v + positions[i] * row, sizeof(float) * row);
    }
    causal_attention(q, ks.data(), vs.data(), hd, nq, nkv, npos, scale, out);
}

// ---------------------------------------------------------------------------
// Selection  (crates/selection/src)
// ---------------------------------------------------------------------------

// derive.rs:33-38
static inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
// derive.rs:20-31 (seeded arm only; the clock arm is not reproducible by design)
static inline uint64_t derive_step_value(uint64_t seed, uint64_t position) {
    return mix64(seed ^ (position * 0x9E3779B97F4A7C15ull));
}
// derive.rs:42-45
static inline double to_unit_interval(uint64_t v) { return (double)(v >> 11) * (1.0 / (double)(1ull << 53)); }

TSO_API uint64_t tso_derive_step_value(uint64_t seed, uint64_t position) { return derive_step_value(seed, position); }
TSO_API double tso_to_unit_interval(uint64_t v) { return to_unit_interval(v); }

// shaping.rs:40-50.  top_p <= 0 means None; min_p <= 0 means None.
struct TsoShaping {
    double temperature;
    uint32_t top_k;
    uint32_t _pad;
    double top_p;
    double repetition_penalty;
    double presence_penalty;
    double frequency_penalty;
    double min_p;
    uint64_t seed;
};

struct Shaped {
    std::vector<uint32_t> support;
    std::vector<double> probs;
};

// truncation.rs:79-99 — descending key, NaN last, ties ascending index.
static inline bool rank_before(const std::vector<double>& keys, uint32_t a, uint32_t b) {
    double ka = keys[a], kb = keys[b];
    bool na = std::isnan(ka), nb = std::isnan(kb);
    if (!na && !nb) {
        if (ka != kb) return ka > kb;
        return a < b;
    }
    if (na && nb) return a < b;
    return nb;  // a real key sorts before a NaN one
}

// penalty.rs:15-39
static void apply_repetition_penalty(std::vector<float>& scores, const int32_t* history, int64_t nh, double penalty) {
    if (penalty == 1.0 || nh == 0) return;
    std::unordered_set<int32_t> seen(history, history + nh);
    float p = (float)penalty;
    p = clampf(p, std::numeric_limits<float>::min(), std::numeric_limits<float>::max());
    for (int32_t id : seen) {
        if (id < 0 || (size_t)id >= scores.size()) continue;
        float s = scores[id];
        float att = s > 0.f ? s / p : s * p;
        scores[id] = clampf(att, -std::numeric_limits<float>::max(), std::numeric_limits<float>::max());
    }
}

// penalty.rs:59-82
static void apply_presence_frequency(std::vector<float>& scores, const int32_t* suffix, int64_t ns, double presence,
                                     double frequency) {
    if ((presence == 0.0 && frequency == 0.0) || ns == 0) return;
    std::unordered_map<int32_t, uint32_t> counts;
    for (int64_t i = 0; i < ns; i++) counts[suffix[i]]++;
    for (auto& kv : counts) {
        if (kv.first < 0 || (size_t)kv.first >= scores.size()) continue;
        double pen = presence + frequency * (double)kv.second;
        scores[kv.first] -= (float)pen;
    }
}

// choose.rs:283-291
static uint32_t argmax_first(const std::vector<float>& s) {
    size_t best = 0;
    for (size_t i = 1; i < s.size(); i++)
        if (s[i] > s[best]) best = i;
    return (uint32_t)best;
}

// choose.rs:111-232.  Returns 0 on success, 1 on a non-finite entry, 2 on an
// empty domain.  `exps` stays empty on the deterministic arm.
static int shape_candidates(const uint16_t* raw, int64_t v, const TsoShaping& cfg, const int32_t* history, int64_t nh,
                            uint64_t position, std::vector<float>& working, std::vector<double>& exps,
                            std::vector<uint32_t>& surviving, double* sum_out) {
    if (v <= 0) return 2;
    working.resize((size_t)v);
    bool all_finite = true;
    for (int64_t i = 0; i < v; i++) {
        float f = f16_to_f32(raw[i]);
        all_finite &= std::isfinite(f);
        working[i] = f;
    }
    if (!all_finite) return 1;
    exps.clear();
    surviving.clear();
    if (cfg.temperature == 0.0) {
        surviving.push_back(argmax_first(working));
        *sum_out = 1.0;
        return 0;
    }
    apply_repetition_penalty(working, history, nh, cfg.repetition_penalty);
    int64_t generated = std::min<int64_t>((int64_t)position, nh);
    apply_presence_frequency(working, history + (nh - generated), generated, cfg.presence_penalty,
                             cfg.frequency_penalty);

    float mxf = -std::numeric_limits<float>::infinity();
    for (int64_t i = 0; i < v; i++) mxf = std::fmax(mxf, working[i]);
    double mx = (double)mxf;
    exps.resize((size_t)v);
    for (int64_t i = 0; i < v; i++) exps[i] = std::exp((double)working[i] - mx);
    double sum = 0.0;
    for (int64_t i = 0; i < v; i++) sum += exps[i];

    // truncation.rs:143-236: whole-domain rank when top_k == 0, else the top-k
    // prefix of the same total order (the kth-largest cut is an optimisation
    // that yields the identical list).
    std::vector<uint32_t> ranked((size_t)v);
    for (int64_t i = 0; i < v; i++) ranked[i] = (uint32_t)i;
    auto cmp = [&](uint32_t a, uint32_t b) { return rank_before(exps, a, b); };
    if (cfg.top_k == 0 || (int64_t)cfg.top_k >= v) {
        std::sort(ranked.begin(), ranked.end(), cmp);
    } else {
        std::partial_sort(ranked.begin(), ranked.begin() + cfg.top_k, ranked.end(), cmp);
        ranked.resize(cfg.top_k);
    }

    if (!(cfg.top_p > 0.0)) {
        surviving = ranked;
    } else {
        double cumulative = 0.0;
        for (uint32_t i : ranked) {
            surviving.push_back(i);
            cumulative += exps[i] / sum;
            if (cumulative >= cfg.top_p) break;
        }
        if (surviving.empty() && !ranked.empty()) surviving.push_back(ranked[0]);
    }
    if (cfg.top_k != 0 && surviving.size() > cfg.top_k) surviving.resize(cfg.top_k);
    if (cfg.min_p > 0.0 && !ranked.empty()) {
        uint32_t top = ranked[0];
        double threshold = cfg.min_p * exps[top];
        std::vector<uint32_t> kept;
        for (uint32_t i : surviving)
            if (exps[i] >= threshold) kept.push_back(i);
        surviving.swap(kept);
        if (surviving.empty()) surviving.push_back(top);
    }
    if (surviving.empty()) {
        surviving.push_back(argmax_first(working));
        *sum_out = 1.0;
        return 0;
    }
    *sum_out = sum;
    return 0;
}

// choose.rs:296-321
static void reweight(const std::vector<uint32_t>& surviving, const std::vector<double>& exps, double sum,
                     double temperature, std::vector<double>& out) {
    double inv_t = 1.0 / temperature;
    double top = 0.0;
    for (uint32_t i : surviving) top = std::fmax(top, exps[i] / sum);
    out.resize(surviving.size());
    for (size_t k = 0; k < surviving.size(); k++) {
        double p = exps[surviving[k]] / sum;
        out[k] = top > 0.0 ? std::pow(p / top, inv_t) : std::pow(p, inv_t);
    }
    double total = 0.0;
    for (double w : out) total += w;
    if (total <= 0.0) {
        double n = (double)out.size();
        for (auto& w : out) w = 1.0 / n;
        return;
    }
    for (auto& w : out) w = w / total;
}

// choose.rs:240-281 — the distribution `select` samples from.
static int shaped_distribution(const uint16_t* raw, int64_t v, const TsoShaping& cfg, const int32_t* history,
                               int64_t nh, uint64_t position, Shaped& out) {
    std::vector<float> working;
    std::vector<double> exps;
    double sum = 0.0;
    int rc = shape_candidates(raw, v, cfg, history, nh, position, working, exps, out.support, &sum);
    if (rc) return rc;
    if (cfg.temperature == 0.0) {
        out.probs.assign(1, 1.0);
        return 0;
    }
    if (exps.empty()) {  // defensive-fallback arm returned a single candidate
        out.probs.assign(1, 1.0);
        return 0;
    }
    reweight(out.support, exps, sum, cfg.temperature, out.probs);
    return 0;
}

// distribution.rs:61-66
static double shaped_probability(const Shaped& d, uint32_t token) {
    for (size_t i = 0; i < d.support.size(); i++)
        if (d.support[i] == token) return d.probs[i];
    return 0.0;
}

// distribution.rs:71-83 with an explicit uniform (the caller derives it).
static uint32_t shaped_draw_u(const Shaped& d, double target) {
    double cumulative = 0.0;
    for (size_t i = 0; i < d.probs.size(); i++) {
        cumulative += d.probs[i];
        if (target < cumulative) return d.support[i];
    }
    return d.support.back();
}

// distribution.rs:96-125.  Returns false for None.
static bool residual(const Shaped& p, const Shaped& q, Shaped& out) {
    const double EPS = 1e-12;
    std::unordered_map<uint32_t, double> q_mass;
    q_mass.reserve(q.support.size());
    for (size_t i = 0; i < q.support.size(); i++) q_mass.emplace(q.support[i], q.probs[i]);  // first occurrence kept
    out.support.clear();
    out.probs.clear();
    for (size_t i = 0; i < p.support.size(); i++) {
        auto it = q_mass.find(p.support[i]);
        double qm = it == q_mass.end() ? 0.0 : it->second;
        double mass = std::fmax(p.probs[i] - qm, 0.0);
        if (mass > 0.0) {
            out.support.push_back(p.support[i]);
            out.probs.push_back(mass);
        }
    }
    double total = 0.0;
    for (double m : out.probs) total += m;
    if (total < EPS || out.support.empty()) return false;
    for (auto& m : out.probs) m /= total;
    return true;
}

// choose.rs:62-109 — `select`.  Writes the chosen id; returns 0/1/2 as above.
static int select_token(const uint16_t* raw, int64_t v, const TsoShaping& cfg, const int32_t* history, int64_t nh,
                        uint64_t position, int32_t* chosen) {
    Shaped d;
    int rc = shaped_distribution(raw, v, cfg, history, nh, position, d);
    if (rc) return rc;
    if (cfg.temperature == 0.0) {
        *chosen = (int32_t)d.support[0];
        return 0;
    }
    double target = to_unit_interval(derive_step_value(cfg.seed, position));
    *chosen = (int32_t)shaped_draw_u(d, target);
    return 0;
}

TSO_API int tso_select(const uint16_t* logits, int64_t v, const TsoShaping* cfg, const int32_t* history, int64_t nh,
                       uint64_t position, int32_t* chosen) {
    return select_token(logits, v, *cfg, history, nh, position, chosen);
}

// Materialise a shaped distribution: returns the support size (negative on
// error) and fills support/probs up to `cap` entries.
TSO_API int64_t tso_shaped_distribution(const uint16_t* logits, int64_t v, const TsoShaping* cfg,
                                        const int32_t* history, int64_t nh, uint64_t position, uint32_t* support,
                                        double* probs, int64_t cap) {
    Shaped d;
    int rc = shaped_distribution(logits, v, *cfg, history, nh, position, d);
    if (rc) return -rc;
    int64_t n = (int64_t)d.support.size();
    for (int64_t i = 0; i < std::min(n, cap); i++) {
        support[i] = d.support[i];
        probs[i] = d.probs[i];
    }
    return n;
}

// residual over two explicit distributions; returns size, 0 for None.
TSO_API int64_t tso_residual(const uint32_t* ps, const double* pp, int64_t np, const uint32_t* qs, const double* qp,
                             int64_t nq, uint32_t* os, double* op) {
    Shaped p, q, r;
    p.support.assign(ps, ps + np);
    p.probs.assign(pp, pp + np);
    q.support.assign(qs, qs + nq);
    q.probs.assign(qp, qp + nq);
    if (!residual(p, q, r)) return 0;
    for (size_t i = 0; i < r.support.size(); i++) {
        os[i] = r.support[i];
        op[i] = r.probs[i];
    }
    return (int64_t)r.support.size();
}

TSO_API uint32_t tso_draw(const uint32_t* s, const double* p, int64_t n, double target) {
    Shaped d;
    d.support.assign(s, s + n);
    d.probs.assign(p, p + n);
    return shaped_draw_u(d, target);
}

// ---------------------------------------------------------------------------
// One round's acceptance  (crates/runtime/src/speculative.rs:694-754,861-879)
//
// target_logits: (k+1) rows of V f16 (row i predicts the token after feed[i]);
// draft_logits: k rows (the drafter's logits each proposal was drawn from);
// uniforms: the u64 values the reference would obtain from
// derive_step_value(seed, draw_step) for draw_step = first, first+1, ... —
// passed in so any generator can feed both this oracle and the kernel; each is
// mapped through to_unit_interval.  History grows by each accepted proposal
// before the next row is shaped, and `generated` counts committed tokens.
// Stop/budget handling is the loop's business, not this function's.
//
// out_tokens[0..accepted) are the accepted proposals, out_tokens[accepted] is
// the corrected or bonus token.  margins[0] = min |r*q(x) - p(x)| over tested
// proposals, margins[1] = |target - cumulative| gap at the final draw.
// Returns draws consumed (<0 on error).
// ---------------------------------------------------------------------------
TSO_API int tso_accept_round(const uint16_t* target_logits, const uint16_t* draft_logits, int64_t v, int k,
                             const int32_t* proposals, const TsoShaping* cfg, const uint64_t* uniforms,
                             const int32_t* history, int64_t nh, uint64_t generated, int32_t* out_accepted,
                             int32_t* out_tokens, double* margins) {
    std::vector<int32_t> hist(history, history + nh);
    const uint64_t generated0 = generated;
    int accepted = 0;
    int draws = 0;
    bool sampled = cfg->temperature != 0.0;
    double m_acc = std::numeric_limits<double>::infinity(), m_draw = std::numeric_limits<double>::infinity();
    int32_t corrected = -1;
    auto draw_with_margin = [&](const Shaped& d, double target) {
        double cumulative = 0.0;
        for (size_t i = 0; i < d.probs.size(); i++) {
            double before = cumulative;
            cumulative += d.probs[i];
            if (target < cumulative) {
                m_draw = std::fmin(cumulative - target, i == 0 ? cumulative - target : target - before);
                return d.support[i];
            }
        }
        m_draw = 0.0;
        return d.support.back();
    };
    for (int i = 0; i < k; i++) {
        const uint16_t* row = target_logits + (int64_t)i * v;
        int32_t x = proposals[i];
        if (sampled) {
            Shaped p, q;
            int rc = shaped_distribution(row, v, *cfg, hist.data(), (int64_t)hist.size(), generated, p);
            if (rc) return -rc;
            // q is the distribution proposal i was DRAWN from: shaped when the drafter ran, with the history and the
            // generated count of the round's start (speculative.rs:636-648 stores it, :708 reads it back) - the
            // proposals accepted since then are not part of it
            rc = shaped_distribution(draft_logits + (int64_t)i * v, v, *cfg, hist.data(), nh, generated0, q);
            if (rc) return -rc;
            double r = to_unit_interval(uniforms[draws++]);
            double qx = shaped_probability(q, (uint32_t)x), px = shaped_probability(p, (uint32_t)x);
            m_acc = std::fmin(m_acc, std::fabs(r * qx - px));
            if (r * qx <= px) {
                accepted++;
                out_tokens[i] = x;
                hist.push_back(x);
                generated++;
            } else {
                Shaped res;
                double target = to_unit_interval(uniforms[draws++]);
                corrected = residual(p, q, res) ? (int32_t)draw_with_margin(res, target)
                                                : (int32_t)draw_with_margin(p, target);
                break;
            }
        } else {
            int32_t t;
            int rc = select_token(row, v, *cfg, hist.data(), (int64_t)hist.size(), generated, &t);
            if (rc) return -rc;
            if (t != x) break;
            accepted++;
            out_tokens[i] = x;
            hist.push_back(x);
            generated++;
        }
    }
    const uint16_t* brow = target_logits + (int64_t)accepted * v;
    if (corrected >= 0) {
        out_tokens[accepted] = corrected;
    } else if (sampled) {
        Shaped p;
        int rc = shaped_distribution(brow, v, *cfg, hist.data(), (int64_t)hist.size(), generated, p);
        if (rc) return -rc;
        double target = to_unit_interval(uniforms[draws++]);
        out_tokens[accepted] = (int32_t)draw_with_margin(p, target);
    } else {
        int32_t t;
        int rc = select_token(brow, v, *cfg, hist.data(), (int64_t)hist.size(), generated, &t);
        if (rc) return -rc;
        out_tokens[accepted] = t;
    }
    *out_accepted = accepted;
    if (margins) {
        margins[0] = m_acc;
        margins[1] = m_draw;
    }
    return draws;
}

// Draft-side draw (speculative.rs:636-647): token = q.draw(uniform), q shaped
// from the drafter's logits.
TSO_API int tso_sample(const uint16_t* logits, int64_t v, const TsoShaping* cfg, uint64_t uniform,
                       const int32_t* history, int64_t nh, uint64_t generated, int32_t* token, double* margin) {
    Shaped d;
    int rc = shaped_distribution(logits, v, *cfg, history, nh, generated, d);
    if (rc) return -rc;
    if (cfg->temperature == 0.0) {
        *token = (int32_t)d.support[0];
        if (margin) *margin = 1.0;
        return 0;
    }
    double target = to_unit_interval(uniform);
    double cumulative = 0.0;
    for (size_t i = 0; i < d.probs.size(); i++) {
        double before = cumulative;
        cumulative += d.probs[i];
        if (target < cumulative) {
            *token = (int32_t)d.support[i];
            if (margin) *margin = std::fmin(cumulative - target, i == 0 ? cumulative - target : target - before);
            return 0;
        }
    }
    *token = (int32_t)d.support.back();
    if (margin) *margin = 0.0;
    return 0;
}

// ---------------------------------------------------------------------------
// Trees  (crates/runtime/src/dflash_tree.rs, families/qwen/batched_scratch.rs)
// ---------------------------------------------------------------------------

// batched_scratch.rs:97-124 — depth[] and root paths from a slot-parent array.
// paths is [n, max_depth] padded with -1; returns 0, or the 1-based index of
// the first offending slot.
TSO_API int tso_tree_spec(const int32_t* parent, int n, int32_t* depth, int32_t* paths, int max_depth) {
    if (n < 1 || parent[0] != -1) return 1;
    for (int i = 0; i < n * max_depth; i++) paths[i] = -1;
    for (int s = 0; s < n; s++) {
        if (s == 0) {
            depth[0] = 0;
            paths[0] = 0;
            continue;
        }
        int p = parent[s];
        if (p < 0 || p >= s) return s + 1;
        depth[s] = depth[p] + 1;
        if (depth[s] + 1 > max_depth) return s + 1;
        for (int i = 0; i <= depth[p]; i++) paths[s * max_depth + i] = paths[p * max_depth + i];
        paths[s * max_depth + depth[s]] = s;
    }
    return 0;
}

// dflash_tree.rs:119-124 — node i sits in slot i+1; a root node's parent is the anchor (slot 0).
TSO_API void tso_tree_slot_parents(const int32_t* node_parent, int nodes, int32_t* slot_parent) {
    slot_parent[0] = -1;
    for (int i = 0; i < nodes; i++) slot_parent[i + 1] = node_parent[i] < 0 ? 0 : node_parent[i] + 1;
}

// dflash_tree.rs:96-116 — greedy walk: at the current node, the target's pick
// is accepted when a child of that node carries it (lowest node id first).
// target_pick[slot] is the target's choice at that slot's row (slot 0 = anchor).
TSO_API int tso_tree_accept(const int32_t* node_parent, const int32_t* node_token, int nodes,
                            const int32_t* target_pick, int32_t* accepted_nodes) {
    int n = 0;
    int at = -1;
    for (;;) {
        int32_t want = target_pick[at + 1];
        int hit = -1;
        for (int id = 0; id < nodes; id++)
            if (node_parent[id] == at && node_token[id] == want) {
                hit = id;
                break;
            }
        if (hit < 0) return n;
        accepted_nodes[n++] = hit;
        at = hit;
    }
}

// dflash_tree.rs:30-82 — best-first tree with a fixed per-depth score table
// (scores[depth][cand], branch candidates per depth), child scores through an
// f64 softmax, ties: shallower then lower candidate.
TSO_API int tso_best_first_tree(const float* scores, int depth_max, int branch, int nodes, int32_t* out_depth,
                                int32_t* out_cand, int32_t* out_parent) {
    struct Node {
        int depth, cand, parent;
    };
    auto softmax = [&](const float* s) {
        float mf = -std::numeric_limits<float>::infinity();
        for (int i = 0; i < branch; i++) mf = std::fmax(mf, s[i]);
        double m = (double)mf;
        std::vector<double> e((size_t)branch);
        double z = 0.0;
        for (int i = 0; i < branch; i++) e[i] = std::exp((double)s[i] - m);
        for (int i = 0; i < branch; i++) z += e[i];
        for (auto& v : e) v /= z;
        return e;
    };
    int n_out = 0;
    if (depth_max == 0 || nodes == 0) return 0;
    std::vector<std::pair<double, Node>> frontier;
    {
        auto p = softmax(scores);
        for (int c = 0; c < branch; c++) frontier.push_back({p[c], Node{0, c, -1}});
    }
    while (n_out < nodes && !frontier.empty()) {
        size_t best = 0;
        for (size_t i = 1; i < frontier.size(); i++) {
            double s = frontier[i].first, bs = frontier[best].first;
            const Node &n = frontier[i].second, &bn = frontier[best].second;
            if (s > bs || (s == bs && (n.depth < bn.depth || (n.depth == bn.depth && n.cand < bn.cand)))) best = i;
        }
        auto picked = frontier[best];
        frontier[best] = frontier.back();  // swap_remove
        frontier.pop_back();
        int id = n_out;
        out_depth[id] = picked.second.depth;
        out_cand[id] = picked.second.cand;
        out_parent[id] = picked.second.parent;
        n_out++;
        if (n_out < nodes && picked.second.depth + 1 < depth_max) {
            auto p = softmax(scores + (size_t)(picked.second.depth + 1) * branch);
            for (int c = 0; c < branch; c++)
                frontier.push_back({picked.first * p[c], Node{picked.second.depth + 1, c, id}});
        }
    }
    return n_out;
}

// ---------------------------------------------------------------------------
// KV compaction  (crates/gpu/src/dflash_conv.rs:192-259 gather_rows_fp16;
// families/qwen/dflash_tree.rs:106-207): dst[r] = src[map[r]] in place, legal
// only when map is strictly increasing with map[r] >= r.
// ---------------------------------------------------------------------------
TSO_API int tso_gather_rows_inplace(uint16_t* rows, int64_t row_elems, const uint32_t* map, int n) {
    for (int r = 0; r < n; r++) {
        if (map[r] < (uint32_t)r) return 1;
        if (r > 0 && map[r] <= map[r - 1]) return 1;
    }
    for (int r = 0; r < n; r++)
        if (map[r] != (uint32_t)r) std::memmove(rows + r * row_elems, rows + map[r] * row_elems, 2 * row_elems);
    return 0;
}

// ---------------------------------------------------------------------------
// Adaptive depth  (crates/runtime/src/speculative_adaptive.rs:104-225)
// ---------------------------------------------------------------------------
struct TsoAdaptive {
    int64_t floor, cap, cur, climb, pressure;
};
static int64_t climb_threshold(int64_t depth) {
    if (depth <= 1) return 2;
    if (depth <= 3) return 8;
    if (depth == 4) return 6;
    return 4;
}
TSO_API void tso_adaptive_init(TsoAdaptive* a, int64_t floor, int64_t cap) {
    cap = std::max<int64_t>(cap, 1);
    floor = std::min(std::max<int64_t>(floor, 1), cap);
    *a = TsoAdaptive{floor, cap, floor, 0, 0};
}
TSO_API int64_t tso_adaptive_tile_cap(int64_t cap, int64_t tile_rows) {
    if (tile_rows < 0) return cap;
    int64_t r = tile_rows > 0 ? tile_rows - 1 : 0;
    return std::min(cap, std::max<int64_t>(r, 1));
}
TSO_API void tso_adaptive_observe(TsoAdaptive* a, int64_t offered, int64_t accepted) {
    if (offered == 0) return;
    accepted = std::min(accepted, offered);
    if (accepted == offered) {
        a->pressure = 0;
        if (a->cur < a->cap) {
            a->climb++;
            if (a->climb >= climb_threshold(a->cur)) {
                a->cur++;
                a->climb = 0;
            }
        }
    } else {
        a->climb = 0;
        if (a->cur > a->floor) {
            a->pressure += offered - accepted;
            if (a->pressure >= 2) {
                a->cur--;
                a->pressure = 0;
            }
        }
    }
}

#include "tsb_oracle_model.inc"
