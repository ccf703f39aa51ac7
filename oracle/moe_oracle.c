/* TEST INFRASTRUCTURE, NOT PRODUCT: a plain-C restatement of the reference engine's mixture-of-experts layer arithmetic
 * (router, dispatch, block-format decoders and quantisers, combine).  Only the tests, the smoke check and the bench's
 * cpu_baseline leg may load this library; the shipped CUDA path never does.
 *
 * Parity pins (checked by tests/test_oracle_pins.py): the decoders and quantisers against the reference's own ggml code
 * compiled from its checkout (oracle/_ref/libref_cpu.so) and against committed golden hashes generated from it; the
 * router logits and the sigmoid / sqrt-softplus selection against the reference CUDA kernels run on a B200
 * (oracle/_ref/libref_gpu.so) and the frozen id+weight hash of the reference's router parity test.
 *
 * Every function cites the reference file:line it follows (paths inside the reference project).
 * Build: gcc -O2 -std=gnu11 -fPIC -shared -ffp-contract=off moe_oracle.c -lm   (no FMA contraction: every fused multiply-add
 * below is an explicit fmaf, as in the CUDA sources it restates).
 */
#include <math.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------ fp16 <-> fp32 */
static float h2f(uint16_t h) {
    const uint32_t s = (uint32_t) (h & 0x8000) << 16;
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF, u;
    if (e == 0) {
        if (m == 0) u = s;
        else {
            int sh = 0;
            while (!(m & 0x400)) { m <<= 1; ++sh; }
            m &= 0x3FF;
            u = s | ((uint32_t) (113 - sh) << 23) | (m << 13);
        }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, as F16C / __float2half_rn */
static uint16_t f2h(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint16_t s = (uint16_t) ((u >> 16) & 0x8000);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t) (s | 0x7C00 | ((a > 0x7F800000u) ? 0x200 | ((a >> 13) & 0x3FF) : 0));
    if (a >= 0x477FF000u) return (uint16_t) (s | 0x7C00);          /* rounds to inf */
    if (a < 0x33000001u) return s;                                  /* rounds to zero */
    int e = (int) (a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }              /* subnormal half */
    else { shift = 13; base = (uint32_t) (e + 15) << 10; m &= 0x7FFFFFu; }
    const uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    uint32_t r = base + q;
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t) (s | r);
}

EXPORT float orc_h2f(uint16_t h) { return h2f(h); }
EXPORT uint16_t orc_f2h(float f) { return f2h(f); }

/* ------------------------------------------------------------------------------------------------ block formats */
enum { T_Q5_0 = 6, T_Q5_1 = 7, T_IQ4_NL = 20, T_IQ4_XS = 23, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ1_M = 29, T_NVFP4 = 40,
       T_Q2_K = 10, T_Q3_K = 11, T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ3_S = 21, T_IQ2_S = 22, T_Q2_0 = 42 };

/* include/basalt/ggml/ggml_common.h:1029-1031 - E2M1 values, doubled */
static const int8_t kFp4x2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

/* src/kernels/cpu/ggml/ggml_quants.c:1397-1406 - UE4M3 as ggml reads it: bit 7 ignored, 0 and 0x7F give 0, and the value is
 * halved because the E2M1 table is doubled. */
static float ue4m3_half(uint8_t b) {
    b &= 0x7F;
    if (b == 0 || b == 0x7F) return 0.0f;
    const int e = b >> 3, m = b & 7;
    const float raw = e == 0 ? ldexpf((float) m, -9) : ldexpf(1.0f + (float) m / 8.0f, e - 7);
    return raw * 0.5f;
}
EXPORT float orc_ue4m3_half(uint8_t b) { return ue4m3_half(b); }

static const uint16_t kIq1Grid[2048] = {
#include "../basalt_b200/csrc/iq1_grid_u16.inc"
};
/* the IQ2 and IQ3 codebooks, packed: iq2xxs 256, iq2xs 512, iq2s 1024 points (8 coordinates x 2 bits -> 8, 25, 43), iq3xxs 256 points
 * (4 x 3 bits -> 4, 12, ..., 52, 62), iq3s 512 points (4 x 3 bits -> 1, 3, ..., 15); include/basalt/ggml/ggml_common.h:444-1020 */
static const uint16_t kIqGrids[2560] = {
#include "../basalt_b200/csrc/iq_grids_u16.inc"
};
enum { G_IQ2XXS = 0, G_IQ2XS = 256, G_IQ2S = 768, G_IQ3XXS = 1792, G_IQ3S = 2048 };

EXPORT int64_t orc_row_bytes(int type, int64_t n) {
    switch (type) {
        case T_NVFP4: return n % 64 ? 0 : n / 64 * 36;     /* ggml_common.h:146-156 */
        case T_Q6_K: return n % 256 ? 0 : n / 256 * 210;   /* ggml_common.h:279-285 */
        case T_IQ1_M: return n % 256 ? 0 : n / 256 * 56;   /* ggml_common.h:350-362 */
        case T_Q5_0: return n % 32 ? 0 : n / 32 * 22;      /* block_q5_0: d, qh[4], qs[16] */
        case T_Q5_1: return n % 32 ? 0 : n / 32 * 24;      /* block_q5_1: d, m, qh[4], qs[16] */
        case T_IQ4_NL: return n % 32 ? 0 : n / 32 * 18;    /* block_iq4_nl: d, qs[16] */
        case T_IQ4_XS: return n % 256 ? 0 : n / 256 * 136; /* block_iq4_xs: d, scales_h, scales_l[4], qs[128] */
        case T_Q8_0: return n % 32 ? 0 : n / 32 * 34;      /* block_q8_0: fp16 d, int8 qs[32] */
        case T_Q4_K: return n % 256 ? 0 : n / 256 * 144;   /* block_q4_K: d, dmin, scales[12], qs[128] */
        case T_Q5_K: return n % 256 ? 0 : n / 256 * 176;   /* block_q5_K: d, dmin, scales[12], qh[32], qs[128] */
        case T_Q2_0: return n % 64 ? 0 : n / 64 * 18;      /* block_q2_0: d, qs[16] (ggml_common.h:140-145) */
        case T_Q2_K: return n % 256 ? 0 : n / 256 * 84;    /* block_q2_K: scales[16], qs[64], d, dmin */
        case T_Q3_K: return n % 256 ? 0 : n / 256 * 110;   /* block_q3_K: hmask[32], qs[64], scales[12], d */
        case T_IQ2_XXS: return n % 256 ? 0 : n / 256 * 66; /* block_iq2_xxs: d, qs[32] uint16 */
        case T_IQ2_XS: return n % 256 ? 0 : n / 256 * 74;  /* block_iq2_xs: d, qs[32] uint16, scales[8] */
        case T_IQ2_S: return n % 256 ? 0 : n / 256 * 82;   /* block_iq2_s: d, qs[64], qh[8], scales[8] */
        case T_IQ3_XXS: return n % 256 ? 0 : n / 256 * 98; /* block_iq3_xxs: d, qs[96] */
        case T_IQ3_S: return n % 256 ? 0 : n / 256 * 110;  /* block_iq3_s: d, qs[64], qh[8], signs[32], scales[4] */
        case T_IQ1_S: return n % 256 ? 0 : n / 256 * 50;   /* block_iq1_s: d, qs[32], qh[16] uint16 */
        default: return 0;
    }
}

/* src/kernels/cpu/ggml/ggml_quants.c:1408-1422 */
static void dequant_nvfp4(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 64; ++i, b += 36, y += 64)
        for (int s = 0; s < 4; ++s) {
            const float d = ue4m3_half(b[s]);
            const uint8_t* q = b + 4 + 8 * s;
            for (int j = 0; j < 8; ++j) {
                y[16 * s + j] = (float) kFp4x2[q[j] & 15] * d;
                y[16 * s + j + 8] = (float) kFp4x2[q[j] >> 4] * d;
            }
        }
}

/* src/kernels/cpu/ggml/ggml_quants.c:1048-1075.  Block = ql[128] | qh[64] | scales[16] (int8) | d (fp16). */
static void dequant_q6k(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 210, y += 256) {
        const uint8_t *ql = b, *qh = b + 128;
        const int8_t* sc = (const int8_t*) (b + 192);
        uint16_t dh;
        memcpy(&dh, b + 208, 2);
        const float d = h2f(dh);
        for (int half = 0; half < 2; ++half)
            for (int l = 0; l < 32; ++l) {
                const int is = 8 * half + l / 16;
                const uint8_t h = qh[32 * half + l];
                const uint8_t lo0 = ql[64 * half + l], lo1 = ql[64 * half + 32 + l];
                const int8_t q1 = (int8_t) ((lo0 & 15) | ((h & 3) << 4)) - 32;
                const int8_t q2 = (int8_t) ((lo1 & 15) | (((h >> 2) & 3) << 4)) - 32;
                const int8_t q3 = (int8_t) ((lo0 >> 4) | (((h >> 4) & 3) << 4)) - 32;
                const int8_t q4 = (int8_t) ((lo1 >> 4) | (((h >> 6) & 3) << 4)) - 32;
                float* o = y + 128 * half + l;
                o[0] = d * sc[is + 0] * q1;
                o[32] = d * sc[is + 2] * q2;
                o[64] = d * sc[is + 4] * q3;
                o[96] = d * sc[is + 6] * q4;
            }
    }
}

/* src/kernels/cpu/ggml/ggml_quants.c:1266-1314.  Block = qs[32] | qh[16] | scales[8]; the fp16 super-scale is spread over the
 * top nibbles of the four 16-bit scale words. */
static void dequant_iq1m(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 56) {
        const uint8_t *qs = b, *qh = b + 32;
        uint16_t sc[4];
        memcpy(sc, b + 48, 8);
        const uint16_t dh = (uint16_t) ((sc[0] >> 12) | ((sc[1] >> 8) & 0x00F0) | ((sc[2] >> 4) & 0x0F00) | (sc[3] & 0xF000));
        const float d = h2f(dh);
        for (int ib = 0; ib < 8; ++ib, qs += 4, qh += 2) {
            const float dl[2] = {d * (float) (2 * ((sc[ib / 2] >> (6 * (ib % 2) + 0)) & 7) + 1),
                                 d * (float) (2 * ((sc[ib / 2] >> (6 * (ib % 2) + 3)) & 7) + 1)};
            for (int l = 0; l < 4; ++l) {
                const uint8_t h = qh[l / 2];
                const int idx = qs[l] | (((l & 1) ? (h << 4) : (h << 8)) & 0x700);
                const float delta = (h & ((l & 1) ? 0x80 : 0x08)) ? -0.125f : 0.125f;
                const uint16_t g = kIq1Grid[idx];
                for (int j = 0; j < 8; ++j) *y++ = dl[l / 2] * ((float) ((int) ((g >> (2 * j)) & 3) - 1) + delta);
            }
        }
    }
}

/* ggml's dequantize_row_q8_0 (src/kernels/cpu/ggml/ggml_quants.c): value = code x d. */
static void dequant_q8_0(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 32; ++i, b += 34) {
        uint16_t dh;
        memcpy(&dh, b, 2);
        const float d = h2f(dh);
        for (int j = 0; j < 32; ++j) *y++ = (float) (int8_t) b[2 + j] * d;
    }
}

/* ggml's get_scale_min_k4: the 6-bit scale and minimum j of the 12 packed bytes of a Q4_K / Q5_K block. */
static void k4_scale_min(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t) ((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t) ((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ggml's dequantize_row_q4_K / dequantize_row_q5_K (src/kernels/cpu/ggml/ggml_quants.c): per 64 values two (scale, min) pairs;
 * value = d sc q - dmin m, the product and the difference rounded separately; Q5_K adds 16 where the value's bit of qh is
 * set (bit 2p for the low nibbles of pair p, bit 2p + 1 for the high ones). */
static void dequant_q45k(const uint8_t* b, float* y, int64_t n, int five) {
    const int bs = five ? 176 : 144;
    for (int64_t i = 0; i < n / 256; ++i, b += bs) {
        uint16_t dh, mh;
        memcpy(&dh, b, 2);
        memcpy(&mh, b + 2, 2);
        const float d = h2f(dh), dmin = h2f(mh);
        const uint8_t *scales = b + 4, *qh = b + 16, *q = b + (five ? 48 : 16);
        for (int p = 0; p < 4; ++p, q += 32) {
            uint8_t sc, m;
            k4_scale_min(2 * p, scales, &sc, &m);
            const float d1 = d * sc, m1 = dmin * m;
            k4_scale_min(2 * p + 1, scales, &sc, &m);
            const float d2 = d * sc, m2 = dmin * m;
            for (int l = 0; l < 32; ++l) {
                const int hi = five && ((qh[l] >> (2 * p)) & 1) ? 16 : 0;
                volatile float t = d1 * (float) ((q[l] & 0xF) + hi);
                *y++ = t - m1;
            }
            for (int l = 0; l < 32; ++l) {
                const int hi = five && ((qh[l] >> (2 * p + 1)) & 1) ? 16 : 0;
                volatile float t = d2 * (float) ((q[l] >> 4) + hi);
                *y++ = t - m2;
            }
        }
    }
}

/* src/kernels/cpu/ggml/ggml_quants.c:229-281: Q5_0 value = (nibble | fifth bit from qh) - 16, times d; Q5_1 = code x d + m. */
static void dequant_q5_01(const uint8_t* b, float* y, int64_t n, int one) {
    const int bs = one ? 24 : 22;
    for (int64_t i = 0; i < n / 32; ++i, b += bs, y += 32) {
        uint16_t dh, mh = 0;
        uint32_t qh;
        memcpy(&dh, b, 2);
        if (one) memcpy(&mh, b + 2, 2);
        memcpy(&qh, b + (one ? 4 : 2), 4);
        const float d = h2f(dh), m = one ? h2f(mh) : 0.f;
        const uint8_t* qs = b + (one ? 8 : 6);
        for (int j = 0; j < 16; ++j) {
            const int x0 = (qs[j] & 0x0F) | (int) (((qh >> j) << 4) & 0x10), x1 = (qs[j] >> 4) | (int) ((qh >> (j + 12)) & 0x10);
            if (one) {
                volatile float p0 = (float) x0 * d, p1 = (float) x1 * d;
                y[j] = p0 + m;
                y[j + 16] = p1 + m;
            } else {
                y[j] = (float) (x0 - 16) * d;
                y[j + 16] = (float) (x1 - 16) * d;
            }
        }
    }
}

/* include/basalt/ggml/ggml_common.h:1023-1025 */
static const int8_t kIq4Levels[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* ggml_quants.c:1316-1356: IQ4_NL value = d x level[nibble]; IQ4_XS the same with a 6-bit scale (minus 32) per 32 values. */
static void dequant_iq4(const uint8_t* b, float* y, int64_t n, int xs) {
    if (!xs) {
        for (int64_t i = 0; i < n / 32; ++i, b += 18, y += 32) {
            uint16_t dh;
            memcpy(&dh, b, 2);
            const float d = h2f(dh);
            for (int j = 0; j < 16; ++j) {
                y[j] = d * kIq4Levels[b[2 + j] & 15];
                y[j + 16] = d * kIq4Levels[b[2 + j] >> 4];
            }
        }
        return;
    }
    for (int64_t i = 0; i < n / 256; ++i, b += 136) {
        uint16_t dh, sh;
        memcpy(&dh, b, 2);
        memcpy(&sh, b + 2, 2);
        const float d = h2f(dh);
        const uint8_t* qs = b + 8;
        for (int ib = 0; ib < 8; ++ib, qs += 16, y += 32) {
            const int ls = ((b[4 + ib / 2] >> (4 * (ib % 2))) & 0xF) | (((sh >> (2 * ib)) & 3) << 4);
            const float dl = d * (float) (ls - 32);
            for (int j = 0; j < 16; ++j) {
                y[j] = dl * kIq4Levels[qs[j] & 15];
                y[j + 16] = dl * kIq4Levels[qs[j] >> 4];
            }
        }
    }
}

/* ---- the low-bit formats.  Each follows the reference's dequantize_row_* of src/kernels/cpu/ggml/ggml_quants.c, walking a
 * block in the order the values are stored. */

static float h16_at(const uint8_t* p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return h2f(h);
}

/* ggml_quants.c:209-227 - Q2_0: four 2-bit codes a byte, value = (code - 1) d */
static void dequant_q2_0(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 64; ++i, b += 18) {
        const float d = h16_at(b);
        for (int j = 0; j < 16; ++j)
            for (int l = 0; l < 4; ++l) *y++ = (float) ((int) ((b[2 + j] >> (2 * l)) & 3) - 1) * d;
    }
}

/* ggml_quants.c:593-625 - Q2_K: per 16 values a byte (scale | min << 4); value = d scale code - dmin min, product and
 * difference rounded separately.  128 values share 32 code bytes, bit pair p of a byte belonging to values 32 p + l. */
static void dequant_q2k(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 84) {
        const float d = h16_at(b + 80), dmin = h16_at(b + 82);
        const uint8_t* sc = b;
        for (int half = 0; half < 2; ++half) {
            const uint8_t* q = b + 16 + 32 * half;
            for (int p = 0; p < 4; ++p)
                for (int h = 0; h < 2; ++h, ++sc) {
                    const float dl = d * (float) (*sc & 0xF), ml = dmin * (float) (*sc >> 4);
                    for (int l = 0; l < 16; ++l) {
                        volatile float t = dl * (float) ((q[16 * h + l] >> (2 * p)) & 3);
                        *y++ = t - ml;
                    }
                }
        }
    }
}

/* ggml_quants.c:712-760 - Q3_K: sixteen 6-bit scales in 12 bytes (low nibbles of bytes 0..7, high nibbles of bytes 0..7, then
 * the two top bits of scale j in byte 8 + j % 4 at bit 2 (j / 4)); value = d (scale - 32) (code - (hmask bit ? 0 : 4)). */
static void dequant_q3k(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 110) {
        const float d = h16_at(b + 108);
        const uint8_t *hm = b, *s12 = b + 96;
        int scales[16];
        for (int j = 0; j < 16; ++j) {
            const int lo = j < 8 ? (s12[j] & 0xF) : (s12[j - 8] >> 4);
            const int hi = (s12[8 + j % 4] >> (2 * (j / 4))) & 3;
            scales[j] = (lo | (hi << 4)) - 32;
        }
        int is = 0, bit = 0;
        for (int half = 0; half < 2; ++half) {
            const uint8_t* q = b + 32 + 32 * half;
            for (int p = 0; p < 4; ++p, ++bit)
                for (int h = 0; h < 2; ++h, ++is) {
                    const float dl = d * (float) scales[is];
                    for (int l = 0; l < 16; ++l) {
                        const int code = (int) ((q[16 * h + l] >> (2 * p)) & 3) - ((hm[16 * h + l] >> bit) & 1 ? 0 : 4);
                        *y++ = dl * (float) code;
                    }
                }
        }
    }
}

/* include/basalt/ggml/ggml_common.h (ksigns_iq2xs): seven stored sign bits, the eighth keeps the count of minus signs even */
static unsigned signs_from7(unsigned i) { return i | ((unsigned) (__builtin_popcount(i) & 1) << 7); }

static const float kIq2Mag[4] = {8.f, 25.f, 43.f, 43.f};
static void iq2_emit(uint16_t point, unsigned signs, float db, float** y) {
    for (int j = 0; j < 8; ++j) {
        const float v = db * kIq2Mag[(point >> (2 * j)) & 3];
        *(*y)++ = (signs >> j) & 1 ? -v : v;
    }
}
static float iq3_mag(int s_table, unsigned c) { return s_table ? (float) (2 * c + 1) : (c == 7 ? 62.f : (float) (4 + 8 * c)); }
static void iq3_emit(uint16_t point, unsigned signs4, float db, int s_table, float** y) {
    for (int j = 0; j < 4; ++j) {
        const float v = db * iq3_mag(s_table, (point >> (3 * j)) & 7);
        *(*y)++ = (signs4 >> j) & 1 ? -v : v;
    }
}

/* ggml_quants.c:1081-1107 - IQ2_XXS: per 32 values four point bytes and a word: 4 x 7 sign bits, scale in the top nibble;
 * db = d (0.5 + scale) / 4 */
static void dequant_iq2xxs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 66) {
        const float d = h16_at(b);
        for (int ib = 0; ib < 8; ++ib) {
            const uint8_t* q = b + 2 + 8 * ib;
            uint32_t w;
            memcpy(&w, q + 4, 4);
            const float db = d * (0.5f + (float) (w >> 28)) * 0.25f;
            for (int l = 0; l < 4; ++l) iq2_emit(kIqGrids[G_IQ2XXS + q[l]], signs_from7((w >> (7 * l)) & 127), db, &y);
        }
    }
}

/* ggml_quants.c:1109-1134 - IQ2_XS: a uint16 per 8 values (9-bit point, 7 sign bits), a 4-bit scale per 16 values */
static void dequant_iq2xs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 74) {
        const float d = h16_at(b);
        for (int ib = 0; ib < 8; ++ib) {
            const uint8_t sc = b[66 + ib];
            for (int l = 0; l < 4; ++l) {
                uint16_t q;
                memcpy(&q, b + 2 + 2 * (4 * ib + l), 2);
                const float db = d * (0.5f + (float) (l < 2 ? (sc & 0xF) : (sc >> 4))) * 0.25f;
                iq2_emit(kIqGrids[G_IQ2XS + (q & 511)], signs_from7(q >> 9), db, &y);
            }
        }
    }
}

/* ggml_quants.c:1136-1166 - IQ2_S: point = low byte | two bits of qh, the sign byte stored whole (after the 32 point bytes) */
static void dequant_iq2s(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 82) {
        const float d = h16_at(b);
        const uint8_t *qs = b + 2, *sg = b + 34, *qh = b + 66, *scl = b + 74;
        for (int ib = 0; ib < 8; ++ib) {
            for (int l = 0; l < 4; ++l) {
                const float db = d * (0.5f + (float) (l < 2 ? (scl[ib] & 0xF) : (scl[ib] >> 4))) * 0.25f;
                const unsigned idx = qs[4 * ib + l] | ((unsigned) ((qh[ib] >> (2 * l)) & 3) << 8);
                iq2_emit(kIqGrids[G_IQ2S + idx], sg[4 * ib + l], db, &y);
            }
        }
    }
}

/* ggml_quants.c:1168-1198 - IQ3_XXS: a point byte per 4 values; per 32 values a word of 4 x 7 sign bits and the scale;
 * db = d (0.5 + scale) / 2 */
static void dequant_iq3xxs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 98) {
        const float d = h16_at(b);
        for (int ib = 0; ib < 8; ++ib) {
            uint32_t w;
            memcpy(&w, b + 66 + 4 * ib, 4);
            const float db = d * (0.5f + (float) (w >> 28)) * 0.5f;
            for (int l = 0; l < 4; ++l) {
                const unsigned signs = signs_from7((w >> (7 * l)) & 127);
                iq3_emit(kIqGrids[G_IQ3XXS + b[2 + 8 * ib + 2 * l]], signs & 15, db, 0, &y);
                iq3_emit(kIqGrids[G_IQ3XXS + b[2 + 8 * ib + 2 * l + 1]], signs >> 4, db, 0, &y);
            }
        }
    }
}

/* ggml_quants.c:1200-1239 - IQ3_S: point = byte | ninth bit from qh (bit k of qh[ib] for the k-th point of the 32 values),
 * sign bytes stored whole, db = d (1 + 2 scale) with a 4-bit scale per 32 values */
static void dequant_iq3s(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 110) {
        const float d = h16_at(b);
        const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *scl = b + 106;
        for (int ib = 0; ib < 8; ++ib) {
            const int nib = (scl[ib / 2] >> (4 * (ib % 2))) & 0xF;
            const float db = d * (float) (1 + 2 * nib);
            for (int k = 0; k < 8; ++k) {
                const unsigned idx = qs[8 * ib + k] | ((unsigned) ((qh[ib] >> k) & 1) << 8);
                const unsigned s = sg[4 * ib + k / 2];
                iq3_emit(kIqGrids[G_IQ3S + idx], (k & 1) ? (s >> 4) : (s & 15), db, 1, &y);
            }
        }
    }
}

/* ggml_quants.c:1241-1264 - IQ1_S: per 32 values a uint16: 4 x 3 high point bits, a 3-bit scale, the sign of delta;
 * value = d (2 scale + 1) (g + delta), g in {-1, 0, 1}, delta = +-1/8 */
static void dequant_iq1s(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 256; ++i, b += 50) {
        const float d = h16_at(b);
        for (int ib = 0; ib < 8; ++ib) {
            uint16_t qh;
            memcpy(&qh, b + 34 + 2 * ib, 2);
            const float dl = d * (float) (2 * ((qh >> 12) & 7) + 1);
            const float delta = (qh & 0x8000) ? -0.125f : 0.125f;
            for (int l = 0; l < 4; ++l) {
                const uint16_t g = kIq1Grid[b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
                for (int j = 0; j < 8; ++j) *y++ = dl * ((float) ((int) ((g >> (2 * j)) & 3) - 1) + delta);
            }
        }
    }
}

EXPORT int orc_dequant_row(int type, const void* src, float* y, int64_t n) {
    if (orc_row_bytes(type, n) == 0) return -1;
    if (type == T_NVFP4) dequant_nvfp4(src, y, n);
    else if (type == T_Q6_K) dequant_q6k(src, y, n);
    else if (type == T_Q8_0) dequant_q8_0(src, y, n);
    else if (type == T_Q4_K) dequant_q45k(src, y, n, 0);
    else if (type == T_Q5_K) dequant_q45k(src, y, n, 1);
    else if (type == T_Q5_0) dequant_q5_01(src, y, n, 0);
    else if (type == T_Q5_1) dequant_q5_01(src, y, n, 1);
    else if (type == T_IQ4_NL) dequant_iq4(src, y, n, 0);
    else if (type == T_IQ4_XS) dequant_iq4(src, y, n, 1);
    else if (type == T_Q2_0) dequant_q2_0(src, y, n);
    else if (type == T_Q2_K) dequant_q2k(src, y, n);
    else if (type == T_Q3_K) dequant_q3k(src, y, n);
    else if (type == T_IQ2_XXS) dequant_iq2xxs(src, y, n);
    else if (type == T_IQ2_XS) dequant_iq2xs(src, y, n);
    else if (type == T_IQ2_S) dequant_iq2s(src, y, n);
    else if (type == T_IQ3_XXS) dequant_iq3xxs(src, y, n);
    else if (type == T_IQ3_S) dequant_iq3s(src, y, n);
    else if (type == T_IQ1_S) dequant_iq1s(src, y, n);
    else dequant_iq1m(src, y, n);
    return 0;
}

/* src/kernels/cpu/ggml/ggml_quants.c:1447-1476 - round-to-nearest NVFP4: per 16 values the UE4M3 code whose (undoubled)
 * value is nearest amax/6, first code wins a tie; then per value the nearest E2M1 code under that scale, first code wins. */
static void quant_nvfp4(const float* x, uint8_t* b, int64_t n) {
    for (int64_t i = 0; i < n / 64; ++i, x += 64, b += 36) {
        memset(b + 4, 0, 32);
        for (int s = 0; s < 4; ++s) {
            const float* xs = x + 16 * s;
            float amax = 0.0f;
            for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(xs[j]));
            const float want = amax / 6.0f;
            int best = 0;
            float be = INFINITY;
            for (int c = 0; c < 0x7F; ++c) {
                const float e = fabsf(2.0f * ue4m3_half((uint8_t) c) - want);
                if (e < be) { be = e; best = c; }
            }
            b[s] = (uint8_t) best;
            const float d = ue4m3_half((uint8_t) best);
            for (int j = 0; j < 16; ++j) {
                int q = 0;
                float qe = INFINITY;
                for (int c = 0; c < 16; ++c) {
                    const float e = fabsf((float) kFp4x2[c] * d - xs[j]);
                    if (e < qe) { qe = e; q = c; }
                }
                b[4 + 8 * s + (j & 7)] |= (uint8_t) (j < 8 ? q : q << 4);
            }
        }
    }
}

/* src/kernels/cpu/ggml/ggml_quants.c:305-310 */
static int nearest_int(float v) {
    const float t = v + 12582912.f;
    int i;
    memcpy(&i, &t, 4);
    return (i & 0x007fffff) - 0x00400000;
}
static int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

/* src/kernels/cpu/ggml/ggml_quants.c:312-381 with rmse_type 1 (weights x^2) and no importance matrix: the scale search the
 * Q6_K quantiser runs per 16 values.  L gets codes offset by nmax; returns the chosen scale. */
static float qx_scale_search(int n, int nmax, const float* x, int8_t* L) {
    float max = 0, amax = 0;
    for (int i = 0; i < n; ++i) {
        const float ax = fabsf(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < 1e-15f) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        return 0.f;
    }
    float iscale = -nmax / max, sumlx = 0, suml2 = 0;
    for (int i = 0; i < n; ++i) {
        const int l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        L[i] = (int8_t) (l + nmax);
        const float w = x[i] * x[i];
        sumlx += w * x[i] * l;
        suml2 += w * l * l;
    }
    float scale = suml2 ? sumlx / suml2 : 0.0f, best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        iscale = -(nmax + 0.1f * is) / max;
        sumlx = suml2 = 0;
        for (int i = 0; i < n; ++i) {
            const int l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
            const float w = x[i] * x[i];
            sumlx += w * x[i] * l;
            suml2 += w * l * l;
        }
        if (suml2 > 0 && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) L[i] = (int8_t) (nmax + clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1));
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

/* src/kernels/cpu/ggml/ggml_quants.c:978-1046 */
static void quant_q6k(const float* x, uint8_t* b, int64_t n) {
    int8_t L[256];
    float scales[16];
    for (int64_t i = 0; i < n / 256; ++i, x += 256, b += 210) {
        float max_scale = 0, max_abs = 0;
        for (int ib = 0; ib < 16; ++ib) {
            const float s = qx_scale_search(16, 32, x + 16 * ib, L + 16 * ib);
            scales[ib] = s;
            if (fabsf(s) > max_abs) { max_abs = fabsf(s); max_scale = s; }
        }
        memset(b, 0, 210);
        if (max_abs < 1e-15f) continue;
        const float iscale = -128.f / max_scale;
        const uint16_t dh = f2h(1 / iscale);
        memcpy(b + 208, &dh, 2);
        int8_t* sc = (int8_t*) (b + 192);
        for (int ib = 0; ib < 16; ++ib) {
            const int v = nearest_int(iscale * scales[ib]);
            sc[ib] = (int8_t) (v < 127 ? v : 127);
        }
        for (int j = 0; j < 16; ++j) {
            const float d = h2f(dh) * sc[j];
            if (!d) continue;
            for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t) (clampi(nearest_int(x[16 * j + ii] / d), -32, 31) + 32);
        }
        for (int half = 0; half < 2; ++half)
            for (int l = 0; l < 32; ++l) {
                const int8_t* q = L + 128 * half + l;
                b[64 * half + l] = (uint8_t) ((q[0] & 15) | ((q[64] & 15) << 4));
                b[64 * half + 32 + l] = (uint8_t) ((q[32] & 15) | ((q[96] & 15) << 4));
                b[128 + 32 * half + l] = (uint8_t) ((q[0] >> 4) | ((q[32] >> 4) << 2) | ((q[64] >> 4) << 4) | ((q[96] >> 4) << 6));
            }
    }
}

/* Quantises rows x cols floats; returns bytes written, 0 for a type without a quantiser (IQ1_M: the reference has none
 * either, include/basalt/ggml/ggml.h:74-77). */
EXPORT int64_t orc_quantize_rows(int type, const float* x, void* dst, int64_t rows, int64_t cols) {
    const int64_t rb = orc_row_bytes(type, cols);
    if (!rb || type == T_IQ1_M) return 0;
    for (int64_t r = 0; r < rows; ++r) {
        if (type == T_NVFP4) quant_nvfp4(x + r * cols, (uint8_t*) dst + r * rb, cols);
        else quant_q6k(x + r * cols, (uint8_t*) dst + r * rb, cols);
    }
    return rows * rb;
}

/* src/kernels/cuda/iq_kernels.cu:2471-2483 + include/basalt/kernels/q8_1_finite.hpp:17-31: fp32 row -> q8_1 blocks of 32
 * (fp16 d, fp16 sum, 32 int8).  The sum runs as the warp's xor-butterfly does. */
EXPORT void orc_quantize_q8_1(const float* x, int64_t n, uint8_t* y) {
    for (int64_t ib = 0; ib < n / 32; ++ib, x += 32, y += 36) {
        float amax = 0, s[32];
        for (int j = 0; j < 32; ++j) { amax = fmaxf(amax, fabsf(x[j])); s[j] = x[j]; }
        for (int o = 16; o > 0; o >>= 1) {
            float t[32];
            for (int j = 0; j < 32; ++j) t[j] = s[j] + s[j ^ o];
            memcpy(s, t, sizeof s);
        }
        float d = amax / 127.0f;
        if (fabsf(d) > 65504.0f) d = copysignf(65504.0f, d);
        float sum = s[0];
        if (fabsf(sum) > 65504.0f) sum = copysignf(65504.0f, sum);
        const uint16_t dh = f2h(d), sh = f2h(sum);
        memcpy(y, &dh, 2);
        memcpy(y + 2, &sh, 2);
        for (int j = 0; j < 32; ++j) {
            float q = amax == 0.0f ? 0.0f : roundf(x[j] / d);
            q = q > 127.0f ? 127.0f : q < -127.0f ? -127.0f : q;
            y[4 + j] = (uint8_t) (int8_t) q;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ router */
static float butterfly_sum32(float* v) {
    for (int o = 16; o; o >>= 1) {
        float t[32];
        for (int j = 0; j < 32; ++j) t[j] = v[j] + v[j ^ o];
        memcpy(v, t, 32 * sizeof(float));
    }
    return v[0];
}

/* src/kernels/cuda/router.cu:49-88 - logits[t][e] = gate[e] . x[t] in the kernel's summation order: 256 threads, thread i
 * owns float4 columns i, i+256, ... as one fmaf chain (x, y, z, w inside a float4), each warp sums by xor-butterfly, the 8
 * warp sums are added in warp order starting from 0. */
EXPORT void orc_router_logits(const float* x, const float* gate, int T, int E, int H, float* logits) {
    const int n4 = H / 4;
    for (int t = 0; t < T; ++t)
        for (int e = 0; e < E; ++e) {
            const float *g = gate + (size_t) e * H, *xv = x + (size_t) t * H;
            float acc[256];
            for (int th = 0; th < 256; ++th) {
                float a = 0.f;
                for (int i = th; i < n4; i += 256)
                    for (int c = 0; c < 4; ++c) a = fmaf(g[4 * i + c], xv[4 * i + c], a);
                acc[th] = a;
            }
            float s = 0.f;
            for (int w = 0; w < 8; ++w) s += butterfly_sum32(acc + 32 * w);
            logits[(size_t) t * E + e] = s;
        }
}

enum { GATE_SQRT_SOFTPLUS = 0, GATE_SIGMOID = 1, GATE_SOFTMAX = 2 };

/* src/kernels/cuda/router.cu:148-153 */
static float gate_score(float x, int kind) {
    if (kind == GATE_SQRT_SOFTPLUS) return sqrtf(x > 20.f ? x : logf(1.f + expf(x)));
    return 1.f / (1.f + expf(-x));
}

/* src/kernels/cuda/router.cu:170-217 (selection by rank: higher biased score first, the lower index on a tie; weights are the
 * unbiased scores of the chosen over their sum + 1e-20, times scale) with the group-limited step in front of it:
 * the experts form n_group contiguous groups, a group scores the sum of its two largest biased scores, the topk_group
 * best groups (lower group index on a tie) stay and the others cannot be chosen.  n_group <= 1 is the reference's plain
 * selection.  `held` ([E] slot or -1, may be null) and `prior` follow router.cu:180 (--route-prior). */
static void router_select_impl(const float* logits, const float* scores, const float* bias, int T, int E, int k, int kind, float scale,
                               int n_group, int topk_group, float prior, const int32_t* held, int32_t* ids, float* weights) {
    float* s = malloc(sizeof(float) * (size_t) E);
    float* b = malloc(sizeof(float) * (size_t) E);
    char* live = malloc((size_t) E);
    for (int t = 0; t < T; ++t) {
        for (int e = 0; e < E; ++e) {
            s[e] = scores ? scores[(size_t) t * E + e] : gate_score(logits[(size_t) t * E + e], kind);
            b[e] = s[e] + (bias ? bias[e] : 0.f);
            if (held && prior > 0.f && held[e] >= 0) b[e] += prior;
            live[e] = 1;
        }
        if (n_group > 1 && topk_group < n_group) {
            const int gs = E / n_group;
            float gsc[64];
            for (int g = 0; g < n_group; ++g) {
                float m1 = -INFINITY, m2 = -INFINITY;
                for (int j = 0; j < gs; ++j) {
                    const float v = b[g * gs + j];
                    if (v > m1) { m2 = m1; m1 = v; }
                    else if (v > m2) m2 = v;
                }
                gsc[g] = gs > 1 ? m1 + m2 : m1;
            }
            for (int g = 0; g < n_group; ++g) {
                int rank = 0;
                for (int j = 0; j < n_group; ++j) rank += (gsc[j] > gsc[g]) | ((gsc[j] == gsc[g]) & (j < g));
                if (rank >= topk_group)
                    for (int j = 0; j < gs; ++j) live[g * gs + j] = 0;
            }
        }
        float sel[64];
        for (int e = 0; e < E; ++e) {
            if (!live[e]) continue;
            int rank = 0;
            for (int j = 0; j < E; ++j) rank += live[j] && ((b[j] > b[e]) | ((b[j] == b[e]) & (j < e)));
            if (rank < k) { sel[rank] = s[e]; ids[(size_t) t * k + rank] = e; }
        }
        float sum = 0.f;
        for (int r = 0; r < k; ++r) sum += sel[r];
        const float denom = sum + 1e-20f;
        for (int r = 0; r < k; ++r) weights[(size_t) t * k + r] = sel[r] / denom * scale;
    }
    free(s);
    free(b);
    free(live);
}

EXPORT void orc_router_select(const float* logits, const float* bias, int T, int E, int k, int kind, float scale,
                              int n_group, int topk_group, float prior, const int32_t* held, int32_t* ids, float* weights) {
    router_select_impl(logits, NULL, bias, T, E, k, kind, scale, n_group, topk_group, prior, held, ids, weights);
}

/* The same selection from gate scores computed elsewhere (the device's own expf / logf results): everything after the score
 * is fp32 IEEE arithmetic, so with the device's scores the ids and the weight bits must equal the device's. */
EXPORT void orc_router_select_scores(const float* scores, const float* bias, int T, int E, int k, float scale,
                                     int n_group, int topk_group, float prior, const int32_t* held, int32_t* ids, float* weights) {
    router_select_impl(NULL, scores, bias, T, E, k, 1, scale, n_group, topk_group, prior, held, ids, weights);
}

/* src/models/qwen4exp/prefill/kernels.cu:351-390 generalised from (512 | 256 experts, top-10) to E % 32 == 0, k <= 32:
 * one warp per token, lane l holds experts l, l+32, ...; softmax over all experts (max-subtracted expf, per-lane sums in
 * index order then xor-butterfly, times the reciprocal of the sum), NaN -> -FLT_MAX; k argmax passes (value desc, index
 * asc); the chosen probabilities are summed per winning lane in selection order, then by butterfly, clamped below at
 * 2^-14; weight = p / that sum.  `fast` follows src/models/qwen4exp/kernels/native_router.cu:44-99 instead (weight = p times
 * the reciprocal); libm's expf stands in for both expf and __expf here, so ids can differ from the GPU on near-ties. */
EXPORT void orc_router_softmax(const float* logits, int T, int E, int k, int fast, int32_t* ids, float* weights) {
    const int reg = E / 32;
    float* v = malloc(sizeof(float) * (size_t) E);   /* v[i*32 + lane] */
    for (int t = 0; t < T; ++t) {
        const float* lg = logits + (size_t) t * E;
        float mx = -INFINITY;
        for (int e = 0; e < E; ++e) mx = fmaxf(mx, lg[e]);
        float lane_sum[32];
        for (int l = 0; l < 32; ++l) {
            float sum = 0.f;
            for (int i = 0; i < reg; ++i) {
                v[i * 32 + l] = expf(lg[l + 32 * i] - mx);
                sum += v[i * 32 + l];
            }
            lane_sum[l] = sum;
        }
        const float rcp = 1.0f / butterfly_sum32(lane_sum);
        for (int e = 0; e < E; ++e) {
            v[e] *= rcp;
            if (isnan(v[e])) v[e] = -FLT_MAX;
        }
        float picked[32], lane_sel[32];
        for (int l = 0; l < 32; ++l) lane_sel[l] = 0.f;
        for (int r = 0; r < k; ++r) {
            int ex = 0;
            float best = v[0];
            for (int e = 1; e < E; ++e)     /* v is indexed by expert id here: v[i*32+lane] == expert lane + 32 i */
                if (v[e] > best) { best = v[e]; ex = e; }
            v[ex] = -INFINITY;
            lane_sel[ex & 31] += best;
            ids[(size_t) t * k + r] = ex;
            picked[r] = best;
        }
        const float tot = fmaxf(butterfly_sum32(lane_sel), 6.103515625e-5f);
        for (int r = 0; r < k; ++r) weights[(size_t) t * k + r] = fast ? picked[r] * (1.0f / tot) : picked[r] / tot;
    }
    free(v);
}

/* src/models/qwen4exp/kernels/router_top10.cu:57-174 - the fp64 softmax router: p[e] = (float)(exp((double)l - (double)mx) *
 * (float)(1/sum)), sum serial ascending in double; k passes of (value desc, index asc); weights renormalised in double
 * over max(sum, 2^-14). */
EXPORT void orc_router_top10(const float* logits, int T, int E, int k, int32_t* ids, float* weights) {
    double* ex = malloc(sizeof(double) * (size_t) E);
    float* p = malloc(sizeof(float) * (size_t) E);
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t) t * E;
        float mx = -INFINITY;
        for (int e = 0; e < E; ++e) mx = fmaxf(mx, l[e]);
        double sum = 0.0;
        for (int e = 0; e < E; ++e) { ex[e] = exp((double) l[e] - (double) mx); sum += ex[e]; }
        const float inv = (float) (1.0 / sum);
        for (int e = 0; e < E; ++e) p[e] = (float) (ex[e] * inv);
        float w[64];
        for (int i = 0; i < k; ++i) {
            float bv = -INFINITY;
            int bi = E;
            for (int e = 0; e < E; ++e)
                if (p[e] > bv) { bv = p[e]; bi = e; }
            if (bi < E) { ids[(size_t) t * k + i] = bi; w[i] = bv; p[bi] = -INFINITY; }
            else w[i] = 0.f;
        }
        double s = 0.0;
        for (int i = 0; i < k; ++i) s += (double) w[i];
        const double sc = fmax(s, 6.103515625e-05);
        for (int i = 0; i < k; ++i) weights[(size_t) t * k + i] = (float) ((double) w[i] / sc);
    }
    free(ex);
    free(p);
}

/* include/basalt/kernels/route_lossy.hpp:34-60 + src/kernels/cuda/route_tail_skip.cu:14-53 - the opt-in tail skip on a window
 * of n <= 128 entries: an entry whose expert is held by no table and whose every namesake in the window ranks `rank` or
 * lower by weight inside its token becomes id -1, weight 0.  counts[0..2] += entries, misses, drops. */
EXPORT void orc_route_tail_skip(int32_t* ids, float* w, const int32_t* held, int n, int k, int rank, int E, uint64_t* counts) {
    if (rank < 1 || rank >= k || n < 1 || n > 128 || k < 1) return;
    int32_t id0[128];
    uint8_t tail[128], miss[128];
    int n_miss = 0, n_drop = 0;
    for (int i = 0; i < n; ++i) {
        id0[i] = ids[i];
        const int base = i - i % k;
        int r = 0;
        for (int j = 0; j < k; ++j) r += w[base + j] > w[i] || (w[base + j] == w[i] && base + j < i);
        tail[i] = r >= rank;
        miss[i] = ids[i] >= 0 && ids[i] < E && !(held && held[ids[i]] >= 0);
        n_miss += miss[i];
    }
    for (int i = 0; i < n; ++i) {
        int drop = miss[i];
        for (int j = 0; drop && j < n; ++j)
            if (id0[j] == id0[i] && !tail[j]) drop = 0;
        if (drop) { ids[i] = -1; w[i] = 0.0f; ++n_drop; }
    }
    if (counts) { counts[0] += (uint64_t) n; counts[1] += (uint64_t) n_miss; counts[2] += (uint64_t) n_drop; }
}

/* ------------------------------------------------------------------------------------------------ dispatch */
/* src/models/qwen4exp/prefill/routing.cpp:67-108 (host counting sort; the one ordering every reference variant can
 * reproduce): cnt[e] = pairs naming e, off = exclusive prefix sum in expert-id order, slot[i] = row of pair i (pairs keep
 * their order inside an expert), src[row] = token i / k.  Ids outside [0, E) (the tail skip's -1) get slot -1 and no row.
 * tiles (optional, [2 * max_tiles]): {expert, first row} of each tile of `tile_rows` rows, experts ascending
 * (src/models/qwen4exp/prefill/moe_fused.cu:140-156); returns the tile count. */
EXPORT int orc_dispatch(const int32_t* ids, int64_t n, int k, int E, int32_t* cnt, int32_t* off, int32_t* slot, int32_t* src,
                        int tile_rows, int32_t* tiles) {
    for (int e = 0; e < E; ++e) cnt[e] = 0;
    for (int64_t i = 0; i < n; ++i)
        if (ids[i] >= 0 && ids[i] < E) ++cnt[ids[i]];
    off[0] = 0;
    for (int e = 0; e < E; ++e) off[e + 1] = off[e] + cnt[e];
    int32_t* fill = malloc(sizeof(int32_t) * (size_t) E);
    memcpy(fill, off, sizeof(int32_t) * (size_t) E);
    for (int64_t i = 0; i < n; ++i) {
        const int32_t e = ids[i];
        if (e < 0 || e >= E) { slot[i] = -1; continue; }
        const int32_t p = fill[e]++;
        slot[i] = p;
        src[p] = (int32_t) (i / k);
    }
    free(fill);
    int nt = 0;
    if (tile_rows > 0)
        for (int e = 0; e < E; ++e)
            for (int r = 0; r < cnt[e]; r += tile_rows) {
                if (tiles) { tiles[2 * nt] = e; tiles[2 * nt + 1] = off[e] + r; }
                ++nt;
            }
    return nt;
}

/* src/models/inkling2/kernels/ops.cu:275-340 - the decode-window plan: the experts that have pairs and a blob, ascending, as
 * groups (ptr[g] = blob address, start[g] = first entry; start[n_groups] = start[n_groups + 1] = total); entries inside a
 * group in pair order; dst[entry] = pair index (the output row), tok[entry] = pair / k. */
EXPORT void orc_moe_plan(const int32_t* ids, int n, int k, int E, const uint64_t* blobs, uint64_t* ptr, int32_t* start,
                         int32_t* n_groups, int32_t* dst, int32_t* tok) {
    int g = 0, at = 0;
    for (int e = 0; e < E; ++e) {
        if (!blobs[e]) continue;
        int c = 0;
        for (int i = 0; i < n; ++i)
            if (ids[i] == e) {
                if (c == 0) { ptr[g] = blobs[e]; start[g] = at; }
                dst[at + c] = i;
                tok[at + c] = i / k;
                ++c;
            }
        if (c) { at += c; ++g; }
    }
    start[g] = at;
    start[g + 1] = at;
    *n_groups = g;
}

/* ------------------------------------------------------------------------------------------------ combine */
/* src/models/qwen4exp/kernels/native_moe.cu:36-50 and src/models/qwen4exp/prefill/kernels.cu:438-449 (the two agree bit for
 * bit: nvcc contracts `sum += a * b` to one fma, and fma(w0, p0, 0) is the rounded first product):
 * y[t] = fma chain over the k rows rows[slot[t*k+j]] * w[t*k+j] in j order, then + shared[t] (times the per-token sigmoid
 * gate 1/(1+exp(-sg[t])) as one more fma when sg is given).  slot may be null (row = pair index); slot < 0 = no row. */
EXPORT void orc_combine(const float* rows, const int32_t* slot, const float* w, const float* shared, const float* sg, int T,
                        int k, int H, float* y) {
    for (int t = 0; t < T; ++t) {
        const float gate = sg ? 1.0f / (1.0f + expf(-sg[t])) : 1.0f;
        for (int c = 0; c < H; ++c) {
            float s = 0.0f;
            for (int j = 0; j < k; ++j) {
                const int64_t r = slot ? slot[(size_t) t * k + j] : (int64_t) t * k + j;
                if (r < 0) continue;
                s = fmaf(w[(size_t) t * k + j], rows[(size_t) r * H + c], s);
            }
            if (shared) s = sg ? fmaf(shared[(size_t) t * H + c], gate, s) : s + shared[(size_t) t * H + c];
            y[(size_t) t * H + c] = s;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ one expert, fp32 */
/* tests/kernels/native_expert_parity.cpp:58-84 with fp32 accumulation (`dbl` = 0) or double (`dbl` = 1): one expert on nt
 * tokens from already-decoded matrices G, U [I][H] and D [H][I]; tail = {s_gate, s_up, s_down} (1 for formats without).
 * h = silu(s_gate g) * (s_up u) with optional clamp (gate capped above at L, up clamped to +-L:
 * src/kernels/cuda/iq_kernels.cu:3263-3279); out = s_down * D h. */
EXPORT void orc_expert_dense(const float* G, const float* U, const float* D, const float* tail, const float* x, int nt, int H,
                             int I, float limit, int dbl, float* out) {
    float* h = malloc(sizeof(float) * (size_t) I);
    for (int t = 0; t < nt; ++t) {
        const float* xv = x + (size_t) t * H;
        for (int r = 0; r < I; ++r) {
            float g, u;
            if (dbl) {
                double ag = 0, au = 0;
                for (int i = 0; i < H; ++i) { ag += (double) G[(size_t) r * H + i] * xv[i]; au += (double) U[(size_t) r * H + i] * xv[i]; }
                g = (float) (ag * tail[0]);
                u = (float) (au * tail[1]);
            } else {
                float ag = 0, au = 0;
                for (int i = 0; i < H; ++i) { ag = fmaf(G[(size_t) r * H + i], xv[i], ag); au = fmaf(U[(size_t) r * H + i], xv[i], au); }
                g = ag * tail[0];
                u = au * tail[1];
            }
            if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
            h[r] = dbl ? (float) ((double) g / (1.0 + exp(-(double) g)) * (double) u) : g / (1.0f + expf(-g)) * u;
        }
        for (int r = 0; r < H; ++r) {
            if (dbl) {
                double a = 0;
                for (int i = 0; i < I; ++i) a += (double) D[(size_t) r * I + i] * h[i];
                out[(size_t) t * H + r] = (float) (a * tail[2]);
            } else {
                float a = 0;
                for (int i = 0; i < I; ++i) a = fmaf(D[(size_t) r * I + i], h[i], a);
                out[(size_t) t * H + r] = a * tail[2];
            }
        }
    }
    free(h);
}

/* FNV-1a over a byte range continuing from *h (src/models/deepseek41/kernels/router_parity.cpp:181-186) */
EXPORT uint64_t orc_fnv1a(uint64_t h, const void* p, size_t n) {
    const uint8_t* b = p;
    for (size_t i = 0; i < n; ++i) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}
