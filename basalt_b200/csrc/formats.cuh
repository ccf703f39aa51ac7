// formats.cuh - exact decoders of the ggml block formats the expert kernels read (NVFP4, Q6_K, IQ1_M).
//
// The meaning of every weight byte is the reference's (paths inside the Basalt project): block layouts
// include/basalt/ggml/ggml_common.h:146-156 (NVFP4), :279-285 (Q6_K), :350-362 (IQ1_M); decoding rules
// src/kernels/cpu/ggml/ggml_quants.c:1397-1422 (NVFP4, UE4M3 scale), :1048-1075 (Q6_K), :1266-1314 (IQ1_M).
// All functions are __host__ __device__ so the same code is checked on the CPU against the reference's to_float.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bsx {

enum : int { kTypeQ5_0 = 6, kTypeQ5_1 = 7, kTypeQ8_0 = 8, kTypeQ2K = 10, kTypeQ3K = 11, kTypeQ4K = 12, kTypeQ5K = 13, kTypeQ6K = 14,
              kTypeIQ2XXS = 16, kTypeIQ2XS = 17, kTypeIQ3XXS = 18, kTypeIQ1S = 19, kTypeIQ4NL = 20, kTypeIQ3S = 21, kTypeIQ2S = 22, kTypeIQ4XS = 23,
              kTypeIQ1M = 29, kTypeNVFP4 = 40, kTypeQ2_0 = 42 };

// One table of uint16 words holds every codebook: the IQ1 points (2048, 8 coordinates x 2 bits as g + 1), then the IQ2 points
// (iq2xxs 256, iq2xs 512, iq2s 1024; 8 x 2 bits, magnitude index into {8, 25, 43}), then the IQ3 points (iq3xxs 256: 4 x 3 bits,
// magnitude 4 + 8 c, except c = 7 -> 62; iq3s 512: 4 x 3 bits, magnitude 2 c + 1).
constexpr int kGridIQ1 = 0, kGridIQ2XXS = 2048, kGridIQ2XS = 2304, kGridIQ2S = 2816, kGridIQ3XXS = 3840, kGridIQ3S = 4096, kGridWords = 4608;
// the words of the table a format reads: [lo, lo + n)
__host__ __device__ inline void grid_range(int t, int& lo, int& n) {
    lo = 0;
    n = 0;
    if (t == 29 || t == 19) n = 2048;
    else if (t == 16) { lo = kGridIQ2XXS; n = 256; }
    else if (t == 17) { lo = kGridIQ2XS; n = 512; }
    else if (t == 22) { lo = kGridIQ2S; n = 1024; }
    else if (t == 18) { lo = kGridIQ3XXS; n = 256; }
    else if (t == 21) { lo = kGridIQ3S; n = 512; }
}
__host__ __device__ constexpr bool type_needs_grid(int t) {
    return t == kTypeIQ1M || t == kTypeIQ1S || t == kTypeIQ2XXS || t == kTypeIQ2XS || t == kTypeIQ2S || t == kTypeIQ3XXS || t == kTypeIQ3S;
}

// values per block and bytes per block (the GGUF formats' constants, include/basalt/ggml/ggml_common.h)
__host__ __device__ constexpr int block_values(int type) {
    return (type == kTypeNVFP4 || type == kTypeQ2_0) ? 64 : (type == kTypeQ8_0 || type == kTypeQ5_0 || type == kTypeQ5_1 || type == kTypeIQ4NL) ? 32 : 256;
}
__host__ __device__ constexpr int block_bytes(int type) {
    return type == kTypeNVFP4 ? 36 : type == kTypeQ6K ? 210 : type == kTypeIQ1M ? 56 : type == kTypeQ8_0 ? 34 : type == kTypeQ4K ? 144
           : type == kTypeQ5K ? 176 : type == kTypeQ5_0 ? 22 : type == kTypeQ5_1 ? 24 : type == kTypeIQ4NL ? 18 : type == kTypeIQ4XS ? 136
           : type == kTypeQ2K ? 84 : type == kTypeQ3K ? 110 : type == kTypeIQ2XXS ? 66 : type == kTypeIQ2XS ? 74 : type == kTypeIQ2S ? 82
           : type == kTypeIQ3XXS ? 98 : type == kTypeIQ3S ? 110 : type == kTypeIQ1S ? 50 : type == kTypeQ2_0 ? 18 : 0;
}

__host__ __device__ inline bool type_supported(int type) { return block_bytes(type) != 0; }

// UE4M3 scale byte as ggml reads it, already halved (the E2M1 table below is doubled): bit 7 ignored, 0 and 0x7F -> 0.
// (b & 0x7F) << 20 places the 4 exponent bits and 3 mantissa bits where fp32 keeps them; 2^(127-7-1) re-biases, and the
// same product is exact for UE4M3 subnormals because an fp32 subnormal times a power of two is exact.
__host__ __device__ __forceinline__ float ue4m3_half(uint32_t b) {
    b &= 0x7Fu;
    if (b == 0x7Fu) return 0.0f;
    const uint32_t u = b << 20;
#ifdef __CUDA_ARCH__
    return __uint_as_float(u) * 6.646139978924579e35f;   // 2^119
#else
    float f;
    memcpy(&f, &u, 4);
    return f * 6.646139978924579e35f;
#endif
}

// E2M1 code -> doubled value {0,1,2,3,4,6,8,12} with sign (ggml's kvalues_fp4)
__host__ __device__ __forceinline__ float e2m1_x2(uint32_t c) {
    const uint32_t m = c & 7u;
    const float v = m < 4u ? (float) m : m == 4u ? 4.0f : m == 5u ? 6.0f : m == 6u ? 8.0f : 12.0f;
    return ((c & 8u) && m) ? -v : v;   // code 8 is +0, as in ggml's integer table
}

__host__ __device__ __forceinline__ float half_bits_to_float(uint16_t h) {
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half(h));
#else
    const uint32_t s = (uint32_t) (h & 0x8000) << 16;
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF, u;
    if (e == 0) {
        if (m == 0) u = s;
        else {
            int sh = 0;
            while (!(m & 0x400)) { m <<= 1; ++sh; }
            u = s | ((uint32_t) (113 - sh) << 23) | ((m & 0x3FF) << 13);
        }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}

// ---- whole-block decoders (the simple kernels and the host check use these; the fast kernels decode in fragment order)

// one NVFP4 block (36 bytes, 4-byte aligned) -> 64 floats
__host__ __device__ inline void decode_block_nvfp4(const uint8_t* b, float* y) {
    for (int s = 0; s < 4; ++s) {
        const float d = ue4m3_half(b[s]);
        const uint8_t* q = b + 4 + 8 * s;
        for (int j = 0; j < 8; ++j) {
            y[16 * s + j] = e2m1_x2(q[j] & 15u) * d;
            y[16 * s + j + 8] = e2m1_x2(q[j] >> 4) * d;
        }
    }
}

// 32 consecutive values [32u, 32u+32) of a Q6_K block (210 bytes, 2-byte aligned)
__host__ __device__ inline void decode_q6k_32(const uint8_t* b, int u, float* y) {
    const int half = u >> 2, sub = u & 3;              // 128-value half, 32-value quarter inside it
    const uint8_t* ql = b + 64 * half + 32 * (sub & 1);
    const uint8_t* qh = b + 128 + 32 * half;
    const int8_t* sc = (const int8_t*) (b + 192) + 8 * half + 2 * sub;
    const float d = half_bits_to_float((uint16_t) (b[208] | (b[209] << 8)));
    for (int l = 0; l < 32; ++l) {
        const int lo = sub < 2 ? (ql[l] & 15) : (ql[l] >> 4);
        const int hi = (qh[l] >> (2 * sub)) & 3;
        const int q = (lo | (hi << 4)) - 32;
        y[l] = d * (float) sc[l >> 4] * (float) q;
    }
}

// a product and a difference rounded separately, as the reference's dequantisers compute them (no fused multiply-add)
__host__ __device__ inline float mul_then_sub(float a, float b, float c) {
#ifdef __CUDA_ARCH__
    return __fsub_rn(__fmul_rn(a, b), c);
#else
    volatile float p = a * b;
    return p - c;
#endif
}

__host__ __device__ inline float mul_then_add(float a, float b, float c) {
#ifdef __CUDA_ARCH__
    return __fadd_rn(__fmul_rn(a, b), c);
#else
    volatile float p = a * b;
    return p + c;
#endif
}

// one Q5_0 block (22 bytes: fp16 d, qh[4], qs[16]; value j = nibble j | bit j of qh as the fifth bit, minus 16; values j and
// j + 16 share byte j; dequantize_row_q5_0, src/kernels/cpu/ggml/ggml_quants.c:229-253) and one Q5_1 block (24 bytes: d, m, qh,
// qs; value = code x d + m; :255-281) -> 32 floats
__host__ __device__ inline void decode_q5_01_32(const uint8_t* b, bool one, float* y) {
    const float d = half_bits_to_float((uint16_t) (b[0] | (b[1] << 8)));
    const float m = one ? half_bits_to_float((uint16_t) (b[2] | (b[3] << 8))) : 0.f;
    const uint8_t* h = b + (one ? 4 : 2);
    const uint32_t qh = (uint32_t) h[0] | ((uint32_t) h[1] << 8) | ((uint32_t) h[2] << 16) | ((uint32_t) h[3] << 24);
    const uint8_t* qs = h + 4;
    for (int j = 0; j < 16; ++j) {
        const int x0 = (qs[j] & 0x0F) | (int) (((qh >> j) << 4) & 0x10), x1 = (qs[j] >> 4) | (int) ((qh >> (j + 12)) & 0x10);
        if (one) {
            y[j] = mul_then_add((float) x0, d, m);
            y[j + 16] = mul_then_add((float) x1, d, m);
        } else {
            y[j] = (float) (x0 - 16) * d;
            y[j + 16] = (float) (x1 - 16) * d;
        }
    }
}

// the 16 levels of the non-linear 4-bit formats (kvalues_iq4nl, include/basalt/ggml/ggml_common.h:1023-1025)
__host__ __device__ inline float iq4_level(int c) {
    return (float) (int) (int8_t) ((c < 8 ? 0xF6EADDCFBFAD9881ull : 0x7159453526190D01ull) >> (8 * (c & 7)));
}

// one IQ4_NL block (18 bytes: fp16 d, qs[16]; dequantize_row_iq4_nl, ggml_quants.c:1316-1332) -> 32 floats
__host__ __device__ inline void decode_iq4nl_32(const uint8_t* b, float* y) {
    const float d = half_bits_to_float((uint16_t) (b[0] | (b[1] << 8)));
    for (int j = 0; j < 16; ++j) {
        y[j] = d * iq4_level(b[2 + j] & 15);
        y[j + 16] = d * iq4_level(b[2 + j] >> 4);
    }
}

// 32 consecutive values [32u, 32u+32) of an IQ4_XS block (136 bytes: fp16 d, u16 scales_h, scales_l[4], qs[128]; a 6-bit
// scale per 32 values, minus 32; dequantize_row_iq4_xs, ggml_quants.c:1334-1356)
__host__ __device__ inline void decode_iq4xs_32(const uint8_t* b, int u, float* y) {
    const float d = half_bits_to_float((uint16_t) (b[0] | (b[1] << 8)));
    const uint32_t sh = (uint32_t) b[2] | ((uint32_t) b[3] << 8);
    const int ls = (int) ((b[4 + (u >> 1)] >> (4 * (u & 1))) & 0xF) | (int) (((sh >> (2 * u)) & 3) << 4);
    const float dl = d * (float) (ls - 32);
    const uint8_t* qs = b + 8 + 16 * u;
    for (int j = 0; j < 16; ++j) {
        y[j] = dl * iq4_level(qs[j] & 15);
        y[j + 16] = dl * iq4_level(qs[j] >> 4);
    }
}

// one Q8_0 block (34 bytes: fp16 d, 32 int8; src/kernels/cpu/ggml/ggml_quants.c dequantize_row_q8_0) -> 32 floats
__host__ __device__ inline void decode_q8_0_32(const uint8_t* b, float* y) {
    const float d = half_bits_to_float((uint16_t) (b[0] | (b[1] << 8)));
    for (int l = 0; l < 32; ++l) y[l] = (float) (int8_t) b[2 + l] * d;
}

// the 6-bit scale and minimum j (0..7) of a Q4_K / Q5_K block's 12 packed bytes (ggml's get_scale_min_k4)
__host__ __device__ inline void k4_scale_min(const uint8_t* q, int j, int& sc, int& m) {
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// 32 consecutive values [32u, 32u+32) of a Q4_K block (144 bytes: fp16 d, fp16 dmin, scales[12], qs[128]; 64 values share
// 32 bytes, the low nibbles first; dequantize_row_q4_K)
__host__ __device__ inline void decode_q4k_32(const uint8_t* b, int u, float* y) {
    const float d = half_bits_to_float((uint16_t) (b[0] | (b[1] << 8))), dmin = half_bits_to_float((uint16_t) (b[2] | (b[3] << 8)));
    int sc, m;
    k4_scale_min(b + 4, u, sc, m);
    const float d1 = d * (float) sc, m1 = dmin * (float) m;
    const uint8_t* q = b + 16 + 32 * (u >> 1);
    for (int l = 0; l < 32; ++l) y[l] = mul_then_sub(d1, (float) ((u & 1) ? (q[l] >> 4) : (q[l] & 15)), m1);
}

// 32 consecutive values of a Q5_K block (176 bytes: d, dmin, scales[12], qh[32], qs[128]; bit u of qh[l] is value l's fifth
// bit in the 32-value run u; dequantize_row_q5_K)
__host__ __device__ inline void decode_q5k_32(const uint8_t* b, int u, float* y) {
    const float d = half_bits_to_float((uint16_t) (b[0] | (b[1] << 8))), dmin = half_bits_to_float((uint16_t) (b[2] | (b[3] << 8)));
    int sc, m;
    k4_scale_min(b + 4, u, sc, m);
    const float d1 = d * (float) sc, m1 = dmin * (float) m;
    const uint8_t* qh = b + 16;
    const uint8_t* q = b + 48 + 32 * (u >> 1);
    for (int l = 0; l < 32; ++l) {
        const int lo = (u & 1) ? (q[l] >> 4) : (q[l] & 15);
        y[l] = mul_then_sub(d1, (float) (lo + (((qh[l] >> u) & 1) ? 16 : 0)), m1);
    }
}

// 32 consecutive values [32u, 32u+32) of an IQ1_M block (56 bytes, 2-byte aligned... only byte loads are used)
__host__ __device__ inline void decode_iq1m_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const uint8_t* qs = b + 4 * u;
    const uint8_t* qh = b + 32 + 2 * u;
    const uint16_t sc0 = (uint16_t) (b[48] | (b[49] << 8)), sc1 = (uint16_t) (b[50] | (b[51] << 8)),
                   sc2 = (uint16_t) (b[52] | (b[53] << 8)), sc3 = (uint16_t) (b[54] | (b[55] << 8));
    const uint16_t dh = (uint16_t) ((sc0 >> 12) | ((sc1 >> 8) & 0x00F0) | ((sc2 >> 4) & 0x0F00) | (sc3 & 0xF000));
    const float d = half_bits_to_float(dh);
    const uint16_t scw = (u >> 1) == 0 ? sc0 : (u >> 1) == 1 ? sc1 : (u >> 1) == 2 ? sc2 : sc3;
    const float dl[2] = {d * (float) (2 * ((scw >> (6 * (u & 1))) & 7) + 1), d * (float) (2 * ((scw >> (6 * (u & 1) + 3)) & 7) + 1)};
    for (int l = 0; l < 4; ++l) {
        const uint32_t h = qh[l >> 1];
        const uint32_t idx = qs[l] | (((l & 1) ? (h << 4) : (h << 8)) & 0x700u);
        const float delta = (h & ((l & 1) ? 0x80u : 0x08u)) ? -0.125f : 0.125f;
        const uint32_t g = grid[idx];
        for (int j = 0; j < 8; ++j) y[8 * l + j] = dl[l >> 1] * ((float) ((int) ((g >> (2 * j)) & 3u) - 1) + delta);
    }
}

// ---- the remaining ggml formats (block layouts include/basalt/ggml/ggml_common.h:140-145,215-238,298-347; decoding rules
// src/kernels/cpu/ggml/ggml_quants.c:209-227 Q2_0, :593-625 Q2_K, :712-760 Q3_K, :1081-1107 IQ2_XXS, :1109-1134 IQ2_XS, :1136-1166 IQ2_S,
// :1168-1198 IQ3_XXS, :1200-1239 IQ3_S, :1241-1264 IQ1_S).  Each decodes 32 consecutive values [32u, 32u + 32) of a block.

__host__ __device__ inline uint32_t ld_u16le(const uint8_t* p) { return (uint32_t) p[0] | ((uint32_t) p[1] << 8); }
__host__ __device__ inline uint32_t ld_u32le(const uint8_t* p) { return ld_u16le(p) | (ld_u16le(p + 2) << 16); }

// the sign byte of a 7-bit sign index: the eighth sign makes the number of minus signs even (ggml's ksigns_iq2xs)
__host__ __device__ inline uint32_t iq_signs7(uint32_t i) {
    uint32_t p = i ^ (i >> 4);
    p ^= p >> 2;
    p ^= p >> 1;
    return i | ((p & 1u) << 7);
}
__host__ __device__ inline float iq2_mag(uint32_t c) { return c == 0u ? 8.f : c == 1u ? 25.f : 43.f; }
__host__ __device__ inline float iq3xxs_mag(uint32_t c) { return c == 7u ? 62.f : (float) (4u + 8u * c); }

// 8 values of an IQ2 codebook point (2 bits a coordinate) times db, with the sign bits of `signs`
__host__ __device__ inline void iq2_point(uint32_t point, uint32_t signs, float db, float* y) {
    for (int j = 0; j < 8; ++j) {
        const float v = db * iq2_mag((point >> (2 * j)) & 3u);
        y[j] = ((signs >> j) & 1u) ? -v : v;
    }
}

// Q2_0: 18 bytes per 64 values (fp16 d, 16 code bytes, four 2-bit codes a byte: 0 -> -1, 1 -> 0, 2 -> +1, 3 -> +2); u = 32-value half
__host__ __device__ inline void decode_q2_0_32(const uint8_t* b, int u, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint8_t* q = b + 2 + 8 * u;
    for (int j = 0; j < 32; ++j) y[j] = (float) ((int) ((q[j >> 2] >> (2 * (j & 3))) & 3) - 1) * d;
}

// Q2_K: 84 bytes (scales[16]: 4-bit scale | 4-bit min << 4, qs[64], fp16 d, fp16 dmin); 16 values share a scale byte
__host__ __device__ inline void decode_q2k_32(const uint8_t* b, int u, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b + 80)), dmin = half_bits_to_float((uint16_t) ld_u16le(b + 82));
    const int half = u >> 2, shift = 2 * (u & 3);
    const uint8_t* q = b + 16 + 32 * half;
    for (int h = 0; h < 2; ++h) {
        const uint8_t sc = b[8 * half + 2 * (u & 3) + h];
        const float dl = d * (float) (sc & 0xF), ml = dmin * (float) (sc >> 4);
        for (int l = 0; l < 16; ++l) y[16 * h + l] = mul_then_sub(dl, (float) ((q[16 * h + l] >> shift) & 3), ml);
    }
}

// Q3_K: 110 bytes (hmask[32], qs[64], scales[12] = sixteen 6-bit scales, fp16 d); value = d (scale - 32) (2-bit code - (high bit ? 0 : 4))
__host__ __device__ inline void decode_q3k_32(const uint8_t* b, int u, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b + 108));
    const int half = u >> 2, j = u & 3, shift = 2 * j;
    const uint32_t m = 1u << (4 * half + j);
    const uint8_t* hm = b;
    const uint8_t* q = b + 32 + 32 * half;
    const uint8_t* s12 = b + 96;
    for (int h = 0; h < 2; ++h) {
        const int is = 8 * half + 2 * j + h;
        // scale `is` of the sixteen: low 4 bits from byte is (is < 8: low nibble of s12[is]; else high nibble of s12[is - 8]), high 2 bits
        // from bytes 8..11 (byte 8 + is % 4, bit pair is / 4)
        const uint32_t lo = is < 8 ? (s12[is] & 0xFu) : (s12[is - 8] >> 4);
        const uint32_t hi = (s12[8 + (is & 3)] >> (2 * (is >> 2))) & 3u;
        const float dl = d * (float) ((int) (lo | (hi << 4)) - 32);
        for (int l = 0; l < 16; ++l) {
            const int c = (int) ((q[16 * h + l] >> shift) & 3) - ((hm[16 * h + l] & m) ? 0 : 4);
            y[16 * h + l] = dl * (float) c;
        }
    }
}

// IQ2_XXS: 66 bytes (fp16 d, per 32 values 8 bytes: four point indices, then 4 x 7 sign bits and a 4-bit scale)
__host__ __device__ inline void decode_iq2xxs_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint8_t* q = b + 2 + 8 * u;
    const uint32_t aux = ld_u32le(q + 4);
    const float db = d * (0.5f + (float) (aux >> 28)) * 0.25f;
    for (int l = 0; l < 4; ++l) iq2_point(grid[kGridIQ2XXS + q[l]], iq_signs7((aux >> (7 * l)) & 127u), db, y + 8 * l);
}

// IQ2_XS: 74 bytes (fp16 d, qs[32] uint16 = 9-bit point | 7 sign bits << 9, scales[8]: a 4-bit scale per 16 values)
__host__ __device__ inline void decode_iq2xs_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint8_t sc = b[66 + u];
    const float db[2] = {d * (0.5f + (float) (sc & 0xF)) * 0.25f, d * (0.5f + (float) (sc >> 4)) * 0.25f};
    for (int l = 0; l < 4; ++l) {
        const uint32_t q = ld_u16le(b + 2 + 2 * (4 * u + l));
        iq2_point(grid[kGridIQ2XS + (q & 511u)], iq_signs7(q >> 9), db[l >> 1], y + 8 * l);
    }
}

// IQ2_S: 82 bytes (fp16 d, qs[64] = 32 point low bytes then 32 sign bytes, qh[8]: two more point bits per group, scales[8])
__host__ __device__ inline void decode_iq2s_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint8_t sc = b[74 + u];
    const float db[2] = {d * (0.5f + (float) (sc & 0xF)) * 0.25f, d * (0.5f + (float) (sc >> 4)) * 0.25f};
    const uint32_t qh = b[66 + u];
    for (int l = 0; l < 4; ++l) {
        const uint32_t idx = b[2 + 4 * u + l] | ((qh << (8 - 2 * l)) & 0x300u);
        iq2_point(grid[kGridIQ2S + idx], b[2 + 32 + 4 * u + l], db[l >> 1], y + 8 * l);
    }
}

// IQ3_XXS: 98 bytes (fp16 d, qs[64]: a point index per 4 values, then per 32 values a word of 4 x 7 sign bits and a 4-bit scale)
__host__ __device__ inline void decode_iq3xxs_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint32_t aux = ld_u32le(b + 2 + 64 + 4 * u);
    const float db = d * (0.5f + (float) (aux >> 28)) * 0.5f;
    for (int l = 0; l < 4; ++l) {
        const uint32_t signs = iq_signs7((aux >> (7 * l)) & 127u);
        for (int h = 0; h < 2; ++h) {
            const uint32_t point = grid[kGridIQ3XXS + b[2 + 8 * u + 2 * l + h]];
            for (int j = 0; j < 4; ++j) {
                const float v = db * iq3xxs_mag((point >> (3 * j)) & 7u);
                y[8 * l + 4 * h + j] = ((signs >> (4 * h + j)) & 1u) ? -v : v;
            }
        }
    }
}

// IQ3_S: 110 bytes (fp16 d, qs[64], qh[8]: the ninth point bit per 4 values, signs[32], scales[4]: a 4-bit scale per 32 values)
__host__ __device__ inline void decode_iq3s_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint32_t nib = (b[106 + (u >> 1)] >> (4 * (u & 1))) & 0xFu;
    const float db = d * (float) (1 + 2 * (int) nib);
    const uint32_t qh = b[66 + u];
    for (int l = 0; l < 4; ++l) {
        const uint32_t signs = b[74 + 4 * u + l];
        for (int h = 0; h < 2; ++h) {
            const uint32_t idx = b[2 + 8 * u + 2 * l + h] | ((qh << ((h ? 7 : 8) - 2 * l)) & 256u);
            const uint32_t point = grid[kGridIQ3S + idx];
            for (int j = 0; j < 4; ++j) {
                const float v = db * (float) (2u * ((point >> (3 * j)) & 7u) + 1u);
                y[8 * l + 4 * h + j] = ((signs >> (4 * h + j)) & 1u) ? -v : v;
            }
        }
    }
}

// IQ1_S: 50 bytes (fp16 d, qs[32], qh[16] uint16: 4 x 3 high index bits, a 3-bit scale, the delta sign); value = d (2 s + 1) (g +- 1/8)
__host__ __device__ inline void decode_iq1s_32(const uint8_t* b, int u, const uint16_t* grid, float* y) {
    const float d = half_bits_to_float((uint16_t) ld_u16le(b));
    const uint32_t qh = ld_u16le(b + 34 + 2 * u);
    const float dl = d * (float) (2 * (int) ((qh >> 12) & 7u) + 1);
    const float delta = (qh & 0x8000u) ? -0.125f : 0.125f;
    for (int l = 0; l < 4; ++l) {
        const uint32_t g = grid[kGridIQ1 + (b[2 + 4 * u + l] | (((qh >> (3 * l)) & 7u) << 8))];
        for (int j = 0; j < 8; ++j) y[8 * l + j] = dl * ((float) ((int) ((g >> (2 * j)) & 3u) - 1) + delta);
    }
}

// 32 consecutive values [32 unit, 32 unit + 32) of a row of any supported format
__host__ __device__ inline void decode_any_32(int type, const uint8_t* row, int unit, const uint16_t* grid, float* y) {
    switch (type) {
        case kTypeNVFP4: {
            float t[64];
            decode_block_nvfp4(row + (size_t) (unit >> 1) * 36, t);
            for (int i = 0; i < 32; ++i) y[i] = t[32 * (unit & 1) + i];
            break;
        }
        case kTypeQ6K: decode_q6k_32(row + (size_t) (unit >> 3) * 210, unit & 7, y); break;
        case kTypeQ8_0: decode_q8_0_32(row + (size_t) unit * 34, y); break;
        case kTypeQ4K: decode_q4k_32(row + (size_t) (unit >> 3) * 144, unit & 7, y); break;
        case kTypeQ5K: decode_q5k_32(row + (size_t) (unit >> 3) * 176, unit & 7, y); break;
        case kTypeQ5_0: decode_q5_01_32(row + (size_t) unit * 22, false, y); break;
        case kTypeQ5_1: decode_q5_01_32(row + (size_t) unit * 24, true, y); break;
        case kTypeIQ4NL: decode_iq4nl_32(row + (size_t) unit * 18, y); break;
        case kTypeIQ4XS: decode_iq4xs_32(row + (size_t) (unit >> 3) * 136, unit & 7, y); break;
        case kTypeIQ1M: decode_iq1m_32(row + (size_t) (unit >> 3) * 56, unit & 7, grid, y); break;
        case kTypeQ2_0: decode_q2_0_32(row + (size_t) (unit >> 1) * 18, unit & 1, y); break;
        case kTypeQ2K: decode_q2k_32(row + (size_t) (unit >> 3) * 84, unit & 7, y); break;
        case kTypeQ3K: decode_q3k_32(row + (size_t) (unit >> 3) * 110, unit & 7, y); break;
        case kTypeIQ2XXS: decode_iq2xxs_32(row + (size_t) (unit >> 3) * 66, unit & 7, grid, y); break;
        case kTypeIQ2XS: decode_iq2xs_32(row + (size_t) (unit >> 3) * 74, unit & 7, grid, y); break;
        case kTypeIQ2S: decode_iq2s_32(row + (size_t) (unit >> 3) * 82, unit & 7, grid, y); break;
        case kTypeIQ3XXS: decode_iq3xxs_32(row + (size_t) (unit >> 3) * 98, unit & 7, grid, y); break;
        case kTypeIQ3S: decode_iq3s_32(row + (size_t) (unit >> 3) * 110, unit & 7, grid, y); break;
        case kTypeIQ1S: decode_iq1s_32(row + (size_t) (unit >> 3) * 50, unit & 7, grid, y); break;
        default:
            for (int i = 0; i < 32; ++i) y[i] = 0.f;
    }
}

}  // namespace bsx
