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

enum : int { kTypeQ5_0 = 6, kTypeQ5_1 = 7, kTypeQ8_0 = 8, kTypeQ4K = 12, kTypeQ5K = 13, kTypeQ6K = 14, kTypeIQ4NL = 20, kTypeIQ4XS = 23, kTypeIQ1M = 29,
              kTypeNVFP4 = 40 };

// values per block and bytes per block (the GGUF formats' constants, include/basalt/ggml/ggml_common.h)
__host__ __device__ constexpr int block_values(int type) {
    return type == kTypeNVFP4 ? 64 : (type == kTypeQ8_0 || type == kTypeQ5_0 || type == kTypeQ5_1 || type == kTypeIQ4NL) ? 32 : 256;
}
__host__ __device__ constexpr int block_bytes(int type) {
    return type == kTypeNVFP4 ? 36 : type == kTypeQ6K ? 210 : type == kTypeIQ1M ? 56 : type == kTypeQ8_0 ? 34 : type == kTypeQ4K ? 144
           : type == kTypeQ5K ? 176 : type == kTypeQ5_0 ? 22 : type == kTypeQ5_1 ? 24 : type == kTypeIQ4NL ? 18 : type == kTypeIQ4XS ? 136 : 0;
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

}  // namespace bsx
