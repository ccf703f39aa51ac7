// nvf4.cuh - what the block-scaled FP4 (tcgen05 kind::mxf4nvf4) expert kernels share: the geometry of a packed blob, and the
// kernel-side routine that turns an activation row into FP4 terms.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"
#include "experts.cuh"

namespace bsx {

constexpr int kTermsF = 4;                 // FP4 terms per activation row

// A matrix of R rows x K columns becomes (R / 128) x (K / 256) blocks of kBlockF bytes, row tile major: the block of
// (tile, chunk) holds that tile's 128 rows x 256 columns of codes as the 16 KB image a stage wants in shared memory
// (128-byte rows, 16-byte pieces XOR-swizzled by row % 8), followed by the rows' scale words of the chunk's four K-steps,
// each step as 32 lanes x 4 words (word (l, j) = row 32 j + l): what tcgen05.cp reads.  One block = one contiguous 18 KB
// run of HBM = one bulk copy.  Blob: gate blocks, up blocks, down blocks, the fp32 tail.
constexpr int kBlockF = 128 * 128 + 4 * 512;     // 18,432
struct PackedGeom {
    size_t gate, up, down, tail, bytes;
};
__host__ __device__ inline PackedGeom packed_geom(int64_t H, int64_t I) {
    PackedGeom g;
    const size_t gu = (size_t) (I / 128) * (size_t) (H / 256) * kBlockF, d = (size_t) (H / 128) * (size_t) (I / 256) * kBlockF;
    g.gate = 0;
    g.up = gu;
    g.down = 2 * gu;
    g.tail = 2 * gu + d;
    g.bytes = g.tail + 16;
    return g;
}

// UE4M3 (bias 7, no sign, 0x7F unused): the value of a byte, and the smallest byte whose value times 6 reaches amax.
__device__ __forceinline__ float ue4m3_value(uint32_t b) {
    // normal: 2^(e - 7) (1 + m / 8) = fp32 with exponent field e + 120 and the three mantissa bits on top; e = 0: m 2^-9
    return b >= 8u ? __uint_as_float((b + 960u) << 20) : (float) b * 0.001953125f;
}
__device__ __forceinline__ uint32_t ue4m3_cover(float amax) {
    if (!(amax > 0.f)) return 0u;
    const float t = amax * (1.f / 6.f);
    uint32_t b;
    if (t < 0.015625f) {
        b = (uint32_t) ceilf(t * 512.f);
    } else {
        const uint32_t bits = __float_as_uint(t) + 0x000FFFFFu;      // mantissa rounded up to three bits
        b = (bits >> 20) - 960u;                                      // (exponent field - 120) << 3 | mantissa
    }
    b = min(b, 0x7Eu);
    if (b > 0u && ue4m3_value(b - 1) * 6.f >= amax) --b;       // t was rounded up
    if (b < 0x7Eu && ue4m3_value(b) * 6.f < amax) ++b;         // ... or down
    return b;
}
// two floats -> two E2M1 codes (round to nearest even, saturating): `lo` in bits 0-3, `hi` in bits 4-7
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    uint16_t r;
    asm("{\n.reg .b8 t;\ncvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\ncvt.u16.u8 %0, t;\n}\n" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint32_t) r & 0xFFu;
}
// the two values of a code byte: low nibble -> .x, high nibble -> .y
__device__ __forceinline__ float2 e2m1x2_values(uint32_t c) {
    uint32_t h;
    asm("{\n.reg .b8 t;\ncvt.u8.u32 t, %1;\ncvt.rn.f16x2.e2m1x2 %0, t;\n}\n" : "=r"(h) : "r"(c));
    return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// TPR threads per activation row (32, 128 or 256: a thread per 16-value sub-block where the row allows), 256 / TPR rows a
// block; every thread of the block must call (the row maximum is reduced through `shf`, 8 floats of shared memory).
// The row times a power of two (largest magnitude into [2^7, 2^8), so block scales sit well inside UE4M3's range) becomes
// kTermsF FP4 terms.  Term t of a sub-block: scale = the smallest UE4M3 value s with 6 s >= the largest residual, codes =
// rn(residual / s), residual -= code value x s.  Layout: codes [image row][term][K / 2] bytes with ggml's nibble order
// (byte b of a sub-block = values b and b + 8), scales [image row][term][K / 16] bytes, inv[image row] undoes the power of two.
template <int TPR>
__device__ __forceinline__ void fp4_image_row(const void* src, int kind, int64_t row, int64_t K, bool live, int i, uint8_t* __restrict__ codes,
                                              uint8_t* __restrict__ sfs, float* __restrict__ inv, float* shf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tr = (int) threadIdx.x % TPR;
    const int n_sb = (int) (K >> 4);
    float amax = 0.f;
    if (live) {
        for (int sb = tr; sb < n_sb; sb += TPR) {
            float v[16];
            load16(src, kind, row, K, sb, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
        }
    }
    amax = warp_max_xor(amax);
    if (TPR > 32) {
        if (lane == 0) shf[warp] = amax;
        __syncthreads();
        const int w0 = (warp / (TPR / 32)) * (TPR / 32);
        amax = shf[w0];
#pragma unroll
        for (int w = 1; w < TPR / 32; ++w) amax = fmaxf(amax, shf[w0 + w]);
    }
    if (!live) return;
    int ex = 0;
    float s = 1.f, iv = 1.f;
    if (amax > 0.f && amax <= 3.0e38f) {
        frexpf(amax, &ex);                          // amax = f 2^ex, f in [0.5, 1)
        ex = max(-100, min(100, 8 - ex));
        s = ldexpf(1.f, ex);
        iv = ldexpf(1.f, -ex);
    }
    if (tr == 0) inv[i] = iv;
    for (int sb = tr; sb < n_sb; sb += TPR) {
        float v[16];
        load16(src, kind, row, K, sb, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= s;
#pragma unroll
        for (int t = 0; t < kTermsF; ++t) {
            float m = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) m = fmaxf(m, fabsf(v[j]));
            const uint32_t sb8 = ue4m3_cover(m);
            const float sv = ue4m3_value(sb8);
            uint32_t w0 = 0u, w1 = 0u;
            if (sv > 0.f) {
                const float rs = 1.f / sv;          // 6 sv >= every |v|, so |v rs| <= 6 up to rounding, which the conversion saturates
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    const uint32_t c = e2m1x2(v[b] * rs, v[b + 8] * rs);
                    const float2 q = e2m1x2_values(c);
                    v[b] -= q.x * sv;
                    v[b + 8] -= q.y * sv;
                    if (b < 4) w0 |= c << (8 * b);
                    else w1 |= c << (8 * (b - 4));
                }
            }
            const size_t r4 = (size_t) i * kTermsF + t;
            *reinterpret_cast<uint2*>(codes + r4 * (K / 2) + (size_t) sb * 8) = make_uint2(w0, w1);
            sfs[r4 * (K / 16) + sb] = (uint8_t) sb8;
        }
    }
}


}  // namespace bsx
