// norm.cuh - the RMS norm of one activation row by one 512-thread block, in the summation order the Basalt engine fixes for
// its norm_pack / rms_norm_rows kernels (src/kernels/cuda/window_gemm.cu:40-112): thread i owns columns i, i + 512, ... as one
// fmaf chain of squares, a warp's 32 chains are summed by xor butterfly, the 16 warp sums are added in warp order,
// inv = rsqrtf(sum / K + eps), value = (x * inv) * w.  Same order, same operations: the rows carry the reference's bits.
#pragma once
#include "common.cuh"

#include <cuda_bf16.h>

namespace bsx {

constexpr int kNormThreads = 512;

template <bool BF16>
__device__ __forceinline__ float norm_load(const void* x, int64_t i) {
    if (BF16) return __uint_as_float((uint32_t) static_cast<const uint16_t*>(x)[i] << 16);
    return static_cast<const float*>(x)[i];
}

// Row `row` of x ([.][K] fp32 or bf16) -> xn (fp32 row, may be null) and act (bf16 row, may be null).  Every thread of the
// block calls; red: 16 floats of shared memory.  Ends with a block barrier, after which the block sees the rows it wrote.
template <bool BF16>
__device__ __forceinline__ void norm_row(const void* __restrict__ x, const float* __restrict__ w, float eps, int64_t K, int64_t row,
                                         uint16_t* __restrict__ act, float* __restrict__ xn, float* red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t base = row * K;
    constexpr int kHeld = 16;                       // rows up to 8192 values stay in registers between the two passes
    const bool held = K <= (int64_t) kHeld * kNormThreads;
    float xv[kHeld];
    float ss = 0.f;
    if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
            const int64_t c = tid + (int64_t) j * kNormThreads;
            xv[j] = c < K ? norm_load<BF16>(x, base + c) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kHeld; ++j)
            if (tid + (int64_t) j * kNormThreads < K) ss = fmaf(xv[j], xv[j], ss);
    } else {
        for (int64_t c = tid; c < K; c += kNormThreads) {
            const float v = norm_load<BF16>(x, base + c);
            ss = fmaf(v, v, ss);
        }
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) ss += __shfl_xor_sync(kFull, ss, m);
    __syncthreads();
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) t += red[i];
    const float inv = rsqrtf(t / (float) K + eps);
    if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
            const int64_t c = tid + (int64_t) j * kNormThreads;
            if (c < K) {
                const float v = xv[j] * inv * w[c];
                if (xn) xn[base + c] = v;
                if (act) act[base + c] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
            }
        }
    } else {
        for (int64_t c = tid; c < K; c += kNormThreads) {
            const float v = norm_load<BF16>(x, base + c) * inv * w[c];
            if (xn) xn[base + c] = v;
            if (act) act[base + c] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
        }
    }
    __syncthreads();
}

}  // namespace bsx
