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

// Sum of one float per thread over the block: lanes by xor butterfly, then the warp sums added in warp order by every thread.
// scratch: one float per warp.  Two block barriers.
__device__ __forceinline__ float block_sum_warp_order(float v, float* scratch) {
#pragma unroll
    for (int m = 16; m; m >>= 1) v += __shfl_xor_sync(kFull, v, m);
    __syncthreads();                                  // the scratch may still be read by the call before
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < kNormThreads / 32; ++i) total += scratch[i];
    return total;
}

// Row `row` of x ([.][K] fp32 or bf16) -> xn (fp32 row, may be null) and act (bf16 row, may be null).  Every thread of the
// block calls; red: 16 floats of shared memory.  Ends with a block barrier, after which the block sees the rows it wrote.
//
// A thread's columns are tid, tid + 512, ...  The first kKeep of them stay in registers from the squares to the scaling (a row
// of up to 8192 values is read once); columns past those are read again.  Squares enter the chain in column order either way,
// and a column past the row's end adds fmaf(0, 0, s) = s, so no bounds test sits inside the chain.
template <bool BF16>
__device__ __forceinline__ void norm_row(const void* __restrict__ x, const float* __restrict__ w, float eps, int64_t K, int64_t row,
                                         uint16_t* __restrict__ act, float* __restrict__ xn, float* red) {
    constexpr int kKeep = 16;
    const int64_t first = row * K;
    const int64_t mine = threadIdx.x;
    const int64_t beyond = mine + (int64_t) kKeep * kNormThreads;   // this thread's first column that is not kept
    float keep[kKeep];
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int64_t c = mine + (int64_t) j * kNormThreads;
        keep[j] = c < K ? norm_load<BF16>(x, first + c) : 0.f;
        sq = fmaf(keep[j], keep[j], sq);
    }
    for (int64_t c = beyond; c < K; c += kNormThreads) {
        const float v = norm_load<BF16>(x, first + c);
        sq = fmaf(v, v, sq);
    }
    const float scale = rsqrtf(block_sum_warp_order(sq, red) / (float) K + eps);
    auto put = [&](int64_t c, float value) {
        const float v = value * scale * w[c];
        if (xn) xn[first + c] = v;
        if (act) act[first + c] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
    };
#pragma unroll
    for (int j = 0; j < kKeep; ++j) {
        const int64_t c = mine + (int64_t) j * kNormThreads;
        if (c < K) put(c, keep[j]);
    }
    for (int64_t c = beyond; c < K; c += kNormThreads) put(c, norm_load<BF16>(x, first + c));
    __syncthreads();
}

}  // namespace bsx
