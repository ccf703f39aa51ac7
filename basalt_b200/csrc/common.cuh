// common.cuh - small helpers shared by the kernels of the MoE layer.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/basalt_b200.h"

namespace bsx {

constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
    for (int m = 16; m; m >>= 1) v += __shfl_xor_sync(kFull, v, m);
    return v;
}
__device__ __forceinline__ float warp_max_xor(float v) {
#pragma unroll
    for (int m = 16; m; m >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, m));
    return v;
}

// status of the last launch on this thread's device as an ABI return value
inline int32_t launch_status() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? BSX_OK : (int32_t) e;
}

inline bool aligned(const void* p, size_t a) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// number of SMs of the current device (cached per device; 148 on a B200)
int sm_count();

}  // namespace bsx
