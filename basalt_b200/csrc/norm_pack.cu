// norm_pack.cu - the step before the MoE layer: the RMS norm of the layer's input rows, written as fp32 rows (what the router
// reads) and / or bf16 rows, one launch.  Replaces basalt::kernels::wgemm::norm_pack (include/basalt/kernels/window_gemm.hpp:
// 36-40, src/kernels/cuda/window_gemm.cu:75-112,256-266) bit for bit.  The variant that also writes the FP4 images the packed
// expert kernels read lives beside them (experts_nvf4.cu).
#include "norm.cuh"

namespace bsx {
namespace {

template <bool BF16>
__global__ void __launch_bounds__(kNormThreads) norm_pack_kernel(const void* __restrict__ x, const float* __restrict__ w, float eps, int64_t K,
                                                                 uint16_t* __restrict__ act, float* __restrict__ xn) {
    __shared__ float red[kNormThreads / 32];
    norm_row<BF16>(x, w, eps, K, blockIdx.x, act, xn, red);
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" int32_t bsx_norm_pack(const void* x, int32_t x_kind, const float* w, float eps, int64_t K, int32_t T, void* act, float* xn,
                                 void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16) return BSX_E_TYPE;
    if (K <= 0 || T < 0) return BSX_E_GEOMETRY;
    if (T == 0) return BSX_OK;
    if (!x || !w || (!act && !xn)) return BSX_E_POINTER;
    cudaStream_t st = (cudaStream_t) stream;
    if (x_kind == BSX_X_BF16) norm_pack_kernel<true><<<(unsigned) T, kNormThreads, 0, st>>>(x, w, eps, K, static_cast<uint16_t*>(act), xn);
    else norm_pack_kernel<false><<<(unsigned) T, kNormThreads, 0, st>>>(x, w, eps, K, static_cast<uint16_t*>(act), xn);
    return launch_status();
}
