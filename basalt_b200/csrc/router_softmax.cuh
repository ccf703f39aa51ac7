// router_softmax.cuh - the one-warp-per-token fp32 softmax top-k router, included by two translation units: router.cu
// (IEEE expf and division; the Basalt prompt path's route_kernel, src/models/qwen4exp/prefill/kernels.cu:351-390) and
// router_fast.cu (built with --use_fast_math, weight = p * (1 / sum); the decode path's route,
// src/models/qwen4exp/kernels/native_router.cu:44-99).  The including file defines BSX_SOFTMAX_KERNEL (the kernel's name)
// BSX_SOFTMAX_TOKEN (the per-token device routine's name) and BSX_SOFTMAX_RECIPROCAL (0: divide, 1: multiply by the reciprocal).
//
// Arithmetic order, which fixes every bit of the result: lane l holds experts l, l+32, ...; max over all experts; per lane
// v = expf(v - max) summed in index order, lanes summed by xor butterfly; v *= 1/sum; NaN -> -FLT_MAX; k argmax passes
// (value descending, index ascending); the chosen probabilities are added per WINNING lane in selection order, lanes summed
// by butterfly, clamped below at 2^-14.  The reference instantiates 512 and 256 experts with k = 10 only; this is the same
// sequence for any E % 32 == 0 (E <= 1024) and k <= 32.
#include <cfloat>

#include "common.cuh"
#include "pdl.cuh"

namespace bsx {

// one token by one warp: lg = the token's E logits; ids / wout = its k outputs
template <int REGT>
__device__ __forceinline__ void BSX_SOFTMAX_TOKEN(const float* __restrict__ lg, int32_t* __restrict__ ids, float* __restrict__ wout, int E, int k) {
    constexpr int MAXR = REGT > 0 ? REGT : 32;
    const int lane = threadIdx.x & 31;
    const int reg = REGT > 0 ? REGT : (E >> 5);
    float v[MAXR];
#pragma unroll
    for (int i = 0; i < MAXR; ++i) v[i] = i < reg ? lg[lane + i * 32] : -INFINITY;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAXR; ++i)
        if (i < reg) mx = fmaxf(mx, v[i]);
    mx = warp_max_xor(mx);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < MAXR; ++i)
        if (i < reg) { v[i] = expf(v[i] - mx); sum += v[i]; }
    const float rcp = 1.0f / warp_sum_xor(sum);
#pragma unroll
    for (int i = 0; i < MAXR; ++i)
        if (i < reg) { v[i] *= rcp; if (isnan(v[i])) v[i] = -FLT_MAX; }
    // k argmax passes (value descending, index ascending).  Floats are compared through an order-preserving map to
    // unsigned integers, so the warp-wide maximum and the lowest index holding it are one redux instruction each; a lane
    // keeps the maximum of its own values and only the winning lane rescans.  (+0 and -0 would order differently from the
    // float compare, but a probability here is +0 at the lowest, and the markers -FLT_MAX and -inf are distinct values.)
    // The values stay in registers: every index into v[] below is a compile-time constant.  (Reading "the winner's value" as
    // v[ex >> 5] makes the compiler put the array in local memory, and the selection becomes a chain of L1 round trips -
    // measured ~6 us a token.)  A chosen value is recovered from its key, and chosen positions are remembered in a bit mask.
    float selected = 0.0f, selected_sum = 0.0f;
    auto key = [](float f) { const uint32_t b = __float_as_uint(f); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); };
    auto unkey = [](uint32_t q) { return __uint_as_float((q & 0x80000000u) ? (q & 0x7FFFFFFFu) : ~q); };
    uint32_t kv[MAXR];
#pragma unroll
    for (int i = 0; i < MAXR; ++i) kv[i] = i < reg ? key(v[i]) : 0u;
    uint32_t lmax = 0u, taken = 0u;
    int lidx = 0;
    auto rescan = [&]() {
        lmax = 0u;       // below every key (the key of -inf is 0x007FFFFF)
        lidx = 0;
#pragma unroll
        for (int i = 0; i < MAXR; ++i)
            if (i < reg && !((taken >> i) & 1u) && kv[i] > lmax) { lmax = kv[i]; lidx = i; }
    };
    rescan();
    for (int rank = 0; rank < k; ++rank) {
        const uint32_t gmax = __reduce_max_sync(kFull, lmax);
        const int ex = (int) __reduce_min_sync(kFull, lmax == gmax ? (unsigned) (lane + lidx * 32) : 0xFFFFFFFFu);
        float best = 0.f;
        if ((ex & 31) == lane) {
            best = unkey(lmax);
            taken |= 1u << lidx;
            selected_sum += best;
            rescan();
        }
        best = __shfl_sync(kFull, best, ex & 31);
        if (lane == 0) ids[rank] = ex;
        if (rank == lane) selected = best;
    }
    selected_sum = fmaxf(warp_sum_xor(selected_sum), 6.103515625e-5f);
#if BSX_SOFTMAX_RECIPROCAL
    const float inv = 1.0f / selected_sum;
    if (lane < k) wout[lane] = selected * inv;
#else
    if (lane < k) wout[lane] = selected / selected_sum;
#endif
}

template <int REGT>
__global__ void __launch_bounds__(256) BSX_SOFTMAX_KERNEL(const float* __restrict__ logits, int32_t* __restrict__ ids,
                                                         float* __restrict__ wout, int64_t T, int E, int k) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t t = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    BSX_SOFTMAX_TOKEN<REGT>(logits + t * E, ids + t * k, wout + t * k, E, k);
}

static inline int32_t BSX_SOFTMAX_LAUNCH(const float* logits, int64_t T, int E, int k, int32_t* ids, float* w, cudaStream_t st) {
    // decode windows: two tokens a block, so the window's selections spread over the SMs instead of queueing on a few
    const unsigned wpb = T <= 256 ? 2u : 8u, blocks = (unsigned) ((T + wpb - 1) / wpb);
    switch (E >> 5) {
        case 2: launch_k(BSX_SOFTMAX_KERNEL<2>, dim3(blocks), dim3(32 * wpb), 0, st, logits, ids, w, T, E, k); break;
        case 4: launch_k(BSX_SOFTMAX_KERNEL<4>, dim3(blocks), dim3(32 * wpb), 0, st, logits, ids, w, T, E, k); break;
        case 8: launch_k(BSX_SOFTMAX_KERNEL<8>, dim3(blocks), dim3(32 * wpb), 0, st, logits, ids, w, T, E, k); break;
        case 12: launch_k(BSX_SOFTMAX_KERNEL<12>, dim3(blocks), dim3(32 * wpb), 0, st, logits, ids, w, T, E, k); break;
        case 16: launch_k(BSX_SOFTMAX_KERNEL<16>, dim3(blocks), dim3(32 * wpb), 0, st, logits, ids, w, T, E, k); break;
        default: launch_k(BSX_SOFTMAX_KERNEL<0>, dim3(blocks), dim3(32 * wpb), 0, st, logits, ids, w, T, E, k); break;
    }
    return launch_status();
}

}  // namespace bsx
