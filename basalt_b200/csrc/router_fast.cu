// router_fast.cu - the fp32 softmax top-k router built with --use_fast_math (expf -> ex2.approx, 1/x -> rcp.approx, flush to
// zero), as the Basalt decode path builds its own (src/models/qwen4exp/kernels/native_router.cu:44-99 with the flags of
// CMakeLists.txt:572-590), so that BSX_GATE_SOFTMAX_FAST gives that kernel's bits.  Only this file gets the flag.
#define BSX_SOFTMAX_KERNEL softmax_topk_fast_kernel
#define BSX_SOFTMAX_TOKEN softmax_topk_fast_token
#define BSX_SOFTMAX_LAUNCH softmax_topk_fast_launch
#define BSX_SOFTMAX_RECIPROCAL 1
#include "router_softmax.cuh"

namespace bsx {
int32_t softmax_fast(const float* logits, int64_t T, int E, int k, int32_t* ids, float* w, cudaStream_t st) {
    return softmax_topk_fast_launch(logits, T, E, k, ids, w, st);
}
}  // namespace bsx
