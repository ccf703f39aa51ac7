// TEST INFRASTRUCTURE, NOT PRODUCT.  C entry points over the reference engine's own portable CUDA kernels for the
// MoE-layer path, compiled from the reference checkout for sm_100a into oracle/_ref/libref_gpu.so by oracle/Makefile.
// The GPU parity tests use it as the on-device oracle for bit-exact routing (the reference's own expf/logf code paths)
// and as a behavioural check of the grouped decode experts.  Nothing from the reference is copied into this repository.
//
// Wrapped reference interfaces:
//   router / router_select            include/basalt/kernels/router.hpp:30-37
//   route_tail_skip                   include/basalt/kernels/route_lossy.hpp:58-59
//   router_top10                      include/basalt/models/qwen4exp/kernels/router_top10.hpp
//   native_router_top10_multi         include/basalt/models/qwen4exp/kernels/native_router.hpp
//   quantize_q8_1_rows, native_expert_layout, native_expert_scratch_bytes, native_expert_grouped
//                                     include/basalt/kernels/iq_kernels.hpp:23,68,75,84
//   native_moe_combine_multi          include/basalt/models/qwen4exp/kernels/native_moe.hpp
//   wgemm::norm_pack                  include/basalt/kernels/window_gemm.hpp:36-40
// Restated here (their translation unit has many unrelated dependencies and cannot be compiled alone):
//   route_kernel<REG> / route()       src/models/qwen4exp/prefill/kernels.cu:351-390,639-647 (the fp32 one-warp softmax top-k)
//   the gate score of router_select   src/kernels/cuda/router.cu:148-153 (sigmoid, sqrt-softplus), one value per thread
#include "basalt/kernels/iq_kernels.hpp"
#include "basalt/kernels/router.hpp"
#include "basalt/kernels/window_gemm.hpp"
#include "basalt/models/qwen4exp/kernels/native_moe.hpp"
#include "basalt/models/qwen4exp/kernels/native_router.hpp"
#include "basalt/models/qwen4exp/kernels/router_top10.hpp"

#include <cuda_runtime.h>

#include <cstdint>
#include <exception>

#include <cfloat>

using namespace basalt::kernels;

namespace {

// The prompt path's softmax router, restated with its order of operations: one warp per token, lane l holds experts l, l + 32,
// ...; maximum over all; per lane expf(v - max) summed in index order, lanes summed by xor butterfly; every value times the
// reciprocal of the sum; NaN -> -FLT_MAX; K argmax passes, each a per-lane scan (first strictly larger wins) followed by a
// butterfly that prefers the larger value and, on equal values, the lower index; the winner's probability is added on the
// winning lane; the per-lane sums go through the butterfly, are clamped below at 2^-14, and divide the chosen values.
// The reference instantiates REG = 16 and 8 with K = 10; other REG / K are the same sequence at another size.
__device__ __forceinline__ float shim_warp_max(float v) {
    for (int m = 16; m; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}
__device__ __forceinline__ float shim_warp_sum(float v) {
    for (int m = 16; m; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
template <int REG>
__global__ void shim_route_kernel(const float* __restrict__ logits, int32_t* __restrict__ ids, float* __restrict__ wout, int64_t T, int K) {
    const int64_t t = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const int lane = threadIdx.x & 31;
    const float* row = logits + t * (REG * 32);
    float p[REG];
#pragma unroll
    for (int i = 0; i < REG; ++i) p[i] = row[lane + 32 * i];
    float top = -INFINITY;
#pragma unroll
    for (int i = 0; i < REG; ++i) top = fmaxf(top, p[i]);
    top = shim_warp_max(top);
    float lane_sum = 0.0f;
#pragma unroll
    for (int i = 0; i < REG; ++i) {
        p[i] = expf(p[i] - top);
        lane_sum += p[i];
    }
    const float inv = 1.0f / shim_warp_sum(lane_sum);
#pragma unroll
    for (int i = 0; i < REG; ++i) {
        p[i] *= inv;
        if (isnan(p[i])) p[i] = -FLT_MAX;
    }
    float mine = 0.0f, won = 0.0f;
    for (int r = 0; r < K; ++r) {
        float bv = p[0];
        int bi = lane;
#pragma unroll
        for (int i = 1; i < REG; ++i)
            if (p[i] > bv) { bv = p[i]; bi = lane + 32 * i; }
        for (int m = 16; m; m >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((bi & 31) == lane) {
#pragma unroll
            for (int i = 0; i < REG; ++i)
                if (i == bi / 32) p[i] = -INFINITY;
            won += bv;
        }
        if (lane == 0) ids[t * K + r] = bi;
        if (lane == r) mine = bv;
    }
    const float denom = fmaxf(shim_warp_sum(won), 6.103515625e-5f);
    if (lane < K) wout[t * K + lane] = mine / denom;
}

// s = gate(x) exactly as router_select computes it on the device (router.cu:148-153): kind 1 = sigmoid, 0 = sqrt-softplus
__global__ void shim_gate_score_kernel(const float* __restrict__ x, float* __restrict__ s, int64_t n, int kind) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    if (kind == 1) {
        s[i] = 1.f / (1.f + expf(-v));
    } else {
        const float sp = v > 20.f ? v : logf(1.f + expf(v));
        s[i] = sqrtf(sp);
    }
}

}  // namespace

extern "C" {

// All pointers are device pointers.  Returns 0, -1 on a reference exception, or the CUDA error after synchronising.
static int finish() {
    const cudaError_t e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : (int) e;
}

int refg_router(const float* x, const float* gate, const float* bias, int T, int n_expert, int n_embd, int k, float scale,
                int gate_kind, float* logits, int32_t* ids, float* weights) {
    RouterArgs a;
    a.n_expert = n_expert; a.n_embd = n_embd; a.k = k; a.weight_scale = scale;
    a.gate = gate_kind == 1 ? RouterGate::Sigmoid : RouterGate::SqrtSoftplus;
    try { router(x, gate, bias, T, a, logits, ids, weights, nullptr); } catch (const std::exception&) { return -1; }
    return finish();
}

int refg_router_select(const float* logits, const float* bias, int T, int n_expert, int k, float scale, int gate_kind,
                       float prior, const int32_t* held, int32_t* ids, float* weights) {
    RouterArgs a;
    a.n_expert = n_expert; a.k = k; a.weight_scale = scale; a.prior = prior;
    a.gate = gate_kind == 1 ? RouterGate::Sigmoid : RouterGate::SqrtSoftplus;
    if (held) a.held.add(held);
    try { router_select(logits, bias, T, a, ids, weights, nullptr); } catch (const std::exception&) { return -1; }
    return finish();
}

int refg_route_tail_skip(int32_t* ids, float* weights, const int32_t* held, int n_entries, int k, int rank, int n_expert,
                         unsigned long long* counts) {
    ResidentTabs tabs;
    if (held) tabs.add(held);
    route_tail_skip(ids, weights, tabs, n_entries, k, rank, n_expert, counts, nullptr);
    return finish();
}

int refg_router_top10(const float* logits, int T, int n_expert, int k, int32_t* ids, float* weights) {
    router_top10(logits, T, n_expert, k, ids, weights, nullptr);
    return finish();
}

// the prompt path's route(): 512 or 256 experts with k = 10 are the reference's instantiations; 64, 128 and 1024 experts and
// other k (<= 32) run the same restated sequence at that size
int refg_route_softmax(const float* logits, int64_t T, int n_expert, int k, int32_t* ids, float* weights) {
    if (k < 1 || k > 32) return -1;
    const unsigned blocks = (unsigned) ((T + 7) / 8);
    switch (n_expert) {
        case 64: shim_route_kernel<2><<<blocks, 256>>>(logits, ids, weights, T, k); break;
        case 96: shim_route_kernel<3><<<blocks, 256>>>(logits, ids, weights, T, k); break;
        case 128: shim_route_kernel<4><<<blocks, 256>>>(logits, ids, weights, T, k); break;
        case 256: shim_route_kernel<8><<<blocks, 256>>>(logits, ids, weights, T, k); break;
        case 512: shim_route_kernel<16><<<blocks, 256>>>(logits, ids, weights, T, k); break;
        case 1024: shim_route_kernel<32><<<blocks, 256>>>(logits, ids, weights, T, k); break;
        default: return -1;
    }
    return finish();
}

int refg_gate_scores(const float* logits, int64_t n, int gate_kind, float* scores) {
    shim_gate_score_kernel<<<(unsigned) ((n + 255) / 256), 256>>>(logits, scores, n, gate_kind);
    return finish();
}

// the fp32 one-warp softmax router (512 experts, top-10 only; fast-math translation unit)
int refg_native_router_top10(const float* logits, int T, int32_t* ids, float* weights) {
    cudaStream_t s;
    if (cudaStreamCreate(&s) != cudaSuccess) return -2;
    int rc = 0;
    try { native_router_top10_multi(logits, ids, weights, T, s); } catch (const std::exception&) { rc = -1; }
    const int f = finish();
    cudaStreamDestroy(s);
    return rc ? rc : f;
}

int refg_quantize_q8_1(const float* x, int64_t rows, int64_t cols, void* y) {
    quantize_q8_1_rows(x, rows, cols, y, nullptr);
    return finish();
}

int64_t refg_expert_blob_bytes(int gu_type, int d_type, int64_t n_embd, int64_t n_ff) {
    if (!native_expert_supported(gu_type, d_type, n_embd, n_ff)) return 0;
    return (int64_t) native_expert_layout(gu_type, d_type, n_embd, n_ff).bytes;
}
int64_t refg_expert_scratch_bytes(int64_t cap_entries, int64_t n_ff) {
    return (int64_t) native_expert_scratch_bytes(cap_entries, n_ff);
}

// the reference's grouped decode experts on q8_1 activations (unweighted rows out)
int refg_expert_grouped(int gu_type, int d_type, int64_t n_embd, int64_t n_ff, float swiglu_limit,
                        const unsigned long long* grp_ptr, const int32_t* grp_start, const int32_t* n_groups,
                        const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries,
                        const void* x_q8_1, void* scratch, float* out) {
    if (!native_expert_supported(gu_type, d_type, n_embd, n_ff)) return -1;
    const NativeExpertLayout L = native_expert_layout(gu_type, d_type, n_embd, n_ff, swiglu_limit);
    cudaStream_t s;
    if (cudaStreamCreate(&s) != cudaSuccess) return -2;
    native_expert_grouped(L, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, x_q8_1, scratch, out, s);
    const int f = finish();
    cudaStreamDestroy(s);
    return f;
}

int refg_combine_multi(const float* parts, const float* weights, const float* shared, float* output, int64_t n_embd,
                       int64_t k, int n_tok) {
    cudaStream_t s;
    if (cudaStreamCreate(&s) != cudaSuccess) return -2;
    int rc = 0;
    try { native_moe_combine_multi(parts, weights, shared, output, n_embd, k, n_tok, s); } catch (const std::exception&) { rc = -1; }
    const int f = finish();
    cudaStreamDestroy(s);
    return rc ? rc : f;
}

// The RMS norm of T rows of K values (fp32, or bf16 when `bf16` is set) into bf16 rows `act` and fp32 rows `xn` (may be null).
int refg_norm_pack(const void* x, int bf16, const float* w, float eps, int64_t K, int T, void* act, float* xn) {
    try {
        if (bf16) wgemm::norm_pack((const uint16_t*) x, w, eps, K, T, act, xn, nullptr);
        else wgemm::norm_pack((const float*) x, w, eps, K, T, act, xn, nullptr);
    } catch (const std::exception&) { return -1; }
    return finish();
}

}  // extern "C"
