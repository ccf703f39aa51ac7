// router.cu - the MoE router on sm_100a: gate-matrix logits, warp-level top-k selection for the sigmoid / sqrt-softplus
// gates (with the group-limited step), the fp32 and fp64 softmax routers, and the opt-in tail skip.
//
// Parity contract: logits, ids and weights carry the bits of the Basalt engine's kernels (src/kernels/cuda/router.cu,
// src/models/qwen4exp/prefill/kernels.cu:351-390, src/models/qwen4exp/kernels/router_top10.cu) on the same inputs.  The
// launch shapes are this library's own: several gate rows per block so a token vector is read once for all of them, and
// one warp per token for the selection instead of one block.
#define BSX_SOFTMAX_KERNEL softmax_topk_kernel
#define BSX_SOFTMAX_TOKEN softmax_topk_token
#define BSX_SOFTMAX_LAUNCH softmax_topk_launch
#define BSX_SOFTMAX_RECIPROCAL 0
#include "router_softmax.cuh"

#include <atomic>
#include <climits>
#include <cstdlib>

#include "plan.cuh"

namespace bsx {

int32_t softmax_fast(const float* logits, int64_t T, int E, int k, int32_t* ids, float* w, cudaStream_t st);

int sm_count() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

namespace {

constexpr int kLogitThreads = 256;   // the summation order is defined over 256 column-strided chains
constexpr int kTokTile = 8;

// G gate rows a block, NV float4 a thread and row.  Each (row, token) sum runs exactly as
// src/kernels/cuda/router.cu:49-88 defines it: thread i owns float4 columns i, i + 256, ... as one fmaf chain, the warp's 32
// chains are summed by xor butterfly, and the 8 warp sums are added in warp order.
// A token's columns as they lie in memory (four fp32, or four bf16 in a uint2) and widened to fp32.  The next token's
// columns are requested raw and widened only when their turn comes: a conversion right after the load would wait for it and
// undo the prefetch (measured: 5.5 us of a 37 us router stage at 64 bf16 tokens).
template <bool BF16> struct XRaw { using T = float4; };
template <> struct XRaw<true> { using T = uint2; };
template <bool BF16>
__device__ __forceinline__ typename XRaw<BF16>::T load_raw(const void* x, size_t row, int n_embd, int i) {
    if constexpr (BF16) return reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(x) + row * n_embd)[i];
    else return reinterpret_cast<const float4*>(static_cast<const float*>(x) + row * n_embd)[i];
}
__device__ __forceinline__ float4 widen(float4 v) { return v; }
__device__ __forceinline__ float4 widen(uint2 u) {
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xFFFF0000u));
}

// The G butterflies of one token at once (see router_logits_kernel): returns the row whose sum this lane ends up holding in acc[0].
template <int G>
__device__ __forceinline__ int merged_butterfly(float (&acc)[G], int lane) {
    int row = 0;
#pragma unroll
    for (int m = 16, n = G; m; m >>= 1) {
        if (n > 1) {
            const int half = n >> 1;
            const bool up = (lane & m) != 0;
#pragma unroll
            for (int i = 0; i < G / 2; ++i)
                if (i < half) {
                    const float keep = up ? acc[i + half] : acc[i];
                    const float send = up ? acc[i] : acc[i + half];
                    acc[i] = keep + __shfl_xor_sync(kFull, send, m);
                }
            if (up) row += half;
            n = half;
        } else {
            acc[0] += __shfl_xor_sync(kFull, acc[0], m);
        }
    }
    return row;
}

template <int NV, int G, bool BF16>
__global__ void __launch_bounds__(kLogitThreads, (NV <= 4 ? 2 : 1))
router_logits_kernel(const void* __restrict__ x, const float* __restrict__ gate, int n_embd, int n_expert, int n_tokens,
                     int tok_per_block, float* __restrict__ logits, int late_wait) {
    __shared__ float red[G][kTokTile][kLogitThreads / 32];
    const int n4 = n_embd >> 2;
    const int r0 = blockIdx.x * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4 w[G][NV];
    // the gate rows are constant weights: they are requested before the wait for the kernel that wrote x
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < NV; ++c) {
            const int i = threadIdx.x + c * kLogitThreads;
            w[g][c] = i < n4 ? reinterpret_cast<const float4*>(gate + (size_t) (r0 + g) * n_embd)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    // late_wait: x was complete before the kernel ahead of this one started (that kernel makes the expert kernels' images of x),
    // so this grid runs beside it and only orders itself after it before exiting
    if (!late_wait) pdl_wait();
    pdl_launch_dependents();
    const int t_begin = blockIdx.y * tok_per_block;
    const int t_end = min(n_tokens, t_begin + tok_per_block);
    for (int t0 = t_begin; t0 < t_end; t0 += kTokTile) {
        const int nt = min(kTokTile, t_end - t0);
        // the next token's columns are requested while the current token's sums run
        float4 xv[NV];
        typename XRaw<BF16>::T xn[NV] = {};
#pragma unroll
        for (int c = 0; c < NV; ++c) {
            const int i = threadIdx.x + c * kLogitThreads;
            xv[c] = i < n4 ? widen(load_raw<BF16>(x, (size_t) t0, n_embd, i)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int t = 0; t < nt; ++t) {
            if (t + 1 < nt) {
#pragma unroll
                for (int c = 0; c < NV; ++c) {
                    const int i = threadIdx.x + c * kLogitThreads;
                    if (i < n4) xn[c] = load_raw<BF16>(x, (size_t) (t0 + t + 1), n_embd, i);
                }
            }
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.f;
#pragma unroll
            for (int c = 0; c < NV; ++c) {
                const int i = threadIdx.x + c * kLogitThreads;
                if (i < n4) {
                    const float4 v = xv[c];
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        acc[g] = fmaf(w[g][c].x, v.x, acc[g]);
                        acc[g] = fmaf(w[g][c].y, v.y, acc[g]);
                        acc[g] = fmaf(w[g][c].z, v.z, acc[g]);
                        acc[g] = fmaf(w[g][c].w, v.w, acc[g]);
                    }
                }
            }
            // The G butterflies at once: at the xor-16, -8 and -4 stages a lane keeps half of its values and hands the other
            // half to its partner, so each stage adds exactly the pairs the plain butterfly adds (a + b == b + a bit for
            // bit); after the halving stages the lane holds one row's partial sum and the remaining stages run in full.
            const int row = merged_butterfly<G>(acc, lane);
            constexpr int kOwners = 32 / G;   // lanes holding the same row's sum
            if ((lane & (kOwners - 1)) == 0) red[row][t][warp] = acc[0];
#pragma unroll
            for (int c = 0; c < NV; ++c) xv[c] = widen(xn[c]);
        }
        __syncthreads();
        {
            const int g = threadIdx.x / kTokTile, t = threadIdx.x % kTokTile;
            if (g < G && t < nt) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < kLogitThreads / 32; ++i) s += red[g][t][i];
                logits[(size_t) (t0 + t) * n_expert + r0 + g] = s;
            }
        }
        __syncthreads();
    }
    if (late_wait) pdl_wait();
}


// The same sums for decode windows of 16 tokens and more: a block keeps G gate rows in registers, copies its share of the
// token rows into shared memory once (one contiguous range, 16-byte cp.async) and then runs every (row, token) chain from
// there, so a token's columns cost a shared-memory read instead of an L2 round trip per token and the grid is one wave of
// blocks that each read the gate rows once.  The order of every sum is unchanged: thread i owns float4 columns i, i + 256, ...
// as one fmaf chain, xor butterfly over the warp, the 8 warp sums in order.  The per-tile reduction buffer is doubled so a
// tile needs one block barrier.
template <int NV, int G, bool BF16>
__global__ void __launch_bounds__(kLogitThreads, 2)
router_logits_staged_kernel(const void* __restrict__ x, const float* __restrict__ gate, int n_embd, int n_expert, int n_tokens,
                            int tok_per_block, float* __restrict__ logits, int late_wait) {
    extern __shared__ __align__(16) uint8_t xsm[];
    __shared__ float red[2][G][kTokTile][kLogitThreads / 32];
    const int n4 = n_embd >> 2;
    const int r0 = blockIdx.x * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float4 w[G][NV];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int c = 0; c < NV; ++c) {
            const int i = threadIdx.x + c * kLogitThreads;
            w[g][c] = i < n4 ? reinterpret_cast<const float4*>(gate + (size_t) (r0 + g) * n_embd)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    // late_wait: x was complete before the kernel ahead of this one started (that kernel makes the expert kernels' images of x),
    // so this grid runs beside it and only orders itself after it before exiting
    if (!late_wait) pdl_wait();
    pdl_launch_dependents();
    const int t_begin = blockIdx.y * tok_per_block;
    const int nt_all = min(n_tokens, t_begin + tok_per_block) - t_begin;
    const size_t row_bytes = (size_t) n_embd * (BF16 ? 2 : 4);
    {
        const uint8_t* src = static_cast<const uint8_t*>(x) + (size_t) t_begin * row_bytes;
        const uint32_t dst = (uint32_t) __cvta_generic_to_shared(xsm);
        const int pieces = (int) ((size_t) nt_all * row_bytes >> 4);
        for (int i = threadIdx.x; i < pieces; i += kLogitThreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + (uint32_t) i * 16u), "l"(src + (size_t) i * 16) : "memory");
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();
    int tile = 0;
    for (int t0 = 0; t0 < nt_all; t0 += kTokTile, ++tile) {
        const int nt = min(kTokTile, nt_all - t0);
        float (*rd)[kTokTile][kLogitThreads / 32] = red[tile & 1];
#pragma unroll 2
        for (int t = 0; t < nt; ++t) {
            const uint8_t* xrow = xsm + (size_t) (t0 + t) * row_bytes;
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; ++g) acc[g] = 0.f;
#pragma unroll
            for (int c = 0; c < NV; ++c) {
                const int i = threadIdx.x + c * kLogitThreads;
                if (i < n4) {
                    float4 v;
                    if constexpr (BF16) v = widen(reinterpret_cast<const uint2*>(xrow)[i]);
                    else v = reinterpret_cast<const float4*>(xrow)[i];
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        acc[g] = fmaf(w[g][c].x, v.x, acc[g]);
                        acc[g] = fmaf(w[g][c].y, v.y, acc[g]);
                        acc[g] = fmaf(w[g][c].z, v.z, acc[g]);
                        acc[g] = fmaf(w[g][c].w, v.w, acc[g]);
                    }
                }
            }
            const int row = merged_butterfly<G>(acc, lane);
            constexpr int kOwners = 32 / G;
            if ((lane & (kOwners - 1)) == 0) rd[row][t][warp] = acc[0];
        }
        __syncthreads();
        {
            const int g = threadIdx.x / kTokTile, t = threadIdx.x % kTokTile;
            if (g < G && t < nt) {
                float s = 0.f;
#pragma unroll
                for (int i = 0; i < kLogitThreads / 32; ++i) s += rd[g][t][i];
                logits[(size_t) (t_begin + t0 + t) * n_expert + r0 + g] = s;
            }
        }
    }
    if (late_wait) pdl_wait();
}

constexpr size_t kStagedSmemMax = 96 * 1024;

// 1 when this launch may run beside the kernel ahead of it (pdl.cuh); only inside a scope whose launches are programmatic
inline int take_late_wait() {
    PdlState& ps = pdl_state();
    const bool late = ps.late_wait && ps.on && ps.plain == 0;
    ps.late_wait = false;
    return late ? 1 : 0;
}

template <int NV, int G, bool BF16>
int32_t launch_logits_staged(const void* x, const float* gate, int T, int E, int H, int tpb, float* logits, cudaStream_t st) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(router_logits_staged_kernel<NV, G, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) kStagedSmemMax);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    const size_t smem = (size_t) tpb * H * (BF16 ? 2 : 4);
    const dim3 grid((unsigned) (E / G), (unsigned) ((T + tpb - 1) / tpb));
    launch_k(router_logits_staged_kernel<NV, G, BF16>, grid, dim3(kLogitThreads), smem, st, x, gate, H, E, T, tpb, logits, take_late_wait());
    return launch_status();
}

// the staged kernel for the row widths decode layers have (NV float4 a thread and row: hidden up to 2048 with 8 rows a block, up to
// 4096 with 4); -1: not covered, the caller runs the plain kernel
template <bool BF16>
int32_t staged_dispatch(int nv, int G, const void* x, const float* gate, int T, int E, int H, int tpb, float* logits, cudaStream_t st) {
    if (nv == 1 && G == 8) return launch_logits_staged<1, 8, BF16>(x, gate, T, E, H, tpb, logits, st);
    if (nv == 2 && G == 8) return launch_logits_staged<2, 8, BF16>(x, gate, T, E, H, tpb, logits, st);
    if (nv == 1 && G == 4) return launch_logits_staged<1, 4, BF16>(x, gate, T, E, H, tpb, logits, st);
    if (nv == 2 && G == 4) return launch_logits_staged<2, 4, BF16>(x, gate, T, E, H, tpb, logits, st);
    if (nv == 3 && G == 4) return launch_logits_staged<3, 4, BF16>(x, gate, T, E, H, tpb, logits, st);
    if (nv == 4 && G == 4) return launch_logits_staged<4, 4, BF16>(x, gate, T, E, H, tpb, logits, st);
    return -1;
}

template <int NV, int G>
void launch_logits(const void* x, bool bf16, const float* gate, int T, int E, int H, float* logits, cudaStream_t st) {
    const int tpb = T <= 256 ? kTokTile : 8 * kTokTile;
    const dim3 grid((unsigned) (E / G), (unsigned) ((T + tpb - 1) / tpb));
    const int late = take_late_wait();
    if (bf16) launch_k(router_logits_kernel<NV, G, true>, grid, dim3(kLogitThreads), 0, st, x, gate, H, E, T, tpb, logits, late);
    else launch_k(router_logits_kernel<NV, G, false>, grid, dim3(kLogitThreads), 0, st, x, gate, H, E, T, tpb, logits, late);
}

template <int G>
bool dispatch_nv(int nv, const void* x, bool bf16, const float* gate, int T, int E, int H, float* logits, cudaStream_t st) {
    switch (nv) {
        case 1: launch_logits<1, G>(x, bf16, gate, T, E, H, logits, st); return true;
        case 2: launch_logits<2, G>(x, bf16, gate, T, E, H, logits, st); return true;
        case 3: if constexpr (G <= 4) { launch_logits<3, G>(x, bf16, gate, T, E, H, logits, st); return true; } return false;
        case 4: if constexpr (G <= 4) { launch_logits<4, G>(x, bf16, gate, T, E, H, logits, st); return true; } return false;
        case 5: if constexpr (G <= 2) { launch_logits<5, G>(x, bf16, gate, T, E, H, logits, st); return true; } return false;
        case 6: if constexpr (G <= 2) { launch_logits<6, G>(x, bf16, gate, T, E, H, logits, st); return true; } return false;
        case 7: if constexpr (G <= 2) { launch_logits<7, G>(x, bf16, gate, T, E, H, logits, st); return true; } return false;
        case 8: if constexpr (G <= 2) { launch_logits<8, G>(x, bf16, gate, T, E, H, logits, st); return true; } return false;
        default: return false;
    }
}

// ---------------------------------------------------------------------------------------------- sigmoid / sqrt-softplus select
struct HeldTabs {
    const int32_t* t[BSX_MAX_HELD_TABS];
    int n;
    __device__ bool held(int e) const {
        bool in = false;
        for (int q = 0; q < n; ++q) in |= t[q][e] >= 0;
        return in;
    }
};

// src/kernels/cuda/router.cu:148-153
__device__ __forceinline__ float gate_score(float x, int gate) {
    if (gate == BSX_GATE_SQRT_SOFTPLUS) {
        const float sp = x > 20.f ? x : logf(1.f + expf(x));
        return sqrtf(sp);
    }
    return 1.f / (1.f + expf(-x));
}

// One warp per token; lane l holds experts l, l+32, ...  The selection is the reference's rank rule (higher s + bias first,
// the lower index on a tie; src/kernels/cuda/router.cu:170-217) made as k warp-wide argmax passes, which yield the ids in rank
// order directly; lane 0 adds the chosen unbiased scores in that order, as the reference's thread 0 does.
template <int REGT>
__device__ __forceinline__ void select_token(const float* __restrict__ lg, const float* __restrict__ bias, int E, int k, float scale, int gate,
                                             int n_group, int topk_group, float prior, const HeldTabs& held, int32_t* __restrict__ ids,
                                             float* __restrict__ weights) {
    constexpr int MAXR = REGT > 0 ? REGT : 32;
    const int lane = threadIdx.x & 31;
    const int reg = REGT > 0 ? REGT : (E >> 5);
    float s[MAXR], b[MAXR];
    uint32_t dead = 0;   // bit i: expert lane + 32 i cannot be chosen (outside E, masked group, or already taken)
#pragma unroll
    for (int i = 0; i < MAXR; ++i) {
        if (i < reg) {
            const int e = lane + i * 32;
            s[i] = gate_score(lg[e], gate);
            b[i] = s[i] + (bias ? bias[e] : 0.f);
            if (prior > 0.f && held.n > 0 && held.held(e)) b[i] += prior;
        } else {
            s[i] = 0.f;
            b[i] = -INFINITY;
            dead |= 1u << i;
        }
    }
    if (n_group > 1 && topk_group < n_group) {
        const int gs = E / n_group;
        float my_score = -INFINITY;
        for (int g = 0; g < n_group; ++g) {
            float m1 = -INFINITY, m2 = -INFINITY;
#pragma unroll
            for (int i = 0; i < MAXR; ++i)
                if (i < reg && (lane + i * 32) / gs == g) {
                    const float v = b[i];
                    if (v > m1) { m2 = m1; m1 = v; }
                    else if (v > m2) m2 = v;
                }
#pragma unroll
            for (int o = 16; o; o >>= 1) {
                const float o1 = __shfl_xor_sync(kFull, m1, o), o2 = __shfl_xor_sync(kFull, m2, o);
                const float hi = fmaxf(m1, o1), lo = fminf(m1, o1);
                m2 = fmaxf(lo, fmaxf(m2, o2));
                m1 = hi;
            }
            const float sc = gs > 1 ? m1 + m2 : m1;
            if (lane == g) my_score = sc;
        }
        int rank = 0;
        for (int j = 0; j < n_group; ++j) {
            const float oj = __shfl_sync(kFull, my_score, j);
            rank += (oj > my_score) | ((oj == my_score) & (j < lane));
        }
        const unsigned live = __ballot_sync(kFull, lane < n_group && rank < topk_group);
#pragma unroll
        for (int i = 0; i < MAXR; ++i)
            if (i < reg && !((live >> ((lane + i * 32) / gs)) & 1u)) dead |= 1u << i;
    }
    float my_sel = 0.f, sum = 0.f;
    for (int r = 0; r < k; ++r) {
        // every index into s[] / b[] is a compile-time constant (a runtime index would move the arrays to local memory): the scan
        // carries the candidate's unbiased score along, and taken experts are remembered in the `dead` mask
        float best = -INFINITY, best_s = 0.f;
        int ex = INT_MAX;
#pragma unroll
        for (int i = 0; i < MAXR; ++i)
            if (!((dead >> i) & 1u) && (ex == INT_MAX || b[i] > best)) { best = b[i]; best_s = s[i]; ex = lane + i * 32; }
#pragma unroll
        for (int m = 16; m; m >>= 1) {
            const float ob = __shfl_xor_sync(kFull, best, m);
            const int oi = __shfl_xor_sync(kFull, ex, m);
            if (oi != INT_MAX && (ex == INT_MAX || ob > best || (ob == best && oi < ex))) { best = ob; ex = oi; }
        }
        float sv = 0.f;
        if (ex != INT_MAX && (ex & 31) == lane) {     // this lane's candidate won: ex is still its own (lane + 32 i)
            sv = best_s;
            dead |= 1u << (ex >> 5);
        }
        sv = __shfl_sync(kFull, sv, ex == INT_MAX ? 0 : (ex & 31));
        sum += sv;
        if (lane == r) my_sel = sv;
        if (lane == 0) ids[r] = ex == INT_MAX ? -1 : ex;
    }
    const float denom = sum + 1e-20f;
    if (lane < k) weights[lane] = my_sel / denom * scale;
}

template <int REGT>
__global__ void __launch_bounds__(256)
router_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int64_t T, int E, int k, float scale,
                     int gate, int n_group, int topk_group, float prior, HeldTabs held, int32_t* __restrict__ ids,
                     float* __restrict__ weights) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t t = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    select_token<REGT>(logits + t * E, bias, E, k, scale, gate, n_group, topk_group, prior, held, ids + t * k, weights + t * k);
}

// ---------------------------------------------------------------------------------------------- fp64 softmax router
// src/models/qwen4exp/kernels/router_top10.cu:57-174: p[e] = (float)(exp((double) l - (double) max) * (float)(1 / sum)) with the
// sum taken serially in ascending expert order in double; k argmax passes (value desc, index asc); weights renormalised
// in double over max(sum of the chosen, 2^-14).  One warp per token; the exponentials sit in shared memory for the serial sum.
__global__ void __launch_bounds__(128)
router_softmax_f64_kernel(const float* __restrict__ logits, int64_t T, int E, int k, int32_t* __restrict__ ids,
                          float* __restrict__ weights) {
    extern __shared__ double s_ex[];   // [warps][E]
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t) blockIdx.x * (blockDim.x >> 5) + wib;
    if (t >= T) return;
    double* ex = s_ex + (size_t) wib * E;
    const float* l = logits + t * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, l[e]);
    mx = warp_max_xor(mx);
    for (int e = lane; e < E; e += 32) ex[e] = exp((double) l[e] - (double) mx);
    __syncwarp();
    double sum = 0.0;
    if (lane == 0)
        for (int e = 0; e < E; ++e) sum += ex[e];
    sum = __shfl_sync(kFull, sum, 0);
    const float inv = (float) (1.0 / sum);
    float p[32];
    const int reg = E >> 5;
#pragma unroll
    for (int i = 0; i < 32; ++i) p[i] = i < reg ? (float) (ex[lane + i * 32] * inv) : -INFINITY;
    uint32_t taken = 0;
    float my_w = 0.f;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = E;
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < reg && !((taken >> i) & 1u) && p[i] > bv) { bv = p[i]; bi = lane + i * 32; }
#pragma unroll
        for (int m = 16; m; m >>= 1) {
            const float ov = __shfl_xor_sync(kFull, bv, m);
            const int oi = __shfl_xor_sync(kFull, bi, m);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi < E) {
            if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
            if (lane == 0) ids[t * k + r] = bi;
            if (lane == r) my_w = bv;
        }
    }
    double ws = 0.0;
    for (int r = 0; r < k; ++r) ws += (double) __shfl_sync(kFull, my_w, r);
    const double sc = fmax(ws, 6.103515625e-05);
    if (lane < k) weights[t * k + lane] = (float) ((double) my_w / sc);
}

// ---------------------------------------------------------------------------------------------- tail skip
// include/basalt/kernels/route_lossy.hpp:34-60, src/kernels/cuda/route_tail_skip.cu:14-39: one block, a thread per window entry.
__global__ void __launch_bounds__(BSX_TAIL_SKIP_MAX)
route_tail_skip_kernel(int32_t* __restrict__ ids, float* __restrict__ w, HeldTabs held, int n, int k, int R, int n_expert,
                       unsigned long long* counts) {
    __shared__ int32_t s_ids[BSX_TAIL_SKIP_MAX];
    __shared__ uint8_t s_tail[BSX_TAIL_SKIP_MAX];
    const int tid = threadIdx.x;
    bool miss = false;
    if (tid < n) {
        const int32_t e = ids[tid];
        s_ids[tid] = e;
        const float wi = w[tid];
        const int base = tid - tid % k;
        int rank = 0;
        for (int j = 0; j < k; ++j) {
            const float wj = w[base + j];
            rank += wj > wi || (wj == wi && base + j < tid);
        }
        s_tail[tid] = rank >= R;
        miss = e >= 0 && e < n_expert && !held.held(e);
    }
    __syncthreads();
    bool drop = tid < n && miss;
    if (drop)
        for (int j = 0; j < n; ++j)
            if (s_ids[j] == s_ids[tid] && !s_tail[j]) { drop = false; break; }
    const int n_miss = __syncthreads_count(miss), n_drop = __syncthreads_count(drop);
    if (drop) {
        ids[tid] = -1;
        w[tid] = 0.0f;
    }
    if (counts != nullptr && tid == 0) {
        atomicAdd(&counts[0], (unsigned long long) n);
        atomicAdd(&counts[1], (unsigned long long) n_miss);
        atomicAdd(&counts[2], (unsigned long long) n_drop);
    }
}


// ---------------------------------------------------------------------------------------------- selection + plan in one launch
// One block for a window of up to 16 tokens: a warp per token chooses its experts (the per-token routines above, so ids and
// weights carry the same bits as the separate kernels'), leaves the ids in shared memory with their blobs' addresses, and the
// block goes straight on to the window's plan from those pairs alone (plan_small, plan.cuh) - one launch and one round trip
// through global memory fewer in a step that is latency-bound, and nothing in it grows with the number of experts.
// With items / n_items the pass list of the packed expert kernels is written as well.
constexpr int kRoutePlanThreads = 512;     // 16 warps: the window's tokens; and one thread per pair of the plan (T k <= 512)

template <int REGT>
__global__ void __launch_bounds__(kRoutePlanThreads)
route_plan_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k, float scale, int gate, int n_group,
                  int topk_group, float prior, HeldTabs held, const unsigned long long* __restrict__ blobs, unsigned long long shared_blob,
                  int32_t* ids, float* weights, unsigned long long* __restrict__ ptr, int32_t* __restrict__ start,
                  int32_t* __restrict__ n_groups, int32_t* __restrict__ dst, int32_t* __restrict__ tok, PassRec* __restrict__ items,
                  int* __restrict__ n_items) {
    __shared__ int32_t s_sid[kRoutePlanThreads], s_lead[kRoutePlanThreads];
    __shared__ unsigned long long s_blob[kRoutePlanThreads];
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp < T) {
        const int t = warp;
        int32_t* it = ids + (size_t) t * k;
        float* wt = weights + (size_t) t * k;
        if (gate == BSX_GATE_SOFTMAX) softmax_topk_token<REGT>(logits + (size_t) t * E, it, wt, E, k);
        else select_token<REGT>(logits + (size_t) t * E, bias, E, k, scale, gate, n_group, topk_group, prior, held, it, wt);
        __syncwarp();                    // lane 0's ids are visible to the warp
        if (lane < k) {
            int e = it[lane];
            unsigned long long b = 0ull;
            if ((unsigned) e < (unsigned) E) b = blobs[e];
            if (!b) e = -1;              // out of range, or an expert this device does not hold: no entry
            s_sid[t * k + lane] = e;
            s_blob[t * k + lane] = b;
        }
    }
    __syncthreads();
    plan_small(s_sid, s_blob, s_lead, T * k, k, shared_blob, shared_blob != 0ull ? T : 0, ptr, start, n_groups, dst, tok, items, n_items);
}

bool make_held(const int32_t* const* tabs, int n, HeldTabs& h) {
    h.n = 0;
    for (int i = 0; i < BSX_MAX_HELD_TABS; ++i) h.t[i] = nullptr;
    if (n < 0 || n > BSX_MAX_HELD_TABS || (n > 0 && !tabs)) return false;
    for (int i = 0; i < n; ++i)
        if (tabs[i]) h.t[h.n++] = tabs[i];
    return true;
}

}  // namespace
}  // namespace bsx

using namespace bsx;

// launches the logits kernel (no synchronisation); x is fp32 or bf16 rows
static int32_t logits_launch(const void* x, int32_t x_kind, const float* gate, int32_t T, int32_t E, int32_t H, float* logits, cudaStream_t st) {
    if (E < 32 || E % 32 || H < 128 || H % 128 || H > 8192 || T < 0) return BSX_E_GEOMETRY;
    if (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16) return BSX_E_GEOMETRY;
    if (T == 0) return BSX_OK;
    if (!aligned(x, 16) || !aligned(gate, 16) || !aligned(logits, 4)) return BSX_E_POINTER;
    const bool bf16 = x_kind == BSX_X_BF16;
    const int nv = (H / 4 + kLogitThreads - 1) / kLogitThreads;
    // decode windows of 16+ tokens whose rows fit shared memory: the staged kernel, one wave of blocks
    const size_t row_bytes = (size_t) H * (bf16 ? 2 : 4);
    if (T >= 16 && T <= 1024 && nv <= 4 && 8 * row_bytes <= kStagedSmemMax) {
        int tpb = (int) (kStagedSmemMax / row_bytes) & ~7;
        tpb = tpb > 16 ? 16 : tpb;      // 16 tokens (64 KB of bf16 rows at hidden 2048): two or three blocks share an SM
        if (tpb > ((T + 7) & ~7)) tpb = (T + 7) & ~7;
        const int tiles = (T + tpb - 1) / tpb;
        int Gs = nv <= 2 ? 8 : 4;
        while (Gs > 4 && (E / Gs) * tiles < 96) Gs >>= 1;
        if (E % Gs == 0) {
            const int32_t rc = bf16 ? staged_dispatch<true>(nv, Gs, x, gate, T, E, H, tpb, logits, st) : staged_dispatch<false>(nv, Gs, x, gate, T, E, H, tpb, logits, st);
            if (rc != -1) return rc;
        }
    }
    // the most gate rows a block whose registers fit and whose grid still covers the SMs twice
    int G = nv <= 2 ? 8 : nv <= 4 ? 4 : 2;
    const int tiles = (T + kTokTile - 1) / kTokTile;
    while (G > 2 && (int64_t) (E / G) * tiles < 2 * (int64_t) sm_count()) G >>= 1;
    bool ok = false;
    if (G == 8) ok = dispatch_nv<8>(nv, x, bf16, gate, T, E, H, logits, st);
    else if (G == 4) ok = dispatch_nv<4>(nv, x, bf16, gate, T, E, H, logits, st);
    else ok = dispatch_nv<2>(nv, x, bf16, gate, T, E, H, logits, st);
    return ok ? launch_status() : BSX_E_GEOMETRY;
}

static int32_t sync_if_null(int32_t rc, void* stream) {
    if (rc == BSX_OK && !stream) {
        const cudaError_t e = cudaStreamSynchronize(nullptr);
        if (e != cudaSuccess) return (int32_t) e;
    }
    return rc;
}

extern "C" int32_t bsx_router_logits(const float* x, const float* gate, int32_t T, int32_t E, int32_t H, float* logits, void* stream) {
    return sync_if_null(logits_launch(x, BSX_X_F32, gate, T, E, H, logits, (cudaStream_t) stream), stream);
}

extern "C" int32_t bsx_router_logits_x(const void* x, int32_t x_kind, const float* gate, int32_t T, int32_t E, int32_t H, float* logits,
                                       void* stream) {
    return sync_if_null(logits_launch(x, x_kind, gate, T, E, H, logits, (cudaStream_t) stream), stream);
}

extern "C" int32_t bsx_router_select(const float* logits, const float* bias, int32_t T, int32_t E, int32_t k, int32_t gate_kind,
                                     float weight_scale, int32_t n_group, int32_t topk_group, float prior,
                                     const int32_t* const* held_tabs, int32_t n_held, int32_t* ids, float* weights, void* stream) {
    if (E < 32 || E % 32 || E > 1024 || k < 1 || k > 32 || k > E || T < 0) return BSX_E_GEOMETRY;
    if (T == 0) return BSX_OK;
    if (!logits || !ids || !weights) return BSX_E_POINTER;
    const cudaStream_t st = (cudaStream_t) stream;
    int32_t rc;
    if (gate_kind == BSX_GATE_SOFTMAX) {
        rc = softmax_topk_launch(logits, T, E, k, ids, weights, st);
    } else if (gate_kind == BSX_GATE_SOFTMAX_FAST) {
        rc = softmax_fast(logits, T, E, k, ids, weights, st);
    } else if (gate_kind == BSX_GATE_SOFTMAX_F64) {
        const size_t smem = (size_t) 4 * E * sizeof(double);
        router_softmax_f64_kernel<<<(unsigned) ((T + 3) / 4), 128, smem, st>>>(logits, T, E, k, ids, weights);
        rc = launch_status();
    } else if (gate_kind == BSX_GATE_SIGMOID || gate_kind == BSX_GATE_SQRT_SOFTPLUS) {
        if (k > 16) return BSX_E_GEOMETRY;
        if (n_group < 1) n_group = 1;
        if (n_group > 32 || E % n_group) return BSX_E_GEOMETRY;
        if (topk_group < 1 || topk_group > n_group) topk_group = n_group;
        if ((int64_t) topk_group * (E / n_group) < k) return BSX_E_GEOMETRY;
        HeldTabs held;
        if (!make_held(held_tabs, n_held, held)) return BSX_E_POINTER;
        // decode windows: two tokens a block, so the window's selections spread over the SMs instead of queueing on a few
        const unsigned wpb = T <= 256 ? 2u : 8u, blocks = (unsigned) ((T + wpb - 1) / wpb);
#define BSX_SEL(R) launch_k(router_select_kernel<R>, dim3(blocks), dim3(32 * wpb), 0, st, logits, bias, (int64_t) T, E, k, weight_scale, gate_kind, n_group, topk_group, prior, held, ids, weights)
        switch (E >> 5) {
            case 2: BSX_SEL(2); break;
            case 4: BSX_SEL(4); break;
            case 8: BSX_SEL(8); break;
            case 12: BSX_SEL(12); break;
            case 16: BSX_SEL(16); break;
            default: BSX_SEL(0); break;
        }
#undef BSX_SEL
        rc = launch_status();
    } else {
        return BSX_E_GEOMETRY;
    }
    if (rc == BSX_OK && !stream) {
        const cudaError_t e = cudaStreamSynchronize(nullptr);
        if (e != cudaSuccess) return (int32_t) e;
    }
    return rc;
}

extern "C" int32_t bsx_router_x(const void* x, int32_t x_kind, const float* gate, const float* bias, int32_t T, int32_t E, int32_t H,
                                int32_t k, int32_t gate_kind, float weight_scale, int32_t n_group, int32_t topk_group, float prior,
                                const int32_t* const* held_tabs, int32_t n_held, float* logits, int32_t* ids, float* weights,
                                void* stream) {
    // the limits of the reference's router() (src/kernels/cuda/router.cu:235), E widened to 1024
    if (E < 32 || E % 32 || E > 1024 || k < 1 || k > E || k > 32) return BSX_E_GEOMETRY;
    if ((gate_kind == BSX_GATE_SIGMOID || gate_kind == BSX_GATE_SQRT_SOFTPLUS) && k > 16) return BSX_E_GEOMETRY;
    const int32_t rc = logits_launch(x, x_kind, gate, T, E, H, logits, (cudaStream_t) stream);   // same stream, no sync in between
    if (rc != BSX_OK || T == 0) return rc;
    return bsx_router_select(logits, bias, T, E, k, gate_kind, weight_scale, n_group, topk_group, prior, held_tabs, n_held, ids,
                             weights, stream);
}

extern "C" int32_t bsx_router(const float* x, const float* gate, const float* bias, int32_t T, int32_t E, int32_t H, int32_t k,
                              int32_t gate_kind, float weight_scale, int32_t n_group, int32_t topk_group, float prior,
                              const int32_t* const* held_tabs, int32_t n_held, float* logits, int32_t* ids, float* weights,
                              void* stream) {
    return bsx_router_x(x, BSX_X_F32, gate, bias, T, E, H, k, gate_kind, weight_scale, n_group, topk_group, prior, held_tabs, n_held,
                        logits, ids, weights, stream);
}

extern "C" int32_t bsx_route_tail_skip(int32_t* ids, float* weights, const int32_t* const* held_tabs, int32_t n_held,
                                       int32_t n_entries, int32_t k, int32_t rank, int32_t E, unsigned long long* counts,
                                       void* stream) {
    // the reference returns silently outside these bounds (src/kernels/cuda/route_tail_skip.cu:45)
    if (rank < 1 || rank >= k || n_entries < 1 || n_entries > BSX_TAIL_SKIP_MAX || k < 1) return BSX_OK;
    if (!ids || !weights) return BSX_E_POINTER;
    HeldTabs held;
    if (!make_held(held_tabs, n_held, held)) return BSX_E_POINTER;
    route_tail_skip_kernel<<<1, BSX_TAIL_SKIP_MAX, 0, (cudaStream_t) stream>>>(ids, weights, held, n_entries, k, rank, E, counts);
    return launch_status();
}

namespace bsx {
int32_t moe_plan_with_passes(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table, unsigned long long shared_blob,
                             unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok, PassRec* items, int* n_items,
                             cudaStream_t st);

constexpr int kRoutePlanMaxTokens = 16;

// selection + plan (+ the packed kernels' pass list when items is given); BSX_E_TYPE: a gate kind the fused kernel does not cover
int32_t route_plan_launch(const float* logits, const float* bias, int32_t T, int32_t E, int32_t k, int32_t gate_kind, float weight_scale,
                          int32_t n_group, int32_t topk_group, const unsigned long long* blob_table, unsigned long long shared_blob, int32_t* ids,
                          float* weights, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok, PassRec* items,
                          int* n_items, cudaStream_t st) {
    if (gate_kind != BSX_GATE_SOFTMAX && gate_kind != BSX_GATE_SIGMOID && gate_kind != BSX_GATE_SQRT_SOFTPLUS) return BSX_E_TYPE;
    if (E < 32 || E % 32 || E > 1024 || k < 1 || k > 32 || k > E || T < 0) return BSX_E_GEOMETRY;
    if ((int64_t) T * k > BSX_PLAN_MAX_PAIRS) return BSX_E_LIMIT;
    if (T == 0) return BSX_OK;
    if (!logits || !ids || !weights || !blob_table || !ptr || !start || !n_groups || !dst || !tok) return BSX_E_POINTER;
    HeldTabs held;
    make_held(nullptr, 0, held);
    if (gate_kind != BSX_GATE_SOFTMAX) {
        if (k > 16) return BSX_E_GEOMETRY;
        if (n_group < 1) n_group = 1;
        if (n_group > 32 || E % n_group) return BSX_E_GEOMETRY;
        if (topk_group < 1 || topk_group > n_group) topk_group = n_group;
        if ((int64_t) topk_group * (E / n_group) < k) return BSX_E_GEOMETRY;
    }
    if (T > kRoutePlanMaxTokens) {
        // The fused kernel is one block on one SM, and a token's selection is ~2500 warp instructions: with 32 warps at it the SM's
        // four schedulers are the limit (measured: 64 tokens in the one block 31 us, against 16.5 us for selection spread over
        // blocks followed by the plan kernel).  Wider windows keep the selection spread over blocks and fuse only plan + pass list.
        const int32_t rc = bsx_router_select(logits, bias, T, E, k, gate_kind, weight_scale, n_group, topk_group, 0.f, nullptr, 0, ids, weights, (void*) st);
        if (rc != BSX_OK) return rc;
        return moe_plan_with_passes(ids, T, k, E, blob_table, shared_blob, ptr, start, n_groups, dst, tok, items, n_items, st);
    }
    static_assert(kRoutePlanMaxTokens * 32 <= kRoutePlanThreads, "a warp per token, a thread per pair");
#define BSX_RP(R) launch_k(route_plan_kernel<R>, dim3(1), dim3(kRoutePlanThreads), 0, st, logits, bias, (int) T, (int) E, (int) k, weight_scale, (int) gate_kind, (int) n_group, \
                           (int) topk_group, 0.f, held, blob_table, shared_blob, ids, weights, ptr, start, n_groups, dst, tok, items, n_items)
    switch (E >> 5) {
        case 2: BSX_RP(2); break;
        case 4: BSX_RP(4); break;
        case 8: BSX_RP(8); break;
        case 16: BSX_RP(16); break;
        default: BSX_RP(0); break;
    }
#undef BSX_RP
    return launch_status();
}
}  // namespace bsx

extern "C" int32_t bsx_route_plan(const float* logits, const float* bias, int32_t T, int32_t E, int32_t k, int32_t gate_kind, float weight_scale,
                                  int32_t n_group, int32_t topk_group, const unsigned long long* blob_table, unsigned long long shared_blob,
                                  int32_t* ids, float* weights, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok,
                                  void* stream) {
    if (!stream) return BSX_E_STREAM;
    return route_plan_launch(logits, bias, T, E, k, gate_kind, weight_scale, n_group, topk_group, blob_table, shared_blob, ids, weights, ptr, start,
                             n_groups, dst, tok, nullptr, nullptr, (cudaStream_t) stream);
}
