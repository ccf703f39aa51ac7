// router_prefill.cu - the router's gate product for prompt-sized batches on the tcgen05 tensor cores.
//
// logits[t][e] = sum_k x[t][k] gate[e][k] for thousands of tokens is a GEMM; the fixed-order fp32 chain of router.cu, which
// the decode path needs for bit-exact routing, re-reads the gate matrix once per 8 tokens and takes milliseconds there.
// Basalt's prompt path does the same switch: its router product is a bf16 GEMM (src/models/qwen4exp/prefill/routing.cpp:26),
// selection then runs on those logits.  Here both operands become fp16 images scaled per row by a power of two - a bf16
// activation row converts exactly, an fp32 row as hi + lo terms, the fp32 gate matrix always as hi + lo (22 significant
// bits) - and kind::f16 MMAs accumulate the (x term, gate term) products in fp32 in tensor memory, so the logits sit ~1e-6
// (relative to |x| |gate|) from the fp32 chain's, far inside what the bf16 GEMM of the reference gives.  Selection
// (bsx_router_select) is unchanged and reads these logits; ids can differ from the decode path's only where two scores tie
// to that precision.
//
// One CTA per (128 tokens, 256 experts) tile: warp 0 allocates 256 TMEM columns and its lane 0 issues the MMAs; warp 1
// loads activation rows, warps 2-3 gate rows (cp.async into 128-byte-swizzled stages, 4-stage mbarrier ring, every wait
// time-bounded); warps 4-7 are the epilogue (thread = TMEM lane = token).
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "tc5.cuh"

namespace bsx {
namespace {

constexpr int kTM = 128, kTN = 256, kBK = 64, kStg = 4;
constexpr int kThreadsR = 256;
constexpr int kABytesR = kTM * kBK * 2, kBBytesR = kTN * kBK * 2, kStageR = kABytesR + kBBytesR;
constexpr size_t kSmemR = 1024 + (size_t) kStg * kStageR + 128 + kTN * 4 + 64;
constexpr uint32_t kIdescR = instr_desc_f16(kTM, kTN);

size_t al256(size_t v) { return (v + 255) & ~(size_t) 255; }

// rows [R][H] (fp32 or bf16) -> `terms` fp16 planes [terms][R][H], each row scaled by a power of two so its largest magnitude
// lands in [2^13, 2^14), k-permuted inside 16-column groups; inv[r] undoes the scale.  Plane 1 holds the rounding residual
// of plane 0.  One warp per row.
__global__ void __launch_bounds__(256) rows_to_fp16_planes_kernel(const void* __restrict__ x, int kind, int64_t R, int64_t H, int terms,
                                                                  __half* __restrict__ img, float* __restrict__ inv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r = (int64_t) blockIdx.x * 8 + warp;
    if (r >= R) return;
    auto ld = [&](int64_t c) {
        return kind == BSX_X_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(x)[r * H + c]) : static_cast<const float*>(x)[r * H + c];
    };
    float amax = 0.f;
    for (int64_t c = lane; c < H; c += 32) amax = fmaxf(amax, fabsf(ld(c)));
    amax = warp_max_xor(amax);
    int ex = 0;
    float s = 1.f, iv = 1.f;
    if (amax > 0.f && amax <= 3.0e38f) {
        frexpf(amax, &ex);
        ex = max(-100, min(100, 14 - ex));
        s = ldexpf(1.f, ex);
        iv = ldexpf(1.f, -ex);
    }
    if (lane == 0) inv[r] = iv;
    for (int64_t c = lane; c < H; c += 32) {
        const float v = ld(c) * s;
        const __half hi = __float2half_rn(v);
        const int64_t o = r * H + (c & ~(int64_t) 15) + perm16((int) (c & 15));
        img[o] = hi;
        if (terms > 1) img[R * H + o] = __float2half_rn(v - __half2float(hi));
    }
}

struct LogitsArgs {
    const __half* ximg;   // [x_terms][T][H]
    const float* xinv;    // [T]
    const __half* gimg;   // [2][E][H]
    const float* ginv;    // [E]
    float* logits;        // [T][E]
    int32_t* status;
    int64_t T;
    int E, H, x_terms;
};

__global__ void __launch_bounds__(kThreadsR, 1) router_logits_tc_kernel(LogitsArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStg * kStageR);
    uint64_t* empty = full + kStg;
    uint64_t* accum = empty + kStg;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);
    float* s_ginv = reinterpret_cast<float*>(smem + kStg * kStageR + 128);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = blockIdx.x * kTN;
    const int64_t t0 = (int64_t) blockIdx.y * kTM;
    const int nkb = a.H / kBK;
    // the products summed into the accumulator: (x hi, gate hi), (x hi, gate lo) and, for two x terms, (x lo, gate hi)
    const int n_prod = a.x_terms > 1 ? 3 : 2;
    const int n_it = n_prod * nkb;

    for (int i = threadIdx.x; i < kTN; i += kThreadsR) s_ginv[i] = a.ginv[min(e0 + i, a.E - 1)];
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStg; ++s) {
            mbar_init(&full[s], 96);      // three loader warps
            mbar_init(&empty[s], 1);
        }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t) kTN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < n_it; ++it) {
                const uint32_t s = (uint32_t) it % kStg;
                ok = mbar_wait(&full[s], ((uint32_t) it / kStg) & 1u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t sa = smem_u32(smem + s * kStageR), sb = sa + kABytesR;
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) umma_f16(tmem, smem_desc_sw128(sa + k * 32), smem_desc_sw128(sb + k * 32), kIdescR, (it | k) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            umma_commit(accum);
            if (!ok) atomicOr(a.status, 1);
        }
    } else if (warp <= 3) {
        // ---- loaders: warp 1 the 128 token rows, warps 2 and 3 128 expert rows each.  Lane l copies 16-byte chunk l % 8 of
        // rows l / 8 + 4 i.  Rows past the end of the matrix read its last row (their results are never stored).
        const int c = lane & 7, r4 = lane >> 3;
        const bool is_x = warp == 1;
        const int64_t n_rows = is_x ? a.T : (int64_t) a.E;
        const int64_t first = is_x ? t0 : (int64_t) e0 + (warp - 2) * 128;
        const uint32_t tile_off = is_x ? 0u : (uint32_t) (kABytesR + (warp - 2) * 16 * 1024);
        const size_t plane = (size_t) n_rows * a.H * 2;          // bytes of one term's image
        const uint8_t* base = reinterpret_cast<const uint8_t*>(is_x ? a.ximg : a.gimg);
        uint32_t roff[32];   // row starts in 16-byte units
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int64_t r = first + 4 * i + r4;
            roff[i] = (uint32_t) ((r < n_rows ? r : n_rows - 1) * (a.H >> 3)) + (uint32_t) c;
        }
        uint32_t dsto[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r7 = 4 * h + r4;
            dsto[h] = tile_off + (uint32_t) (r7 * 128 + ((c ^ r7) << 4));
        }
        uint32_t issued = 0, arrived = 0;
        for (int it = 0; it < n_it; ++it) {
            const int prod = it / nkb, kb = it - prod * nkb;
            const int term = is_x ? (prod == 2 ? 1 : 0) : (prod == 1 ? 1 : 0);
            const uint32_t s = issued % kStg;
            ok = mbar_wait(&empty[s], ((issued / kStg) & 1u) ^ 1u);
            if (!ok) break;
            const uint32_t dst = smem_u32(smem + s * kStageR);
            const uint8_t* src = base + (size_t) term * plane + (size_t) kb * 128;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + (uint32_t) ((i >> 1) * 1024) + dsto[i & 1]),
                             "l"(src + (size_t) roff[i] * 16)
                             : "memory");
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            ++issued;
            if (issued - arrived > 2) {
                asm volatile("cp.async.wait_group 2;\n" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                mbar_arrive(&full[arrived % kStg]);
                ++arrived;
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (; arrived < issued; ++arrived) mbar_arrive(&full[arrived % kStg]);
        if (!ok) atomicOr(a.status, 1);
    } else {
        // ---- epilogue: thread p = token t0 + p reads TMEM lane p; logits = sum * (1 / x scale) * (1 / gate row scale)
        const int p = (warp & 3) * 32 + lane;
        ok = __all_sync(kFull, mbar_wait(accum, 0u));
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (ok) {
            const bool live = t0 + p < a.T;
            const float xi = live ? a.xinv[t0 + p] : 0.f;
            float* out = a.logits + (size_t) (t0 + p) * a.E + e0;
            const uint32_t tbase = tmem + ((uint32_t) ((warp & 3) * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < kTN; c0 += 32) {
                uint32_t d[32];
                tmem_ld32(tbase + (uint32_t) c0, d);
                if (live && e0 + c0 < a.E) {
#pragma unroll
                    for (int v = 0; v < 8; ++v)
                        reinterpret_cast<float4*>(out + c0)[v] =
                            make_float4(__uint_as_float(d[4 * v]) * xi * s_ginv[c0 + 4 * v], __uint_as_float(d[4 * v + 1]) * xi * s_ginv[c0 + 4 * v + 1],
                                        __uint_as_float(d[4 * v + 2]) * xi * s_ginv[c0 + 4 * v + 2], __uint_as_float(d[4 * v + 3]) * xi * s_ginv[c0 + 4 * v + 3]);
                }
            }
        } else if (lane == 0) {
            atomicOr(a.status, 1);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((uint32_t) kTN) : "memory");
    }
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_router_logits_prefill_scratch_bytes(int64_t T, int32_t E, int32_t H) {
    if (T < 0 || E <= 0 || H <= 0) return 0;
    return al256((size_t) 2 * T * H * 2) + al256((size_t) T * 4) + al256((size_t) 2 * E * H * 2) + al256((size_t) E * 4);
}

extern "C" int32_t bsx_router_logits_prefill(const void* x, int32_t x_kind, const float* gate, int64_t T, int32_t E, int32_t H, float* logits,
                                             void* scratch, int32_t* status, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!aligned(x, 16) || !aligned(gate, 16) || !aligned(logits, 16) || !aligned(scratch, 256) || !status) return BSX_E_POINTER;
    if (T < 0 || E <= 0 || E % 32 || H <= 0 || H % 64 || (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16)) return BSX_E_GEOMETRY;
    if ((T + kTM - 1) / kTM > 65535) return BSX_E_LIMIT;
    if (T == 0) return BSX_OK;
    const cudaStream_t st = (cudaStream_t) stream;
    uint8_t* p = static_cast<uint8_t*>(scratch);
    LogitsArgs a;
    __half* ximg = reinterpret_cast<__half*>(p);
    p += al256((size_t) 2 * T * H * 2);
    float* xinv = reinterpret_cast<float*>(p);
    p += al256((size_t) T * 4);
    __half* gimg = reinterpret_cast<__half*>(p);
    p += al256((size_t) 2 * E * H * 2);
    float* ginv = reinterpret_cast<float*>(p);
    a.ximg = ximg;
    a.xinv = xinv;
    a.gimg = gimg;
    a.ginv = ginv;
    a.logits = logits;
    a.status = status;
    a.T = T;
    a.E = E;
    a.H = H;
    a.x_terms = x_kind == BSX_X_BF16 ? 1 : 2;
    static std::atomic<bool> configured[64];   // per device; threads of different devices call concurrently
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(router_logits_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) kSmemR);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    rows_to_fp16_planes_kernel<<<(unsigned) ((T + 7) / 8), 256, 0, st>>>(x, x_kind, T, H, a.x_terms, ximg, xinv);
    rows_to_fp16_planes_kernel<<<(unsigned) ((E + 7) / 8), 256, 0, st>>>(gate, BSX_X_F32, E, H, 2, gimg, ginv);
    const dim3 grid((unsigned) ((E + kTN - 1) / kTN), (unsigned) ((T + kTM - 1) / kTM));
    router_logits_tc_kernel<<<grid, kThreadsR, kSmemR, st>>>(a);
    return launch_status();
}
