// experts.cu - entry points of the expert stage: blob geometry, q8_1 activation rows, the grouped decode experts and the
// weighted combine.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"
#include "pdl.cuh"

namespace bsx {
namespace {

// every codebook in one table: the IQ1 points, then the IQ2 and IQ3 points (offsets kGrid* of formats.cuh)
__device__ const uint16_t g_iq1_grid[kGridWords] = {
#include "iq1_grid_u16.inc"
#include "iq_grids_u16.inc"
};
const uint16_t h_iq1_grid[kGridWords] = {
#include "iq1_grid_u16.inc"
#include "iq_grids_u16.inc"
};

}  // namespace

const uint16_t* iq1_device_grid() {
    static std::atomic<const uint16_t*> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    const uint16_t* g = cached[dev].load(std::memory_order_acquire);
    if (!g) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_iq1_grid) != cudaSuccess) return nullptr;
        g = static_cast<const uint16_t*>(p);
        cached[dev].store(g, std::memory_order_release);
    }
    return g;
}

namespace {

// src/kernels/cuda/iq_kernels.cu:2471-2503 with include/basalt/kernels/q8_1_finite.hpp:17-31: a warp per 32 values
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, int64_t n) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;   // n % 32 == 0: whole warps leave together
    const float xi = x[i];
    float amax = fabsf(xi), sum = xi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, o));
        sum += __shfl_xor_sync(kFull, sum, o);
    }
    float d = amax / 127.0f;
    if (fabsf(d) > 65504.0f) d = copysignf(65504.0f, d);
    float q = 0.0f;
    if (amax != 0.0f) {
        q = roundf(xi / d);
        q = q > 127.0f ? 127.0f : q < -127.0f ? -127.0f : q;
    }
    uint8_t* blk = y + (i / 32) * 36;
    blk[4 + (i & 31)] = (uint8_t) (int8_t) q;
    if ((i & 31) == 0) {
        if (fabsf(sum) > 65504.0f) sum = copysignf(65504.0f, sum);
        reinterpret_cast<__half2*>(blk)[0] = __halves2half2(__float2half(d), __float2half(sum));
    }
}

// y[t] = fma chain over the k rows in order, then the shared expert: src/models/qwen4exp/kernels/native_moe.cu:36-50 and
// src/models/qwen4exp/prefill/kernels.cu:438-449 (bit-equal forms).  A thread owns 4 consecutive columns.
__global__ void __launch_bounds__(128)
combine_kernel(const float* __restrict__ rows, const int32_t* __restrict__ slot, const float* __restrict__ w,
               const float* __restrict__ shared, const float* __restrict__ sg, const float* __restrict__ resid, int k, int H, int pair0,
               const int32_t* __restrict__ ids, int e_lo, int e_hi, float* __restrict__ y, int blk_tok, int blk_stride, int sh_lo, int sh_n,
               const uint8_t* __restrict__ replicated) {
    __shared__ int s_row[64];
    __shared__ float s_w[64];
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.y;
    if (threadIdx.x < k) {
        int r = slot ? slot[(size_t) t * k + threadIdx.x] : pair0 + t * k + (int) threadIdx.x;
        // ids and weights may lie in per-rank blocks of blk_tok tokens, blk_stride values apart (an all-gather's layout)
        const size_t at = blk_tok > 0 ? (size_t) (t / blk_tok) * blk_stride + (size_t) (t % blk_tok) * k + threadIdx.x : (size_t) t * k + threadIdx.x;
        if (ids) {   // expert-parallel partial sum: only the pairs whose expert lies in [e_lo, e_hi)
            const int e = ids[at];
            // a replicated (hot) expert's pair belongs to the rank that owns the token (tokens sh_lo .. sh_lo + sh_n - 1 here)
            const bool rep = replicated != nullptr && e >= 0 && replicated[e] != 0;
            if (rep ? !(t >= sh_lo && t < sh_lo + sh_n) : (e < e_lo || e >= e_hi)) r = -1;
        }
        s_row[threadIdx.x] = r;
        s_w[threadIdx.x] = w[at];
    }
    __syncthreads();
    const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c4 * 4 >= H) return;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j0 = 0; j0 < k; j0 += 4) {
        // four row reads in flight, then their fused multiply-adds in j order
        float4 p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u;
            p[u] = (j < k && s_row[j] >= 0) ? reinterpret_cast<const float4*>(rows + (size_t) s_row[j] * H)[c4] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = j0 + u;
            if (j < k && s_row[j] >= 0) {
                const float wj = s_w[j];
                s.x = fmaf(wj, p[u].x, s.x);
                s.y = fmaf(wj, p[u].y, s.y);
                s.z = fmaf(wj, p[u].z, s.z);
                s.w = fmaf(wj, p[u].w, s.w);
            }
        }
    }
    if (shared && (sh_n <= 0 || (t >= sh_lo && t < sh_lo + sh_n))) {   // sh_n > 0: shared rows exist for tokens sh_lo .. sh_lo + sh_n - 1 only
        const float4 p = reinterpret_cast<const float4*>(shared + (size_t) (sh_n > 0 ? t - sh_lo : t) * H)[c4];
        if (sg) {
            const float gate = 1.0f / (1.0f + expf(-sg[t]));
            s.x = fmaf(p.x, gate, s.x);
            s.y = fmaf(p.y, gate, s.y);
            s.z = fmaf(p.z, gate, s.z);
            s.w = fmaf(p.w, gate, s.w);
        } else {
            s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
        }
    }
    if (resid) {   // the step after the layer: the residual stream's row, one more rounded add
        const float4 r = reinterpret_cast<const float4*>(resid + (size_t) t * H)[c4];
        s.x += r.x; s.y += r.y; s.z += r.z; s.w += r.w;
    }
    reinterpret_cast<float4*>(y + (size_t) t * H)[c4] = s;
}

// the one-group plan of a dense gated MLP (a shared expert): Basalt's gated_mlp_plan_kernel, src/kernels/cuda/iq_kernels.cu:3414-3426
__global__ void __launch_bounds__(128)
gated_mlp_plan_kernel(unsigned long long blob, int n_tok, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* idx) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        ptr[0] = blob;
        start[0] = 0;
        start[1] = n_tok;
        start[2] = n_tok;
        *n_groups = 1;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_tok; i += gridDim.x * blockDim.x) idx[i] = i;
}

// out[r] = x[src[r]]: the rows of a dispatch in expert order (the prompt path's gather_rows16, src/models/qwen4exp/prefill/kernels.cu:
// 430-437), 16 bytes a thread
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ src, uint4* __restrict__ out, int64_t n_rows, int64_t per) {
    const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * per) return;
    const int64_t r = i / per, j = i - r * per;
    const int32_t s = src[r];
    out[i] = s >= 0 ? x[(int64_t) s * per + j] : make_uint4(0u, 0u, 0u, 0u);
}

size_t gated_plan_bytes(int64_t cap_tok) { return ((size_t) (64 + cap_tok * 4) + 255) & ~(size_t) 255; }

size_t row_bytes(int type, int64_t n) {
    if (!type_supported(type) || n <= 0 || n % block_values(type)) return 0;
    return (size_t) (n / block_values(type)) * (size_t) block_bytes(type);
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_row_bytes(int32_t type, int64_t n) { return row_bytes(type, n); }
extern "C" const char* bsx_version(void) { return "basalt_b200 0.1 (sm_100a)"; }

extern "C" int32_t bsx_host_decode_row(int32_t type, const void* row, float* y, int64_t n) {
    if (!row_bytes(type, n) || !row || !y) return BSX_E_TYPE;
    const uint8_t* b = static_cast<const uint8_t*>(row);
    for (int64_t u = 0; u < n / 32; ++u) decode_any_32(type, b, (int) u, h_iq1_grid, y + u * 32);
    return BSX_OK;
}

extern "C" int32_t bsx_expert_supported(int32_t gu_type, int32_t d_type, int32_t up_type, int64_t n_embd, int64_t n_ff) {
    if (up_type < 0) up_type = gu_type;
    if (!type_supported(gu_type) || !type_supported(d_type) || !type_supported(up_type)) return 0;
    // NVFP4 tail scales belong to an all-NVFP4 gate/up pair (src/kernels/cuda/iq_kernels.cu:3236)
    if ((gu_type == kTypeNVFP4) != (up_type == kTypeNVFP4)) return 0;
    if (n_embd <= 0 || n_ff <= 0 || n_embd % 256 || n_embd > 16384 || n_ff > 16384) return 0;
    if (!row_bytes(gu_type, n_embd) || !row_bytes(up_type, n_embd) || !row_bytes(d_type, n_ff)) return 0;
    return 1;
}

extern "C" int32_t bsx_expert_layout_init(int32_t gu_type, int32_t d_type, int32_t up_type, int64_t n_embd, int64_t n_ff,
                                          float swiglu_limit, float gate_softcap, float up_softcap, bsx_expert_layout* L) {
    if (!L) return BSX_E_POINTER;
    if (up_type < 0) up_type = gu_type;
    if (!bsx_expert_supported(gu_type, d_type, up_type, n_embd, n_ff)) return BSX_E_TYPE;
    memset(L, 0, sizeof *L);
    L->gu_type = gu_type;
    L->d_type = d_type;
    L->up_type = up_type;
    L->n_embd = n_embd;
    L->n_ff = n_ff;
    L->gu_row = row_bytes(gu_type, n_embd);
    L->up_row = row_bytes(up_type, n_embd);
    L->d_row = row_bytes(d_type, n_ff);
    L->up_off = (uint64_t) n_ff * L->gu_row;
    L->down_off = L->up_off + (uint64_t) n_ff * L->up_row;
    L->bytes = L->down_off + (uint64_t) n_embd * L->d_row + (gu_type == kTypeNVFP4 ? 16 : 0);
    L->swiglu_limit = swiglu_limit;
    L->gate_softcap = gate_softcap;
    L->up_softcap = up_softcap;
    return BSX_OK;
}

extern "C" size_t bsx_expert_scratch_bytes(const bsx_expert_layout* L, int64_t cap_entries) {
    if (!L || cap_entries < 0 || L->n_ff <= 0 || L->n_embd <= 0) return 0;
    const size_t f = (((size_t) cap_entries * (size_t) L->n_ff * sizeof(float)) + 255) & ~(size_t) 255;
    const size_t m = experts_mma_scratch_bytes(cap_entries, L->n_embd, L->n_ff), q = experts_kq_scratch_bytes(cap_entries, L->n_embd, L->n_ff);
    return f + (m > q ? m : q) + 4096;
}

extern "C" int32_t bsx_quantize_q8_1_rows(const float* x, int64_t n_rows, int64_t n_cols, void* y, void* stream) {
    if (n_rows < 0 || n_cols < 0 || n_cols % 32) return BSX_E_GEOMETRY;
    const int64_t n = n_rows * n_cols;
    if (n == 0) return BSX_OK;
    if (!x || !aligned(y, 4)) return BSX_E_POINTER;
    quantize_q8_1_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(x, (uint8_t*) y, n);
    const int32_t rc = launch_status();
    if (rc == BSX_OK && !stream) {
        const cudaError_t e = cudaStreamSynchronize(nullptr);
        if (e != cudaSuccess) return (int32_t) e;
    }
    return rc;
}

static int32_t experts_grouped_impl(int32_t n_x_rows, const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                       const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                       int64_t cap_entries, const void* x, int32_t x_kind, void* scratch, void* out,
                                       int32_t out_kind, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout) return BSX_E_POINTER;
    if (!bsx_expert_supported(layout->gu_type, layout->d_type, layout->up_type, layout->n_embd, layout->n_ff)) return BSX_E_TYPE;
    if (x_kind < BSX_X_F32 || x_kind > BSX_X_Q8_1 || (out_kind != BSX_OUT_F32 && out_kind != BSX_OUT_BF16)) return BSX_E_GEOMETRY;
    if (cap_groups < 0 || cap_entries < 0 || cap_entries > (int64_t) 1 << 30) return BSX_E_GEOMETRY;
    if (cap_groups == 0 || cap_entries == 0) return BSX_OK;
    if (!grp_ptr || !grp_start || !n_groups || !ent_dst || !ent_tok || !aligned(x, 16) || !aligned(scratch, 16) || !aligned(out, 16))
        return BSX_E_POINTER;
    ExpertArgs a;
    a.L = *layout;
    a.grp_ptr = grp_ptr;
    a.grp_start = grp_start;
    a.n_groups = n_groups;
    a.ent_dst = ent_dst;
    a.ent_tok = ent_tok;
    a.cap_groups = cap_groups;
    a.cap_entries = cap_entries;
    a.x = x;
    a.x_kind = x_kind;
    a.h = static_cast<float*>(scratch);
    a.out = out;
    a.out_kind = out_kind;
    a.n_x_rows = n_x_rows > 0 ? n_x_rows : 0;
    a.grid = iq1_device_grid();
    if (!a.grid) return (int32_t) cudaErrorInvalidSymbol;
    const cudaStream_t st = (cudaStream_t) stream;
    if (!(a.L.options & BSX_EXPERT_PLAIN)) {
        int32_t rc = experts_grouped_mma(a, st);      // NVFP4 blobs: fp16 images, mma.sync
        if (rc != BSX_E_TYPE) return rc;
        rc = experts_grouped_kq(a, st);               // Q6_K / IQ1_M blobs: int8 images, integer mma.sync
        if (rc != BSX_E_TYPE) return rc;
    }
    return experts_grouped_simple(a, st);
}

extern "C" int32_t bsx_experts_grouped(const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                       const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                       int64_t cap_entries, const void* x, int32_t x_kind, void* scratch, void* out, int32_t out_kind,
                                       void* stream) {
    return experts_grouped_impl(0, layout, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, x, x_kind, scratch, out,
                                out_kind, stream);
}

extern "C" int32_t bsx_experts_grouped_rows(const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                            const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                            int64_t cap_entries, const void* x, int32_t x_kind, int32_t n_x_rows, void* scratch, void* out,
                                            int32_t out_kind, void* stream) {
    if (n_x_rows < 0 || n_x_rows > cap_entries) n_x_rows = 0;   // more rows than entries: per-entry images are the cheaper form
    return experts_grouped_impl(n_x_rows, layout, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, x, x_kind, scratch,
                                out, out_kind, stream);
}

extern "C" int32_t bsx_gather_rows(const void* x, int64_t row_bytes, const int32_t* src, int64_t n_rows, void* out, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (n_rows < 0 || row_bytes <= 0 || row_bytes % 16) return BSX_E_GEOMETRY;
    if (n_rows == 0) return BSX_OK;
    if (!aligned(x, 16) || !aligned(out, 16) || !src) return BSX_E_POINTER;
    const int64_t per = row_bytes / 16, n = n_rows * per;
    gather_rows_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(static_cast<const uint4*>(x), src, static_cast<uint4*>(out),
                                                                                        n_rows, per);
    return launch_status();
}

extern "C" size_t bsx_gated_mlp_scratch_bytes(const bsx_expert_layout* L, int64_t cap_tok) {
    const size_t e = bsx_expert_scratch_bytes(L, cap_tok);
    return e ? e + gated_plan_bytes(cap_tok) : 0;
}

extern "C" int32_t bsx_gated_mlp(const bsx_expert_layout* layout, const void* blob, int32_t n_tok, int64_t cap_tok, const void* x,
                                 int32_t x_kind, void* scratch, void* out, int32_t out_kind, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout || !blob || !aligned(scratch, 16)) return BSX_E_POINTER;
    if (n_tok < 0 || n_tok > cap_tok) return BSX_E_GEOMETRY;
    if (n_tok == 0) return BSX_OK;
    uint8_t* p = static_cast<uint8_t*>(scratch);
    unsigned long long* ptr = reinterpret_cast<unsigned long long*>(p);
    int32_t* start = reinterpret_cast<int32_t*>(p + 16);
    int32_t* n_groups = reinterpret_cast<int32_t*>(p + 32);
    int32_t* idx = reinterpret_cast<int32_t*>(p + 64);
    gated_mlp_plan_kernel<<<(unsigned) ((n_tok + 127) / 128), 128, 0, (cudaStream_t) stream>>>((unsigned long long) (uintptr_t) blob, n_tok, ptr, start,
                                                                                             n_groups, idx);
    const int32_t rc = launch_status();
    if (rc != BSX_OK) return rc;
    return experts_grouped_impl(n_tok, layout, ptr, start, n_groups, idx, idx, 1, n_tok, x, x_kind, p + gated_plan_bytes(cap_tok), out, out_kind,
                                stream);
}

static int32_t combine_impl(const float* rows, const int32_t* slot, const float* weights, const float* shared, const float* shared_gate,
                            const float* resid, int32_t T, int32_t k, int32_t H, const int32_t* ids, int32_t e_lo, int32_t e_hi, float* y, void* stream,
                            int32_t blk_tok = 0, int32_t blk_stride = 0, int32_t sh_lo = 0, int32_t sh_n = 0, const uint8_t* replicated = nullptr) {
    if (!stream) return BSX_E_STREAM;
    if (T < 0 || k < 1 || k > 64 || H < 4 || H % 4) return BSX_E_GEOMETRY;
    if (T == 0) return BSX_OK;
    if (!aligned(rows, 16) || !weights || !aligned(y, 16) || (shared && !aligned(shared, 16)) || (resid && !aligned(resid, 16))) return BSX_E_POINTER;
    for (int32_t t0 = 0; t0 < T; t0 += 65535) {   // grid.y limit
        const int32_t nt = T - t0 < 65535 ? T - t0 : 65535;
        const dim3 grid((unsigned) ((H / 4 + 127) / 128), (unsigned) nt);
        launch_k(combine_kernel, grid, dim3(128), 0, (cudaStream_t) stream, rows, slot ? slot + (size_t) t0 * k : nullptr, weights + (size_t) t0 * k,
                 shared ? shared + (size_t) t0 * H : nullptr, shared_gate ? shared_gate + t0 : nullptr, resid ? resid + (size_t) t0 * H : nullptr,
                 (int) k, (int) H, (int) (t0 * k), ids ? ids + (size_t) t0 * k : nullptr, (int) e_lo, (int) e_hi, y + (size_t) t0 * H, (int) blk_tok,
                 (int) blk_stride, (int) sh_lo, (int) sh_n, replicated);
        if (blk_tok > 0 || sh_n > 0) break;   // the blocked / own-token forms take one launch (T <= 65535)
    }
    return launch_status();
}

extern "C" int32_t bsx_combine(const float* rows, const int32_t* slot, const float* weights, const float* shared,
                               const float* shared_gate, int32_t T, int32_t k, int32_t H, float* y, void* stream) {
    return combine_impl(rows, slot, weights, shared, shared_gate, nullptr, T, k, H, nullptr, 0, 0, y, stream);
}

extern "C" int32_t bsx_combine_residual(const float* rows, const int32_t* slot, const float* weights, const float* shared,
                                        const float* shared_gate, const float* residual, int32_t T, int32_t k, int32_t H, float* y, void* stream) {
    return combine_impl(rows, slot, weights, shared, shared_gate, residual, T, k, H, nullptr, 0, 0, y, stream);
}

extern "C" int32_t bsx_combine_partial_ep(const float* rows, const float* weights, const int32_t* ids, int32_t tokens_per_block, int32_t block_stride,
                                          int32_t e_lo, int32_t e_hi, int32_t T, int32_t k, int32_t H, const float* shared, int32_t tok_lo, int32_t tok_n,
                                          const uint8_t* replicated, float* y, void* stream) {
    if (!ids) return BSX_E_POINTER;
    if (T > 65535 || tokens_per_block < 0 || tok_lo < 0 || tok_n < 0 || (replicated && tok_n <= 0)) return BSX_E_GEOMETRY;
    return combine_impl(rows, nullptr, weights, tok_n > 0 ? shared : nullptr, nullptr, nullptr, T, k, H, ids, e_lo, e_hi, y, stream, tokens_per_block,
                        block_stride, tok_lo, tok_n, replicated);
}

extern "C" int32_t bsx_combine_partial(const float* rows, const int32_t* slot, const float* weights, const int32_t* ids, int32_t e_lo,
                                       int32_t e_hi, int32_t T, int32_t k, int32_t H, float* y, void* stream) {
    if (!ids) return BSX_E_POINTER;
    return combine_impl(rows, slot, weights, nullptr, nullptr, nullptr, T, k, H, ids, e_lo, e_hi, y, stream);
}
