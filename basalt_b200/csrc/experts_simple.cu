// experts_simple.cu - the plain grouped-expert kernels: one warp per weight row, 32 values per lane step, fp32 FMA on exactly
// decoded weights.  They handle every supported format pair, activation kind and group size, and serve as the in-library
// twin the tensor-core decode kernels (experts_mma.cu) are checked against; the entry point uses them when the fast path
// does not cover a shape.
//
// Semantics: Basalt's native_expert_grouped (include/basalt/kernels/iq_kernels.hpp:77-92, src/kernels/cuda/iq_kernels.cu:3304-3411):
// group g's blob at grp_ptr[g], entries [grp_start[g], grp_start[g+1]) read activation row ent_tok[e] and write output row
// ent_dst[e]; NVFP4 tail scales multiply each finished dot (iq_kernels.cu:683-701); SwiGLU forms of iq_kernels.cu:2512-2524,
// :3263-3298.  Unlike the reference, neither x nor h is rounded to int8.
#include <cuda_bf16.h>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"

namespace bsx {
namespace {

constexpr int kTok = 4;   // entries per pass of a weight row

__device__ __forceinline__ void decode32(int type, const uint8_t* row, int unit, const uint16_t* grid, float* y) {
    if (type == kTypeNVFP4) {
        const uint8_t* b = row + (size_t) (unit >> 1) * 36;
        const uint32_t* w = reinterpret_cast<const uint32_t*>(b);   // rows are 4-byte aligned
        const uint32_t dw = w[0];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int sb = 2 * (unit & 1) + s;
            const float d = ue4m3_half((dw >> (8 * sb)) & 0xFFu);
            const uint32_t q0 = w[1 + 2 * sb], q1 = w[2 + 2 * sb];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                y[16 * s + j] = e2m1_x2((q0 >> (8 * j)) & 15u) * d;
                y[16 * s + j + 8] = e2m1_x2((q0 >> (8 * j + 4)) & 15u) * d;
                y[16 * s + j + 4] = e2m1_x2((q1 >> (8 * j)) & 15u) * d;
                y[16 * s + j + 12] = e2m1_x2((q1 >> (8 * j + 4)) & 15u) * d;
            }
        }
    } else if (type == kTypeQ6K) {
        decode_q6k_32(row + (size_t) (unit >> 3) * 210, unit & 7, y);
    } else if (type == kTypeQ8_0) {
        decode_q8_0_32(row + (size_t) unit * 34, y);
    } else if (type == kTypeQ4K) {
        decode_q4k_32(row + (size_t) (unit >> 3) * 144, unit & 7, y);
    } else if (type == kTypeQ5K) {
        decode_q5k_32(row + (size_t) (unit >> 3) * 176, unit & 7, y);
    } else if (type == kTypeQ5_0 || type == kTypeQ5_1) {
        decode_q5_01_32(row + (size_t) unit * (type == kTypeQ5_1 ? 24 : 22), type == kTypeQ5_1, y);
    } else if (type == kTypeIQ4NL) {
        decode_iq4nl_32(row + (size_t) unit * 18, y);
    } else if (type == kTypeIQ4XS) {
        decode_iq4xs_32(row + (size_t) (unit >> 3) * 136, unit & 7, y);
    } else if (type == kTypeIQ1M) {
        decode_iq1m_32(row + (size_t) (unit >> 3) * 56, unit & 7, grid, y);
    } else {
        decode_any_32(type, row, unit, grid, y);
    }
}

// the codebook words the formats `t0` and `t1` read, from the device table to the block's copy (same offsets)
__device__ __forceinline__ void stage_grid(uint16_t* s_grid, const uint16_t* grid, int t0, int t1) {
    if (!type_needs_grid(t0) && !type_needs_grid(t1)) return;   // uniform over the block
    int lo, n;
    grid_range(t0, lo, n);
    for (int i = threadIdx.x; i < n; i += blockDim.x) s_grid[lo + i] = grid[lo + i];
    if (t1 != t0) {
        grid_range(t1, lo, n);
        for (int i = threadIdx.x; i < n; i += blockDim.x) s_grid[lo + i] = grid[lo + i];
    }
    __syncthreads();
}

// 32 consecutive activations [32 unit, 32 unit + 32) of row `tok`
__device__ __forceinline__ void load_x32(const void* x, int kind, int64_t tok, int64_t K, int unit, float* v) {
    if (kind == BSX_X_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + tok * K + 32 * unit);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 f = p[i];
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else if (kind == BSX_X_BF16) {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + tok * K + 32 * unit);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 u = p[i];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            }
        }
    } else {   // q8_1: 36-byte blocks {fp16 d, fp16 sum, 32 int8}; value = d * q
        const uint32_t* p = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(x) + (tok * (K / 32) + unit) * 36);
        const float d = __half2float(__ushort_as_half((unsigned short) (p[0] & 0xFFFFu)));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w = p[1 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[4 * i + j] = d * (float) (int8_t) ((w >> (8 * j)) & 0xFFu);
        }
    }
}

__device__ __forceinline__ float dot32(const float* w, const float* v, float acc) {
#pragma unroll
    for (int i = 0; i < 32; ++i) acc = fmaf(w[i], v[i], acc);
    return acc;
}

// gate and up row r of every group against the group's entries -> h[entry][r]
__global__ void __launch_bounds__(256)
gu_simple_kernel(ExpertArgs a) {
    __shared__ uint16_t s_grid[kGridWords];
    stage_grid(s_grid, a.grid, a.L.gu_type, a.L.up_type);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    if (r >= a.L.n_ff) return;
    const int ng = min(*a.n_groups, (int) a.cap_groups);
    const int64_t K = a.L.n_embd;
    const int units = (int) (K / 32);
    for (int g = blockIdx.y; g < ng; g += gridDim.y) {
        const uint8_t* blob = reinterpret_cast<const uint8_t*>(a.grp_ptr[g]);
        const uint8_t* grow = blob + (size_t) r * a.L.gu_row;
        const uint8_t* urow = blob + a.L.up_off + (size_t) r * a.L.up_row;
        float sg = 1.f, su = 1.f;
        if (a.L.gu_type == kTypeNVFP4) {
            const float* tail = reinterpret_cast<const float*>(blob + a.L.bytes - 16);
            sg = tail[0];
            su = tail[1];
        }
        const int e0 = a.grp_start[g], e1 = min(a.grp_start[g + 1], (int) a.cap_entries);
        for (int eb = e0; eb < e1; eb += kTok) {
            const int nt = min(kTok, e1 - eb);
            int64_t tok[kTok];
#pragma unroll
            for (int t = 0; t < kTok; ++t) tok[t] = t < nt ? a.ent_tok[eb + t] : 0;
            float ag[kTok] = {}, au[kTok] = {};
            for (int u = lane; u < units; u += 32) {
                float w[32], v[32];
                decode32(a.L.gu_type, grow, u, s_grid, w);
#pragma unroll
                for (int t = 0; t < kTok; ++t)
                    if (t < nt) { load_x32(a.x, a.x_kind, tok[t], K, u, v); ag[t] = dot32(w, v, ag[t]); }
                decode32(a.L.up_type, urow, u, s_grid, w);
#pragma unroll
                for (int t = 0; t < kTok; ++t)
                    if (t < nt) { load_x32(a.x, a.x_kind, tok[t], K, u, v); au[t] = dot32(w, v, au[t]); }
            }
#pragma unroll
            for (int t = 0; t < kTok; ++t) {
                const float gs = warp_sum_xor(ag[t]), us = warp_sum_xor(au[t]);
                if (lane == 0 && t < nt) a.h[(size_t) (eb + t) * a.L.n_ff + r] = swiglu(gs * sg, us * su, a.L);
            }
        }
    }
}

// down row r of every group against h[entry] -> out[dst[entry]][r]
__global__ void __launch_bounds__(256)
down_simple_kernel(ExpertArgs a) {
    __shared__ uint16_t s_grid[kGridWords];
    stage_grid(s_grid, a.grid, a.L.d_type, a.L.d_type);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    if (r >= a.L.n_embd) return;
    const int ng = min(*a.n_groups, (int) a.cap_groups);
    const int64_t K = a.L.n_ff;
    const int units = (int) (K / 32);
    for (int g = blockIdx.y; g < ng; g += gridDim.y) {
        const uint8_t* blob = reinterpret_cast<const uint8_t*>(a.grp_ptr[g]);
        const uint8_t* drow = blob + a.L.down_off + (size_t) r * a.L.d_row;
        const float sd = a.L.gu_type == kTypeNVFP4 ? reinterpret_cast<const float*>(blob + a.L.bytes - 16)[2] : 1.f;
        const int e0 = a.grp_start[g], e1 = min(a.grp_start[g + 1], (int) a.cap_entries);
        for (int eb = e0; eb < e1; eb += kTok) {
            const int nt = min(kTok, e1 - eb);
            float acc[kTok] = {};
            for (int u = lane; u < units; u += 32) {
                float w[32], v[32];
                decode32(a.L.d_type, drow, u, s_grid, w);
#pragma unroll
                for (int t = 0; t < kTok; ++t)
                    if (t < nt) { load_x32(a.h, BSX_X_F32, eb + t, K, u, v); acc[t] = dot32(w, v, acc[t]); }
            }
#pragma unroll
            for (int t = 0; t < kTok; ++t) {
                const float s = warp_sum_xor(acc[t]) * sd;
                if (lane == 0 && t < nt) store_out(a.out, a.out_kind, (int64_t) a.ent_dst[eb + t] * a.L.n_embd + r, s);
            }
        }
    }
}

}  // namespace

int32_t experts_grouped_simple(const ExpertArgs& a, cudaStream_t st) {
    const unsigned gy = (unsigned) (a.cap_groups < 1 ? 1 : a.cap_groups > 512 ? 512 : a.cap_groups);
    const int phase = experts_phase(a.L);
    if (phase != 2) gu_simple_kernel<<<dim3((unsigned) ((a.L.n_ff + 7) / 8), gy), 256, 0, st>>>(a);
    if (phase != 1) down_simple_kernel<<<dim3((unsigned) ((a.L.n_embd + 7) / 8), gy), 256, 0, st>>>(a);
    return launch_status();
}

}  // namespace bsx
