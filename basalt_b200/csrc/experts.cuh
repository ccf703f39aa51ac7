// experts.cuh - argument block and epilogue helpers shared by the grouped-expert kernels.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace bsx {

struct ExpertArgs {
    bsx_expert_layout L;
    const unsigned long long* grp_ptr;
    const int32_t* grp_start;
    const int32_t* n_groups;
    const int32_t* ent_dst;
    const int32_t* ent_tok;
    int64_t cap_groups, cap_entries;
    const void* x;
    int32_t x_kind;
    float* h;            // scratch: [cap_entries][n_ff] fp32, the SwiGLU output
    void* out;
    int32_t out_kind;
    const uint16_t* grid;   // the IQ1 codebook on this device (2048 x uint16)
    int32_t n_x_rows;       // rows of x when the caller knows them (activation images are then made once per row), else 0
};

// SwiGLU forms of the Basalt engine (src/kernels/cuda/iq_kernels.cu:2520-2521 plain, :3263-3279 limited, :3283-3298
// softcapped); g and u already carry their NVFP4 tail scales.  expf is the accurate one throughout.
__device__ __forceinline__ float swiglu(float g, float u, const bsx_expert_layout& L) {
    if (L.gate_softcap > 0.f && L.up_softcap > 0.f) {
        const float sig = 1.f / (1.f + expf(-g));
        return L.gate_softcap * tanhf(g / L.gate_softcap) * sig * (L.up_softcap * tanhf(u / L.up_softcap));
    }
    if (L.swiglu_limit > 0.f) {
        g = fminf(g, L.swiglu_limit);
        u = fminf(fmaxf(u, -L.swiglu_limit), L.swiglu_limit);
    }
    return g / (1.f + expf(-g)) * u;
}

__device__ __forceinline__ void store_out(void* out, int kind, int64_t i, float v) {
    if (kind == BSX_OUT_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else static_cast<float*>(out)[i] = v;
}

// 16 consecutive values [16 sb, 16 sb + 16) of an activation row
__device__ __forceinline__ void load16(const void* x, int kind, int64_t row, int64_t K, int sb, float (&v)[16]) {
    if (kind == BSX_X_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + row * K + 16 * sb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = p[i];
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else if (kind == BSX_X_BF16) {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(x) + row * K + 16 * sb);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 u = p[i];
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
            }
        }
    } else {   // q8_1: 36-byte blocks {fp16 d, fp16 sum, 32 int8}; value = d * q
        const uint32_t* p = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(x) + (row * (K / 32) + (sb >> 1)) * 36);
        const float d = __half2float(__ushort_as_half((unsigned short) (p[0] & 0xFFFFu)));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = p[1 + 4 * (sb & 1) + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[4 * i + j] = d * (float) (int8_t) ((w >> (8 * j)) & 0xFFu);
        }
    }
}

// the IQ1 codebook (2048 x uint16, 2 bits a coordinate) in this device's global memory; null on a CUDA error
const uint16_t* iq1_device_grid();

// 0 all launches, 1 gate/up only, 2 down only (the stage bits of bsx_expert_layout.options)
inline int experts_phase(const bsx_expert_layout& L) { return L.options & BSX_EXPERT_STAGE_MASK; }

int32_t experts_grouped_simple(const ExpertArgs& a, cudaStream_t st);
// returns BSX_E_TYPE when the fast path does not cover the layout (the caller then runs the plain kernels)
int32_t experts_grouped_mma(const ExpertArgs& a, cudaStream_t st);
// the same call over blobs repacked by bsx_expert_pack (experts_nvf4.cu): block-scaled FP4 MMAs straight on the NVFP4 codes
// pass_list_ready: the pass list (plan.cuh) already sits in the scratch (the fused selection + plan kernel wrote it)
struct PassRec;
int32_t experts_grouped_packed(const ExpertArgs& a, int32_t* status, cudaStream_t st, bool x_images_ready, bool pass_list_ready);
void experts_packed_pass_list(void* scratch, int64_t cap_entries, int64_t n_embd, int64_t n_ff, PassRec** items, int** n_items);
int32_t experts_packed_x_images(const bsx_expert_layout& L, const void* x, int32_t x_kind, int32_t n_x_rows, int64_t cap, void* scratch, cudaStream_t st);
// Q6_K / IQ1_M blobs in place on the integer tensor cores (experts_kq.cu); BSX_E_TYPE when the layout is not covered
int32_t experts_grouped_kq(const ExpertArgs& a, cudaStream_t st);
size_t experts_kq_scratch_bytes(int64_t cap_entries, int64_t n_embd, int64_t n_ff);
size_t experts_packed_scratch_bytes(int64_t cap_entries, int64_t n_embd, int64_t n_ff);
size_t experts_mma_scratch_bytes(int64_t cap_entries, int64_t n_embd, int64_t n_ff);

}  // namespace bsx
