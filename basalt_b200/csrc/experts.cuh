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

// 0 all launches, 1 gate/up only, 2 down only (bsx_experts_set_phase)
int experts_phase();

int32_t experts_grouped_simple(const ExpertArgs& a, cudaStream_t st);
// returns BSX_E_TYPE when the fast path does not cover the layout (the caller then runs the plain kernels)
int32_t experts_grouped_mma(const ExpertArgs& a, cudaStream_t st);
size_t experts_mma_scratch_bytes(int64_t cap_entries, int64_t n_embd, int64_t n_ff);

}  // namespace bsx
