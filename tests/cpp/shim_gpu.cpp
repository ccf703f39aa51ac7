// Runs one decode-window step of a small MoE layer ON THE GPU through the reference-signature shim alone (basalt_shim.hpp +
// the CUDA runtime): router -> moe_plan -> quantize_q8_1_rows -> native_expert_grouped -> native_moe_combine_multi, then the
// prompt path's group call (fp4::quantize_tokens + fp4::run_group) on the same layer.  Inputs come from a file the Python
// test writes; outputs go to a file it compares, bit for bit, with the same calls made through ctypes.
//
// file in:  int32 header {E, H, I, k, T, blob_stride}, then gate [E][H] f32, x [T][H] f32, blobs [E][stride] u8
// file out: logits [T][E] f32, ids [T][k] i32, w [T][k] f32, y [T][H] f32, dm [T*k][H] f32 (prompt path rows in dispatch order)
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <vector>

#include "basalt_shim.hpp"

using namespace basalt::kernels;

#define CK(e)                                                                                   \
    do {                                                                                        \
        const cudaError_t err_ = (e);                                                           \
        if (err_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #e, cudaGetErrorString(err_)); return 2; } \
    } while (0)

template <typename T>
static T* dev_alloc(size_t n) {
    void* p = nullptr;
    if (cudaMalloc(&p, n * sizeof(T) + 256) != cudaSuccess) { std::fprintf(stderr, "cudaMalloc failed\n"); std::exit(2); }
    cudaMemset(p, 0, n * sizeof(T) + 256);
    return static_cast<T*>(p);
}

int main(int argc, char** argv) {
    if (argc != 3) { std::fprintf(stderr, "usage: shim_gpu <in> <out>\n"); return 2; }
    FILE* f = std::fopen(argv[1], "rb");
    if (!f) return 2;
    int32_t hd[6];
    if (std::fread(hd, 4, 6, f) != 6) return 2;
    const int E = hd[0], H = hd[1], I = hd[2], k = hd[3], T = hd[4];
    const size_t stride = (size_t) hd[5];
    std::vector<float> gate((size_t) E * H), x((size_t) T * H);
    std::vector<uint8_t> blobs((size_t) E * stride);
    if (std::fread(gate.data(), 4, gate.size(), f) != gate.size() || std::fread(x.data(), 4, x.size(), f) != x.size() ||
        std::fread(blobs.data(), 1, blobs.size(), f) != blobs.size()) return 2;
    std::fclose(f);

    cudaStream_t st;
    CK(cudaStreamCreate(&st));
    float* d_gate = dev_alloc<float>(gate.size());
    float* d_x = dev_alloc<float>(x.size());
    uint8_t* d_blobs = dev_alloc<uint8_t>(blobs.size());
    CK(cudaMemcpy(d_gate, gate.data(), gate.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_x, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_blobs, blobs.data(), blobs.size(), cudaMemcpyHostToDevice));
    const int n = T * k;
    float* d_logits = dev_alloc<float>((size_t) T * E);
    int32_t* d_ids = dev_alloc<int32_t>(n);
    float* d_w = dev_alloc<float>(n);
    std::vector<unsigned long long> table(E);
    for (int e = 0; e < E; ++e) table[e] = (unsigned long long) (uintptr_t) (d_blobs + (size_t) e * stride);
    unsigned long long* d_table = dev_alloc<unsigned long long>(E);
    CK(cudaMemcpy(d_table, table.data(), (size_t) E * 8, cudaMemcpyHostToDevice));
    unsigned long long* d_ptr = dev_alloc<unsigned long long>(n + 3);
    int32_t* d_start = dev_alloc<int32_t>(n + 3);
    int32_t* d_ng = dev_alloc<int32_t>(4);
    int32_t* d_dst = dev_alloc<int32_t>(n);
    int32_t* d_tok = dev_alloc<int32_t>(n);
    float* d_rows = dev_alloc<float>((size_t) n * H);
    float* d_y = dev_alloc<float>((size_t) T * H);

    // ---- decode window, the reference's call sequence (src/models/inkling2/session.cpp:680-716)
    RouterArgs ra;
    ra.n_expert = E; ra.n_embd = H; ra.k = k; ra.weight_scale = 2.5f; ra.gate = RouterGate::Sigmoid;
    router(d_x, d_gate, nullptr, T, ra, d_logits, d_ids, d_w, st);
    moe_plan(d_ids, T, k, E, d_table, d_ptr, d_start, d_ng, d_dst, d_tok, st);
    const NativeExpertLayout L = native_expert_layout(40, 40, H, I);
    uint8_t* d_q8 = dev_alloc<uint8_t>((size_t) T * H / 32 * 36);
    quantize_q8_1_rows(d_x, T, H, d_q8, st);
    uint8_t* d_scr = dev_alloc<uint8_t>(native_expert_scratch_bytes(L, n));
    native_expert_grouped(L, d_ptr, d_start, d_ng, d_dst, d_tok, n < E ? n : E, n, d_q8, d_scr, d_rows, st);
    native_moe_combine_multi(d_rows, d_w, nullptr, d_y, H, k, T, st);
    CK(cudaStreamSynchronize(st));

    // ---- the same window as ONE call (bsx_moe_layer): fp32 rows in, the layer's rows out, everything else in a workspace.
    // With the blobs in place and fp32 activations the experts run the fp16-image kernels, so the rows differ from the q8_1
    // sequence above by that rounding only; the routing is the same to the bit.
    bsx_moe_layer_desc ld;
    std::memset(&ld, 0, sizeof ld);
    if (bsx_expert_layout_init(40, 40, -1, H, I, 0.f, 0.f, 0.f, &ld.layout) != 0) return 4;
    ld.n_expert = E; ld.top_k = k; ld.gate_kind = BSX_GATE_SIGMOID; ld.n_group = 1; ld.topk_group = 1; ld.packed = 0;
    ld.weight_scale = 2.5f;
    ld.gate = d_gate; ld.blob_table = d_table;
    const size_t ws_bytes = bsx_moe_layer_workspace_bytes(&ld, T);
    if (!ws_bytes) return 4;
    uint8_t* d_ws = dev_alloc<uint8_t>(ws_bytes);
    float* d_y1 = dev_alloc<float>((size_t) T * H);
    int32_t* d_st1 = dev_alloc<int32_t>(4);
    const int rc1 = bsx_moe_layer(&ld, d_x, BSX_X_F32, T, T, nullptr, d_ws, d_y1, d_st1, st);
    if (rc1 != 0) { std::fprintf(stderr, "bsx_moe_layer: %d\n", rc1); return 4; }
    CK(cudaStreamSynchronize(st));
    bsx_moe_layer_views_t lv;
    if (bsx_moe_layer_views(&ld, T, d_ws, &lv) != 0) return 4;
    std::vector<int32_t> ids1(n);
    std::vector<float> y1((size_t) T * H);
    CK(cudaMemcpy(ids1.data(), lv.ids, (size_t) n * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(y1.data(), d_y1, y1.size() * 4, cudaMemcpyDeviceToHost));

    // ---- the prompt path on the same layer: rows grouped by expert (fused::group), then the experts in groups of 16
    namespace pf = basalt::prefill;
    uint8_t* d_gscr = dev_alloc<uint8_t>(pf::fused::group_bytes(n, E));
    int32_t* d_slot = dev_alloc<int32_t>(n);
    int32_t* d_src = dev_alloc<int32_t>(n);
    pf::fused::group(d_ids, n, k, E, d_gscr, d_slot, d_src, st);
    CK(cudaStreamSynchronize(st));
    std::vector<int32_t> bounds(E + 1);
    CK(cudaMemcpy(bounds.data(), reinterpret_cast<int32_t*>(d_gscr) + E, (size_t) (E + 1) * 4, cudaMemcpyDeviceToHost));   // off[E + 1] follows cnt[E]
    const int32_t* d_bounds = reinterpret_cast<int32_t*>(d_gscr) + E;
    float* d_dm = dev_alloc<float>((size_t) n * H);
    uint8_t* d_a4x = dev_alloc<uint8_t>(pf::fp4::token_bytes(T, H));
    float* d_gsx = dev_alloc<float>(T);
    pf::fp4::quantize_tokens(d_x, T, H, H, d_a4x, d_gsx, st);
    int32_t* d_status = dev_alloc<int32_t>(4);
    const size_t gbytes = pf::fp4::group_scratch_bytes(L, T, n);
    uint8_t* d_grp = dev_alloc<uint8_t>(gbytes);
    int runs = 0;
    for (int j0 = 0; j0 < E; j0 += pf::fp4::kMaxExperts) {
        pf::fp4::Group g;
        g.n = E - j0 < pf::fp4::kMaxExperts ? E - j0 : pf::fp4::kMaxExperts;
        for (int i = 0; i < g.n; ++i) g.blob[i] = d_blobs + (size_t) (j0 + i) * stride;
        g.bounds_host = bounds.data() + j0;
        g.bounds_dev = d_bounds + j0;
        g.ids = d_src;
        g.a4x = d_a4x; g.gsx = d_gsx; g.tokens = T;
        g.down_off = L.down_off; g.tail_off = L.bytes - 16;
        g.dm = d_dm;
        g.layout = L; g.scratch = d_grp; g.scratch_bytes = gbytes; g.status = d_status;
        // bounds_host[g.n] must bound every row of the layer the scratch covers: the last group's end is the layer's row count
        runs += pf::fp4::run_group(g, 4096, st);
    }
    CK(cudaStreamSynchronize(st));
    int32_t status = 0;
    CK(cudaMemcpy(&status, d_status, 4, cudaMemcpyDeviceToHost));
    if (status != 0 || runs < 1) { std::fprintf(stderr, "prompt path: status %d runs %d\n", status, runs); return 3; }

    std::vector<float> logits((size_t) T * E), w(n), y((size_t) T * H), dm((size_t) n * H);
    std::vector<int32_t> ids(n);
    CK(cudaMemcpy(logits.data(), d_logits, logits.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(ids.data(), d_ids, ids.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(w.data(), d_w, w.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(y.data(), d_y, y.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dm.data(), d_dm, dm.size() * 4, cudaMemcpyDeviceToHost));
    FILE* o = std::fopen(argv[2], "wb");
    if (!o) return 2;
    std::fwrite(logits.data(), 4, logits.size(), o);
    std::fwrite(ids.data(), 4, ids.size(), o);
    std::fwrite(w.data(), 4, w.size(), o);
    std::fwrite(y.data(), 4, y.size(), o);
    std::fwrite(dm.data(), 4, dm.size(), o);
    std::fwrite(ids1.data(), 4, ids1.size(), o);
    std::fwrite(y1.data(), 4, y1.size(), o);
    std::fclose(o);
    std::puts("shim gpu ok");
    return 0;
}
