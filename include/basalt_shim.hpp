// basalt_shim.hpp - the Basalt engine's MoE operator signatures over the B200 C ABI (basalt_b200.h).
//
// Including this header instead of the engine's own include/basalt/kernels/{router,route_lossy,iq_kernels}.hpp and
// include/basalt/models/qwen4exp/kernels/{native_moe,native_router,router_top10}.hpp lets its callers (src/model, src/prefill,
// src/spec, the per-model layer loops) compile unchanged against libbasalt_b200.so: same namespaces, names, argument order
// and meaning, and the same error behaviour - geometry errors throw std::invalid_argument where the reference throws
// (src/kernels/cuda/router.cu:236,258; src/models/qwen4exp/kernels/native_moe.cu:62-71), launch failures throw std::runtime_error
// where the reference logs and exits (src/kernels/cuda/iq_kernels.cu:31-34).  Header-only; no CUDA headers needed.
//
// Differences a caller can observe, all documented at the C ABI:
//   - native_expert_scratch_bytes(cap, n_ff) cannot know n_embd (the tensor-core path keeps fp16 activation images in
//     scratch), so it returns the bound for n_embd = 8192, the router's own limit; use the layout form to size exactly;
//   - expert outputs sit ~1e-5 (not ~1e-2) from the dequantised fp32 reference, because activations are not rounded to int8.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "basalt_b200.h"

namespace basalt::kernels {

namespace shim_detail {
inline void raise(const char* fn, int32_t rc) {
    if (rc == BSX_OK) return;
    if (rc < 0) throw std::invalid_argument(std::string(fn) + ": unsupported geometry or arguments (" + std::to_string(rc) + ")");
    throw std::runtime_error(std::string(fn) + ": CUDA error " + std::to_string(rc));
}
}  // namespace shim_detail

// ---- include/basalt/kernels/route_lossy.hpp
struct ResidentTabs {
    static constexpr int kMax = BSX_MAX_HELD_TABS;
    const int32_t* t[kMax] = {};
    int n = 0;
    void add(const int32_t* tab) { if (tab != nullptr && n < kMax) t[n++] = tab; }
};
constexpr int kRouteTailSkipMax = BSX_TAIL_SKIP_MAX;

inline void route_tail_skip(int32_t* ids, float* weights, const ResidentTabs& held, int n_entries, int k, int rank, int n_expert,
                            unsigned long long* counts, void* stream) {
    shim_detail::raise("route_tail_skip", bsx_route_tail_skip(ids, weights, held.t, held.n, n_entries, k, rank, n_expert, counts, stream));
}

// ---- include/basalt/kernels/router.hpp
enum class RouterGate : int { SqrtSoftplus = BSX_GATE_SQRT_SOFTPLUS, Sigmoid = BSX_GATE_SIGMOID };

struct RouterArgs {
    int n_expert = 384;
    int n_embd = 5120;
    int k = 6;
    float weight_scale = 1.5f;
    RouterGate gate = RouterGate::SqrtSoftplus;
    float prior = 0.0f;
    ResidentTabs held;
    // group-limited selection (not in the reference; 1 / 1 = the reference's router, bit for bit)
    int n_group = 1;
    int topk_group = 1;
};

inline void router(const float* x, const float* gate, const float* bias, int n_tokens, const RouterArgs& a, float* logits, int32_t* ids,
                   float* weights, void* stream) {
    if (a.n_expert > 512 && a.n_group <= 1)   // the reference's own limit (router.cu:235); the wider range needs the C ABI
        throw std::invalid_argument("router: unsupported geometry");
    shim_detail::raise("router", bsx_router(x, gate, bias, n_tokens, a.n_expert, a.n_embd, a.k, (int) a.gate, a.weight_scale, a.n_group,
                                           a.topk_group, a.prior, a.held.t, a.held.n, logits, ids, weights, stream));
}

inline void router_select(const float* logits, const float* bias, int n_tokens, const RouterArgs& a, int32_t* ids, float* weights,
                          void* stream) {
    shim_detail::raise("router_select", bsx_router_select(logits, bias, n_tokens, a.n_expert, a.k, (int) a.gate, a.weight_scale, a.n_group,
                                                         a.topk_group, a.prior, a.held.t, a.held.n, ids, weights, stream));
}

// ---- include/basalt/models/qwen4exp/kernels/router_top10.hpp, native_router.hpp and the prompt path's route()
inline void router_top10(const float* logits, int n_tokens, int n_expert, int k, int* ids, float* weights, void* stream) {
    if (n_tokens <= 0 || n_expert <= 0 || k <= 0) return;
    shim_detail::raise("router_top10", bsx_router_select(logits, nullptr, n_tokens, n_expert, k, BSX_GATE_SOFTMAX_F64, 1.0f, 1, 1, 0.0f, nullptr,
                                                        0, ids, weights, stream));
}
inline void native_router_top10_multi(const float* logits, int32_t* ids, float* weights, int n_tok, void* stream) {
    if (!stream) throw std::invalid_argument("native router requires a stream");
    shim_detail::raise("native_router_top10", bsx_router_select(logits, nullptr, n_tok, 512, 10, BSX_GATE_SOFTMAX_FAST, 1.0f, 1, 1, 0.0f,
                                                               nullptr, 0, ids, weights, stream));
}
inline void native_router_top10(const float* logits, int32_t* ids, float* weights, void* stream) {
    native_router_top10_multi(logits, ids, weights, 1, stream);
}

// ---- include/basalt/kernels/iq_kernels.hpp (the MoE part)
struct NativeExpertLayout {
    int gu_type = -1, d_type = -1;
    int up_type = -1;
    int64_t n_embd = 0, n_ff = 0;
    size_t gu_row = 0, d_row = 0;
    size_t up_row = 0;
    size_t up_off = 0, down_off = 0;
    size_t bytes = 0;
    float swiglu_limit = 0.0f;
    float gate_softcap = 0.0f, up_softcap = 0.0f;
};

namespace shim_detail {
inline bsx_expert_layout to_c(const NativeExpertLayout& L) {
    bsx_expert_layout c{};
    c.gu_type = L.gu_type; c.d_type = L.d_type; c.up_type = L.up_type < 0 ? L.gu_type : L.up_type;
    c.n_embd = L.n_embd; c.n_ff = L.n_ff;
    c.gu_row = L.gu_row; c.d_row = L.d_row; c.up_row = L.up_row;
    c.up_off = L.up_off; c.down_off = L.down_off; c.bytes = L.bytes;
    c.swiglu_limit = L.swiglu_limit; c.gate_softcap = L.gate_softcap; c.up_softcap = L.up_softcap;
    return c;
}
}  // namespace shim_detail

inline bool native_expert_supported(int gu_type, int d_type, int64_t n_embd, int64_t n_ff, int up_type = -1) noexcept {
    return bsx_expert_supported(gu_type, d_type, up_type, n_embd, n_ff) != 0;
}

inline NativeExpertLayout native_expert_layout(int gu_type, int d_type, int64_t n_embd, int64_t n_ff, float swiglu_limit = 0.0f,
                                               int up_type = -1) {
    bsx_expert_layout c{};
    shim_detail::raise("native_expert_layout", bsx_expert_layout_init(gu_type, d_type, up_type, n_embd, n_ff, swiglu_limit, 0.f, 0.f, &c));
    NativeExpertLayout L;
    L.gu_type = c.gu_type; L.d_type = c.d_type; L.up_type = c.up_type;
    L.n_embd = c.n_embd; L.n_ff = c.n_ff;
    L.gu_row = c.gu_row; L.d_row = c.d_row; L.up_row = c.up_row;
    L.up_off = c.up_off; L.down_off = c.down_off; L.bytes = c.bytes;
    L.swiglu_limit = swiglu_limit;
    return L;
}

inline size_t native_expert_scratch_bytes(const NativeExpertLayout& L, int64_t cap_entries) {
    const bsx_expert_layout c = shim_detail::to_c(L);
    return bsx_expert_scratch_bytes(&c, cap_entries);
}
/// The reference's form: n_embd is unknown here, so this is the bound for n_embd = 8192.
inline size_t native_expert_scratch_bytes(int64_t cap_entries, int64_t n_ff) {
    bsx_expert_layout c{};
    c.n_embd = 8192;
    c.n_ff = n_ff;
    return bsx_expert_scratch_bytes(&c, cap_entries);
}

inline void quantize_q8_1_rows(const float* x, int64_t n_rows, int64_t n_cols, void* y, void* stream) {
    shim_detail::raise("quantize_q8_1_rows", bsx_quantize_q8_1_rows(x, n_rows, n_cols, y, stream));
}

/// x_q8_1: the caller's q8_1 activation rows, as in the reference.  grid_groups only shapes the reference's launch; ignored.
inline void native_expert_grouped(const NativeExpertLayout& L, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                  const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                  int64_t cap_entries, const void* x_q8_1, void* scratch, float* out, void* stream,
                                  int64_t grid_groups = 0) {
    (void) grid_groups;
    const bsx_expert_layout c = shim_detail::to_c(L);
    shim_detail::raise("native_expert_grouped", bsx_experts_grouped(&c, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries,
                                                                   x_q8_1, BSX_X_Q8_1, scratch, out, BSX_OUT_F32, stream));
}

inline void native_expert_grouped_clamped(const NativeExpertLayout& L, float swiglu_limit, const unsigned long long* grp_ptr,
                                          const int32_t* grp_start, const int32_t* n_groups, const int32_t* ent_dst,
                                          const int32_t* ent_tok, int64_t cap_groups, int64_t cap_entries, const void* x_q8_1,
                                          void* scratch, float* out, void* stream, int64_t grid_groups = 0) {
    NativeExpertLayout M = L;
    M.swiglu_limit = swiglu_limit;
    native_expert_grouped(M, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, x_q8_1, scratch, out, stream,
                          grid_groups);
}

/// The load-time plane packing (cf. include/basalt/kernels/nvfp4_planes.hpp:6-20) and native_expert_grouped over packed blobs:
/// grp_ptr[g] points at a blob packed by native_expert_pack; x are fp32 (or, with x_bf16, bf16) activation rows - the packed
/// path makes its own FP4 images, so no quantize_q8_1_rows.  status: a device int32 the caller zeroes (bit 0 = a bounded
/// wait inside a kernel ran out).
inline size_t native_expert_packed_bytes(const NativeExpertLayout& L) {
    const bsx_expert_layout c = shim_detail::to_c(L);
    return bsx_expert_packed_bytes(&c);
}
inline void native_expert_pack(const NativeExpertLayout& L, const void* blob, void* packed, void* stream) {
    const bsx_expert_layout c = shim_detail::to_c(L);
    shim_detail::raise("native_expert_pack", bsx_expert_pack(&c, blob, packed, stream));
}
inline size_t native_expert_packed_scratch_bytes(const NativeExpertLayout& L, int64_t cap_entries) {
    const bsx_expert_layout c = shim_detail::to_c(L);
    return bsx_experts_packed_scratch_bytes(&c, cap_entries);
}
inline void native_expert_grouped_packed(const NativeExpertLayout& L, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                         const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                         int64_t cap_entries, const void* x, bool x_bf16, int n_x_rows, void* scratch, float* out,
                                         int32_t* status, void* stream) {
    const bsx_expert_layout c = shim_detail::to_c(L);
    shim_detail::raise("native_expert_grouped_packed",
                       bsx_experts_grouped_packed(&c, grp_ptr, grp_start, n_groups, ent_dst, ent_tok, cap_groups, cap_entries, x,
                                                  x_bf16 ? BSX_X_BF16 : BSX_X_F32, n_x_rows, scratch, out, BSX_OUT_F32, status, stream));
}

inline size_t gated_mlp_scratch_bytes(int64_t cap_tok, int64_t n_ff) {
    bsx_expert_layout c{};
    c.n_embd = 8192;
    c.n_ff = n_ff;
    return bsx_gated_mlp_scratch_bytes(&c, cap_tok);
}

inline void gated_mlp_clamped(const NativeExpertLayout& L, float swiglu_limit, const void* blob, int n_tok, int64_t cap_tok,
                              const void* x_q8_1, void* scratch, float* out, void* stream) {
    bsx_expert_layout c = shim_detail::to_c(L);
    c.swiglu_limit = swiglu_limit;
    shim_detail::raise("gated_mlp_clamped", bsx_gated_mlp(&c, blob, n_tok, cap_tok, x_q8_1, BSX_X_Q8_1, scratch, out, BSX_OUT_F32, stream));
}

// ---- include/basalt/models/qwen4exp/kernels/native_moe.hpp
inline void native_moe_combine_multi(const float* parts, const float* weights, const float* shared, float* output, int64_t n_embd,
                                     int64_t k, int n_tok, void* stream) {
    if (!stream || n_embd <= 0 || k < 1 || k > 15 || n_tok < 1)
        throw std::invalid_argument("native MoE combine (multi) requires a stream, width, 1..15 experts, tokens");
    shim_detail::raise("native_moe_combine", bsx_combine(parts, nullptr, weights, shared, nullptr, n_tok, (int32_t) k, (int32_t) n_embd, output,
                                                        stream));
}
inline void native_moe_combine(const float* parts, const float* weights, const float* shared, float* output, int64_t n_embd, int64_t k,
                               void* stream) {
    native_moe_combine_multi(parts, weights, shared, output, n_embd, k, 1, stream);
}

}  // namespace basalt::kernels

// ---- the prompt path's grouping and combine (src/models/qwen4exp/prefill: fused::group, route_count, moe_combine)
namespace basalt::prefill::fused {
inline size_t group_bytes(int64_t n, int n_expert) { return bsx_dispatch_scratch_bytes(n, n_expert) + (size_t) (2 * n_expert + 1) * 4 + 256; }
/// `scratch` holds cnt [E], off [E + 1], then the chunk table; slot / src as in the reference, but in the stable order.
inline void group(const int32_t* ids, int64_t n, int k, int n_expert, void* scratch, int32_t* slot, int32_t* src, void* stream) {
    int32_t* cnt = static_cast<int32_t*>(scratch);
    int32_t* off = cnt + n_expert;
    void* tbl = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(off + n_expert + 1) + 255) & ~(uintptr_t) 255);
    basalt::kernels::shim_detail::raise("prefill fused group", bsx_dispatch(ids, n, k, n_expert, cnt, off, slot, src, 0, nullptr, nullptr, tbl, stream));
}
}  // namespace basalt::prefill::fused

namespace basalt::prefill {
inline void moe_combine(const float* Dm, const int32_t* slot, const float* w, const float* shared, const float* sg, float* bo, int64_t T,
                        int k, int n_embd, void* stream) {
    basalt::kernels::shim_detail::raise("moe_combine", bsx_combine(Dm, slot, w, shared, sg, (int32_t) T, k, n_embd, bo, stream));
}
}  // namespace basalt::prefill

// The step before the layer (include/basalt/kernels/window_gemm.hpp:36-40): both overloads, same argument order.  Unlike the
// reference, which takes a null stream as the default stream, the stream must be given.
namespace basalt::kernels::wgemm {
inline void norm_pack(const float* x, const float* w, float eps, int64_t K, int T, void* act, float* xn, void* stream) {
    basalt::kernels::shim_detail::raise("wgemm::norm_pack", bsx_norm_pack(x, BSX_X_F32, w, eps, K, T, act, xn, stream));
}
inline void norm_pack(const uint16_t* x, const float* w, float eps, int64_t K, int T, void* act, float* xn, void* stream) {
    basalt::kernels::shim_detail::raise("wgemm::norm_pack", bsx_norm_pack(x, BSX_X_BF16, w, eps, K, T, act, xn, stream));
}
}  // namespace basalt::kernels::wgemm

// The model file's expert table (include/basalt/kernels/cpu/expert_layout.hpp:17-35,53-65): the same struct fields a caller
// reads (fmt holds the kernel-side layout in place of the CPU pool's NativeFmt), the same process-wide table filled by
// expert_layout_load_text, the same bool + err contract.
namespace basalt::kernels::cpu {
struct ExpertLayout {
    bool native = false;
    int64_t n_layers = 0, n_expert = 0;
    std::vector<basalt::kernels::NativeExpertLayout> fmt;   ///< per layer
    std::vector<uint64_t> offset, bytes;                   ///< per layer: where its blobs start, bytes per blob
    int version = 0;
    uint64_t max_blob = 0;
    uint64_t total = 0;

    uint64_t blob_bytes(int64_t layer) const { return bytes[(size_t) layer]; }
    uint64_t layer_offset(int64_t layer) const { return offset[(size_t) layer]; }
    uint64_t blob_offset(int64_t layer, int64_t expert) const { return layer_offset(layer) + (uint64_t) expert * blob_bytes(layer); }
};

inline constexpr int kExpertLayoutVersion = 7;

namespace shim_detail {
inline ExpertLayout& table() {
    static ExpertLayout g;
    return g;
}
}  // namespace shim_detail

inline const ExpertLayout& expert_layout() { return shim_detail::table(); }

inline bool expert_layout_load_text(const std::string& text, int64_t n_layers, int64_t n_expert, std::string& err, int64_t n_embd,
                                    int64_t n_ff, float swiglu_limit = 0.f) {
    if (n_layers <= 0) {
        err = "expert layout: no layers";
        return false;
    }
    std::vector<bsx_layout_row> rows((size_t) n_layers);
    bsx_layout_info info{};
    char why[512];
    if (bsx_layout_parse(text.data(), text.size(), n_layers, n_expert, n_embd, n_ff, swiglu_limit, rows.data(), &info, why, sizeof why) != BSX_OK) {
        err = why;
        return false;
    }
    ExpertLayout L;
    L.native = true;
    L.n_layers = info.n_layers;
    L.n_expert = info.n_expert;
    L.version = info.version;
    L.max_blob = info.max_blob;
    L.total = info.total;
    for (const bsx_layout_row& r : rows) {
        L.fmt.push_back(basalt::kernels::native_expert_layout(r.gu_type, r.d_type, n_embd, n_ff, swiglu_limit, r.up_type));
        L.offset.push_back(r.offset);
        L.bytes.push_back(r.blob_bytes);
    }
    shim_detail::table() = L;
    return true;
}
}  // namespace basalt::kernels::cpu
