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

// ---- the decode window's plan (src/models/inkling2/kernels/ops.hpp: moe_plan) and the whole step as one call
namespace basalt::kernels {
inline void moe_plan(const int32_t* ids, int n_tokens, int k, int n_expert, const unsigned long long* blob_table, unsigned long long* ptr,
                     int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok, void* stream) {
    shim_detail::raise("moe_plan", bsx_moe_plan(ids, n_tokens, k, n_expert, blob_table, ptr, start, n_groups, dst, tok, stream));
}
}  // namespace basalt::kernels

// ---- include/basalt/prefill/moe_fp4.hpp: the prompt path's NVFP4 experts, a group of up to 16 experts at a time.
// Same names, argument order and meaning as the reference's, with these differences a caller can observe:
//   - The reference rounds activations to FP4 planes (one or two terms) that run() and run_group() then read.  This library
//     multiplies exactly decoded weights by fp16 activations instead (results ~2e-4 from the dequantised fp32 reference, not
//     ~1e-1 .. 1e-2), so quantize_tokens() does no arithmetic: it notes which rows the planes `a4` stand for, and run_group()
//     reads those rows (they must still be there when it runs, as they are in the reference's call sites: the layer's input
//     is not rewritten before its experts have run).  The planes and scale arrays are left untouched.
//   - The kernels need scratch of their own that the reference's buffers cannot hold (fp16 images of the layer's rows):
//     Group carries two more fields at its end, `scratch` / `scratch_bytes` (size: group_scratch_bytes) and `status` (a device
//     int32 the caller zeroes; bit 0 = a bounded wait inside a kernel ran out).  run_group() throws std::invalid_argument
//     when they are missing.
//   - run_experts() runs any layer geometry the layout describes (the reference's is built for 2560 x 640); set
//     Group::layout (basalt::kernels::NativeExpertLayout) - down_off / tail_off are then read from it.
//   - The plane-level calls quantize() and run(Product) have no counterpart here (there are no planes to multiply); they
//     throw std::logic_error.  plan(), plan_blocks(), rebase(), cut_pieces(), run_length() and the size helpers are the
//     reference's.
#include <algorithm>
#include <mutex>
#include <unordered_map>

namespace basalt::prefill::fp4 {

constexpr int kTileTokens = 64;
constexpr int kMaxExperts = 16;   // experts per launch

namespace shim_detail {
using basalt::kernels::shim_detail::raise;
struct Rows {
    const void* x;
    int64_t tokens, cols;
};
inline std::mutex& mu() {
    static std::mutex m;
    return m;
}
inline std::unordered_map<const void*, Rows>& noted() {
    static std::unordered_map<const void*, Rows> m;
    return m;
}
}  // namespace shim_detail

// the reference's sizes (src/prefill/moe_fp4.cu:527-532,566): a caller that sizes its buffers by them keeps working
inline size_t a4_bytes(int64_t rows, int64_t cols, int experts) {
    return (size_t) ((rows + kTileTokens - 1) / kTileTokens + experts) * (size_t) (cols / 128) * 4608u;
}
inline size_t scale_count(int64_t rows, int experts) { return (size_t) ((rows + kTileTokens - 1) / kTileTokens + experts) * kTileTokens; }
inline size_t token_bytes(int64_t tokens, int64_t cols) { return (size_t) tokens * (size_t) (cols / 2 + cols / 16); }
inline int64_t max_blocks(int64_t rows, int n) { return (rows + 2 * kTileTokens - 1) / (2 * kTileTokens) + n; }

inline void plan(const int32_t* bounds, int n, int32_t* tile_off, void* stream) {
    shim_detail::raise("fp4::plan", bsx_unit_offsets(bounds, n, kTileTokens, tile_off, stream));
}
inline void rebase(const int32_t* bounds, int n, int32_t* out, void* stream) { shim_detail::raise("fp4::rebase", bsx_rebase_bounds(bounds, n, out, stream)); }
inline void plan_blocks(const int32_t* bounds, int n, int32_t* tile_off, int32_t* blk_off, void* stream) {
    shim_detail::raise("fp4::plan_blocks", bsx_unit_offsets(bounds, n, kTileTokens, tile_off, stream));
    shim_detail::raise("fp4::plan_blocks", bsx_unit_offsets(bounds, n, 2 * kTileTokens, blk_off, stream));
}

/// Notes that the planes `a4` stand for rows x[0 .. tokens) of `cols` floats (ld == cols); see the header comment.
inline void quantize_tokens(const float* x, int64_t tokens, int64_t cols, int64_t ld, void* a4, float* gs, void* stream, bool two = false) {
    (void) gs; (void) stream; (void) two;
    if (tokens <= 0) return;
    if (ld != cols || a4 == nullptr) throw std::invalid_argument("fp4::quantize_tokens: rows must be dense and the planes given");
    std::lock_guard<std::mutex> lock(shim_detail::mu());
    shim_detail::noted()[a4] = shim_detail::Rows{x, tokens, cols};
}
inline void quantize(const float*, const int32_t*, const int32_t*, const int32_t*, int, void*, float*, int64_t, int64_t, int64_t, void*, bool = false) {
    throw std::logic_error("fp4::quantize: this library keeps no FP4 planes of the SwiGLU rows; run the experts through fp4::run_group");
}

struct Product {
    const uint8_t* blob[kMaxExperts] = {};
    size_t w_off = 0;
    int64_t w_rows = 0, w_cols = 0;
    int n = 0;
    const void* a4 = nullptr;
    const float* gs = nullptr;
    const int32_t* bounds = nullptr;
    const int32_t* tile_off = nullptr;
    float* dst = nullptr;
    int64_t ld_dst = 0, max_rows = 0;
    bool swiglu = false;
    const int32_t* ids = nullptr;
    int64_t tokens = 0;
    size_t tail_off = 0;
    const uint8_t* base = nullptr;
    size_t stride = 0;
    const int32_t* blk_off = nullptr;
    int64_t blocks = 0;
    const int32_t* dst_ids = nullptr;
    float gate_softcap = 0.0f, up_softcap = 0.0f;
    bool two = false;
};
inline void run(const Product&, void*) {
    throw std::logic_error("fp4::run: single products over FP4 planes are not provided; fp4::run_group runs gate/up, SwiGLU and down");
}

struct Group {
    int n = 0;
    const uint8_t* blob[kMaxExperts] = {};
    const int32_t* bounds_host = nullptr;   ///< n + 1 absolute row bounds, on the host
    const int32_t* bounds_dev = nullptr;    ///< the same bounds on the device
    const int32_t* ids = nullptr;           ///< the layer's token of each absolute row
    const void* a4x = nullptr;              ///< the planes quantize_tokens() was given for the layer's rows
    const float* gsx = nullptr;
    int64_t tokens = 0;
    size_t down_off = 0, tail_off = 0;
    float *h = nullptr, *dm = nullptr;      ///< dm: the layer's output rows [absolute row][n_embd]; h is not used
    void* a4h = nullptr;
    float* gsh = nullptr;
    int32_t *toh = nullptr, *rel = nullptr;
    // ---- added by this library (see the header comment)
    basalt::kernels::NativeExpertLayout layout;   ///< the experts' blob geometry
    void* scratch = nullptr;                      ///< group_scratch_bytes(layout, tokens, the layer's row count), 256-byte aligned
    size_t scratch_bytes = 0;
    int32_t* status = nullptr;
};
inline size_t group_scratch_bytes(const basalt::kernels::NativeExpertLayout& L, int64_t tokens, int64_t layer_rows) {
    const bsx_expert_layout c = basalt::kernels::shim_detail::to_c(L);
    return bsx_experts_prefill_group_scratch_bytes(&c, tokens, layer_rows);
}

/// How many experts from i0 form the next run: consecutive ones while their rows together stay within row_cap, and at least one.
inline int run_length(const Group& g, int i0, int64_t row_cap) {
    const int32_t* b = g.bounds_host;
    int last = i0 + 1;                             // one past the run's last expert
    while (last < g.n && (int64_t) b[last + 1] - b[i0] <= row_cap) ++last;
    return last - i0;
}

/// Consecutive experts [i0, i0 + n) of the group: gate/up over the rows' tokens, SwiGLU, down -> dm[absolute row].
inline void run_experts(const Group& g, int i0, int n, void* stream) {
    if (n < 1 || i0 < 0 || i0 + n > g.n || n > kMaxExperts) throw std::invalid_argument("fp4::run_experts: experts outside the group");
    shim_detail::Rows rows{};
    {
        std::lock_guard<std::mutex> lock(shim_detail::mu());
        const auto it = shim_detail::noted().find(g.a4x);
        if (it == shim_detail::noted().end()) throw std::invalid_argument("fp4::run_experts: quantize_tokens() was not called for these planes");
        rows = it->second;
    }
    if (!g.scratch || !g.status) throw std::invalid_argument("fp4::run_experts: Group::scratch and Group::status must be set (fp4::group_scratch_bytes)");
    const bsx_expert_layout c = basalt::kernels::shim_detail::to_c(g.layout);
    if (c.n_embd != rows.cols) throw std::invalid_argument("fp4::run_experts: the noted rows are not n_embd wide");
    const int64_t layer_rows = g.bounds_host[g.n];
    if (bsx_experts_prefill_group_scratch_bytes(&c, rows.tokens, layer_rows) > g.scratch_bytes) throw std::invalid_argument("fp4::run_experts: scratch too small");
    const void* blobs[kMaxExperts];
    for (int i = 0; i < n; ++i) blobs[i] = g.blob[i0 + i];
    shim_detail::raise("fp4::run_experts", bsx_experts_prefill_group(&c, blobs, n, g.bounds_dev + i0, g.ids, layer_rows, rows.x, BSX_X_F32, rows.tokens,
                                                                     g.scratch, g.dm, g.status, stream));
}

inline int run_group(const Group& g, int64_t row_cap, void* stream) {
    int runs = 0;
    for (int i0 = 0; i0 < g.n;) {
        const int n = run_length(g, i0, row_cap);
        run_experts(g, i0, n, stream);
        i0 += n;
        ++runs;
    }
    return runs;
}

struct Pieces {
    std::vector<int32_t> expert;   ///< per piece: its expert's index j
    std::vector<int32_t> bounds;   ///< per piece its first row, then the last piece's end
    std::vector<int32_t> group;    ///< per group its first piece, then the piece count
};
/// Splits the rows of n consecutive experts (host row bounds) for buffers of `cap` rows, with the result the reference's
/// cut_pieces gives (include/basalt/prefill/moe_fp4.hpp:115-123): an expert is laid out as pieces of `whole` rows from its first
/// row on, `whole` being the largest multiple of the tile size within cap (at least one tile), so that every piece starts on
/// one of the expert's own tile boundaries; an expert without rows has no piece.  Pieces are then gathered greedily, in order,
/// into groups of at most kMaxExperts pieces and at most `cap` rows.
inline void cut_pieces(const int32_t* bounds, int n, int64_t cap, Pieces& out) {
    out.expert.clear();
    out.bounds.clear();
    out.group.clear();
    int64_t whole = cap - cap % kTileTokens;
    if (whole < kTileTokens) whole = kTileTokens;
    for (int j = 0; j < n; ++j) {
        const int64_t first = bounds[j], rows = bounds[j + 1] - first;
        const int64_t pieces = rows > 0 ? (rows + whole - 1) / whole : 0;
        for (int64_t i = 0; i < pieces; ++i) {
            out.expert.push_back(j);
            out.bounds.push_back((int32_t) (first + i * whole));
        }
    }
    out.bounds.push_back(n > 0 ? bounds[n] : 0);
    const int total = (int) out.expert.size();
    int head = 0;                                  // first piece of the group being filled
    for (int i = 0; i < total; ++i) {
        const bool full = i - head == kMaxExperts || (int64_t) out.bounds[(size_t) i + 1] - out.bounds[(size_t) head] > cap;
        if (i == 0 || full) {
            out.group.push_back(i);
            head = i;
        }
    }
    out.group.push_back(total);
}

}  // namespace basalt::prefill::fp4
