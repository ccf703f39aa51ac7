// layer.cu - one call for the whole decode-window step of a resident MoE layer: (input norm,) router logits, selection, plan,
// grouped experts with the shared expert, weighted combine (+ residual row).
//
// This is the step Basalt's layer loops issue call by call (src/models/inkling2/session.cpp:680-716: router -> moe_plan ->
// native_expert_grouped -> moe_finish), behind one entry point so that a C or C++ caller gets it without the host layer above
// the C ABI, and with the launch gaps the reference hides the same way: every kernel after the first is a programmatic
// dependent launch (include/basalt/kernels/pdl.hpp:20-32), and selection, plan and the packed kernels' pass list are one kernel.
// Nothing is allocated, nothing is read back and nothing synchronises: the caller owns the workspace and may capture the call
// into a CUDA graph.
#include <cstring>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"
#include "pdl.cuh"
#include "plan.cuh"

namespace bsx {

int32_t route_plan_launch(const float* logits, const float* bias, int32_t T, int32_t E, int32_t k, int32_t gate_kind, float weight_scale,
                          int32_t n_group, int32_t topk_group, const unsigned long long* blob_table, unsigned long long shared_blob, int32_t* ids,
                          float* weights, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok, PassRec* items,
                          int* n_items, cudaStream_t st);

namespace {

size_t al256(size_t v) { return (v + 255) & ~(size_t) 255; }

bool same_layout(const bsx_expert_layout& a, const bsx_expert_layout& b) { return memcmp(&a, &b, sizeof a) == 0; }

// where everything lives inside the workspace
struct Carve {
    float* logits;
    int32_t* ids;
    float* w;
    unsigned long long* ptr;
    int32_t *start, *n_groups, *dst, *tok;
    float *rows, *xn, *s_out;
    uint8_t *scratch, *s_scratch;
    unsigned long long* s_ptr;
    int32_t *s_start, *s_one, *s_iota;
    size_t bytes;
    int64_t cap_rows;
    bool fused_shared, own_shared;
};

Carve carve(const bsx_moe_layer_desc& d, int32_t T, void* ws) {
    Carve c;
    memset(&c, 0, sizeof c);
    const int64_t E = d.n_expert, k = d.top_k, H = d.layout.n_embd, n = (int64_t) T * k;
    c.fused_shared = d.shared_blob != 0ull && (d.packed || d.shared_layout.n_embd == 0 || same_layout(d.shared_layout, d.layout));
    c.own_shared = d.shared_blob != 0ull && !c.fused_shared;
    c.cap_rows = n + (c.fused_shared ? T : 0);
    uint8_t* p = static_cast<uint8_t*>(ws);
    size_t at = 0;
    auto take = [&](size_t bytes) {
        uint8_t* r = p ? p + at : nullptr;
        at += al256(bytes);
        return r;
    };
    c.logits = reinterpret_cast<float*>(take((size_t) T * E * 4));
    c.ids = reinterpret_cast<int32_t*>(take((size_t) n * 4));
    c.w = reinterpret_cast<float*>(take((size_t) n * 4));
    c.ptr = reinterpret_cast<unsigned long long*>(take((size_t) (n + 3) * 8));
    c.start = reinterpret_cast<int32_t*>(take((size_t) (n + 3) * 4));
    c.n_groups = reinterpret_cast<int32_t*>(take(16));
    c.dst = reinterpret_cast<int32_t*>(take((size_t) c.cap_rows * 4));
    c.tok = reinterpret_cast<int32_t*>(take((size_t) c.cap_rows * 4));
    c.rows = reinterpret_cast<float*>(take((size_t) c.cap_rows * H * 4));
    if (d.norm_w) c.xn = reinterpret_cast<float*>(take((size_t) T * H * 4));
    c.scratch = take(d.packed ? bsx_experts_packed_scratch_bytes(&d.layout, c.cap_rows) : bsx_expert_scratch_bytes(&d.layout, c.cap_rows));
    if (c.own_shared) {
        c.s_out = reinterpret_cast<float*>(take((size_t) T * H * 4));
        // the decode kernels' scratch, or (windows of 16+ tokens) the prompt kernels': the larger of the two
        const size_t dec = bsx_expert_scratch_bytes(&d.shared_layout, T), pre = bsx_experts_prefill_group_scratch_bytes(&d.shared_layout, T, T);
        c.s_scratch = take(dec > pre ? dec : pre);
        c.s_ptr = reinterpret_cast<unsigned long long*>(take(16));
        c.s_start = reinterpret_cast<int32_t*>(take(16));
        c.s_one = reinterpret_cast<int32_t*>(take(16));
        c.s_iota = reinterpret_cast<int32_t*>(take((size_t) T * 4));
    }
    c.bytes = at;
    return c;
}

// the one-group plan of a shared expert with a layout of its own: every token, rows in token order
__global__ void own_shared_plan_kernel(unsigned long long blob, int n_tok, unsigned long long* ptr, int32_t* start, int32_t* one, int32_t* iota) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        ptr[0] = blob;
        start[0] = 0;
        start[1] = n_tok;
        start[2] = n_tok;
        one[0] = 1;
    }
    for (int i = threadIdx.x; i < n_tok; i += blockDim.x) iota[i] = i;
}

int32_t check_desc(const bsx_moe_layer_desc* d, int32_t max_tokens) {
    if (!d) return BSX_E_POINTER;
    if (d->n_expert < 32 || d->n_expert % 32 || d->n_expert > 1024 || d->top_k < 1 || d->top_k > 32 || max_tokens < 1) return BSX_E_GEOMETRY;
    if ((int64_t) max_tokens * d->top_k > BSX_PLAN_MAX_PAIRS) return BSX_E_LIMIT;
    if (!bsx_expert_supported(d->layout.gu_type, d->layout.d_type, d->layout.up_type, d->layout.n_embd, d->layout.n_ff)) return BSX_E_TYPE;
    if (d->packed && !bsx_expert_packed_bytes(&d->layout)) return BSX_E_TYPE;
    if (d->gate_kind < BSX_GATE_SQRT_SOFTPLUS || d->gate_kind > BSX_GATE_SOFTMAX_F64) return BSX_E_GEOMETRY;
    return BSX_OK;
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_moe_layer_workspace_bytes(const bsx_moe_layer_desc* d, int32_t max_tokens) {
    if (check_desc(d, max_tokens) != BSX_OK) return 0;
    return carve(*d, max_tokens, nullptr).bytes + 256;
}

extern "C" int32_t bsx_moe_layer_views(const bsx_moe_layer_desc* d, int32_t max_tokens, void* workspace, bsx_moe_layer_views_t* v) {
    const int32_t rc = check_desc(d, max_tokens);
    if (rc != BSX_OK) return rc;
    if (!aligned(workspace, 256) || !v) return BSX_E_POINTER;
    const Carve c = carve(*d, max_tokens, workspace);
    v->logits = c.logits;
    v->ids = c.ids;
    v->weights = c.w;
    v->n_groups = c.n_groups;
    v->grp_start = c.start;
    v->ent_dst = c.dst;
    v->ent_tok = c.tok;
    v->rows = c.rows;
    return BSX_OK;
}

extern "C" int32_t bsx_moe_layer(const bsx_moe_layer_desc* d, const void* x, int32_t x_kind, int32_t n_tokens, int32_t max_tokens,
                                 const float* residual, void* workspace, float* y, int32_t* status, void* stream) {
    if (!stream) return BSX_E_STREAM;
    int32_t rc = check_desc(d, max_tokens);
    if (rc != BSX_OK) return rc;
    if (n_tokens < 0 || n_tokens > max_tokens) return BSX_E_GEOMETRY;
    if (n_tokens == 0) return BSX_OK;
    if (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16) return BSX_E_GEOMETRY;
    if (!d->gate || !d->blob_table || !aligned(x, 16) || !aligned(workspace, 256) || !aligned(y, 16) || (d->packed && !status)) return BSX_E_POINTER;
    const cudaStream_t st = (cudaStream_t) stream;
    const bsx_expert_layout& L = d->layout;
    const Carve c = carve(*d, max_tokens, workspace);
    const int32_t T = n_tokens, E = d->n_expert, k = d->top_k, H = (int32_t) L.n_embd;
    const int64_t n = (int64_t) T * k, rows_now = n + (c.fused_shared ? T : 0);
    // every kernel after the first is a programmatic dependent launch; the first follows whatever the caller ran before
    PdlScope pdl((d->flags & BSX_LAYER_NO_PDL) == 0, 1);

    const void* xe = x;          // what the experts and the router read
    int32_t xe_kind = x_kind;
    if (d->norm_w) {
        // the step before the layer: RMS norm of the input rows (fp32 rows), on the packed path together with their FP4 images
        rc = d->packed ? bsx_norm_pack_images(&L, x, x_kind, d->norm_w, d->norm_eps, T, c.cap_rows, c.scratch, c.xn, nullptr, stream)
                       : bsx_norm_pack(x, x_kind, d->norm_w, d->norm_eps, H, T, nullptr, c.xn, stream);
        if (rc != BSX_OK) return rc;
        xe = c.xn;
        xe_kind = BSX_X_F32;
    } else if (d->packed) {
        rc = experts_packed_x_images(L, x, x_kind, T, c.cap_rows, c.scratch, st);
        if (rc != BSX_OK) return rc;
        pdl_state().late_wait = true;   // the logits read x, not the images: the two kernels run side by side
    }
    rc = bsx_router_logits_x(xe, xe_kind, d->gate, T, E, H, c.logits, stream);
    pdl_state().late_wait = false;
    if (rc != BSX_OK) return rc;
    PassRec* items = nullptr;
    int* n_items = nullptr;
    if (d->packed) experts_packed_pass_list(c.scratch, c.cap_rows, L.n_embd, L.n_ff, &items, &n_items);
    const unsigned long long fused_blob = c.fused_shared ? d->shared_blob : 0ull;
    rc = route_plan_launch(c.logits, d->bias, T, E, k, d->gate_kind, d->weight_scale, d->n_group, d->topk_group, d->blob_table, fused_blob, c.ids, c.w,
                           c.ptr, c.start, c.n_groups, c.dst, c.tok, items, n_items, st);
    bool have_passes = rc == BSX_OK && d->packed;
    if (rc == BSX_E_TYPE) {      // a gate kind only the stand-alone selection kernels know
        rc = bsx_router_select(c.logits, d->bias, T, E, k, d->gate_kind, d->weight_scale, d->n_group, d->topk_group, 0.f, nullptr, 0, c.ids, c.w, stream);
        if (rc == BSX_OK) rc = bsx_moe_plan_shared(c.ids, T, k, E, d->blob_table, fused_blob, c.ptr, c.start, c.n_groups, c.dst, c.tok, stream);
    }
    if (rc != BSX_OK) return rc;
    const int64_t cap_groups = (n < E ? n : E) + (c.fused_shared ? 1 : 0);
    if (d->packed) {
        ExpertArgs a;
        a.L = L;
        a.grp_ptr = c.ptr;
        a.grp_start = c.start;
        a.n_groups = c.n_groups;
        a.ent_dst = c.dst;
        a.ent_tok = c.tok;
        a.cap_groups = cap_groups;
        a.cap_entries = c.cap_rows;
        a.x = xe;
        a.x_kind = xe_kind;
        a.h = reinterpret_cast<float*>(c.scratch);
        a.out = c.rows;
        a.out_kind = BSX_OUT_F32;
        a.n_x_rows = T;
        a.grid = nullptr;
        rc = experts_grouped_packed(a, status, st, true, have_passes);
    } else {
        rc = bsx_experts_grouped_rows(&L, c.ptr, c.start, c.n_groups, c.dst, c.tok, cap_groups, rows_now, xe, xe_kind, T, c.scratch, c.rows, BSX_OUT_F32, stream);
    }
    if (rc != BSX_OK) return rc;
    const float* shared = c.fused_shared ? c.rows + (size_t) n * H : nullptr;
    if (c.own_shared) {
        launch_k(own_shared_plan_kernel, dim3(1), dim3(128), 0, st, d->shared_blob, (int) T, c.s_ptr, c.s_start, c.s_one, c.s_iota);
        rc = launch_status();
        if (rc != BSX_OK) return rc;
        // A shared expert sees every token.  From 16 tokens on, an NVFP4 one goes through the prompt-sized kernel (one pass over the
        // blob for the whole window; the decode kernels take 4 or 8 entries a pass and would stream it several times).  K- and
        // I-quant blobs stay on the decode kernels: the prompt kernel's decoders read those formats byte by byte and are slower.
        rc = BSX_E_TYPE;
        if (T >= 16 && status != nullptr && d->shared_layout.gu_type == kTypeNVFP4 && bsx_experts_prefill_group_scratch_bytes(&d->shared_layout, T, T) != 0) {
            const void* blob1[1] = {reinterpret_cast<const void*>((uintptr_t) d->shared_blob)};
            rc = bsx_experts_prefill_group(&d->shared_layout, blob1, 1, c.s_start, c.s_iota, T, xe, xe_kind, T, c.s_scratch, c.s_out, status, stream);
        }
        if (rc == BSX_E_TYPE || rc == BSX_E_GEOMETRY)
            rc = bsx_experts_grouped(&d->shared_layout, c.s_ptr, c.s_start, c.s_one, c.s_iota, c.s_iota, 1, T, xe, xe_kind, c.s_scratch, c.s_out, BSX_OUT_F32, stream);
        if (rc != BSX_OK) return rc;
        shared = c.s_out;
    }
    return bsx_combine_residual(c.rows, nullptr, c.w, shared, nullptr, residual, T, k, H, y, stream);
}
