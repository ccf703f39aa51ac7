// ep_layer.cu - the decode-window step of an expert-parallel MoE layer behind one C entry point: this rank's experts are a
// contiguous block of the layer's (plus replicas of hot experts and the shared expert), every rank brings its own tokens, and the
// rows travel by two NCCL collectives on the caller's communicator.
//
//   1. all-gather of the rank's token rows - on the caller's side stream, beside the router (the exchange needs no routing);
//   2. router logits + selection of the rank's own tokens; ids and weight bits land in one buffer;
//   3. all-gather of that buffer;
//   4. bsx_ep_plan: every gathered pair whose expert is held here -> the groups of the local experts (+ the shared expert's group
//      over the rank's own tokens, + the pass list of the packed kernels);
//   5. the grouped experts over the gathered rows;
//   6. bsx_combine_partial_ep: each token's local pairs summed (the token's owner adds the shared row);
//   7. reduce-scatter (sum) of the fp32 partial rows onto the tokens' owners.
//
// The Basalt engine has no counterpart: it keeps every expert of a layer on one card, and where it spreads experts over cards it
// moves rows through mapped host memory and doorbells (include/basalt/models/qwen4exp/kernels/dec_moe.hpp:1-11,
// src/core/peer_experts.cpp:420-548).  Its correctness argument carries over - an expert gives the same rows on whichever card
// holds it (include/basalt/core/peer_experts.hpp:11-12) - and the cross-rank sum is NCCL's, so a token's row equals the
// single-GPU layer's to fp32 rounding.
//
// NCCL is not a link-time dependency of this library: the four functions used are looked up in the libnccl the process has
// loaded (or loads by its soname) the first time an entry here runs, so a single-GPU user never needs it.  Nothing here waits
// on another rank from inside a kernel; a rank that never joins shows up as NCCL's own timeout on the host.
#include <dlfcn.h>

#include <atomic>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "experts.cuh"
#include "pdl.cuh"
#include "plan.cuh"

namespace bsx {
namespace {

// the slice of NCCL's public C API this file calls (nccl.h: ncclAllGather, ncclReduceScatter, ncclCommCount, ncclCommUserRank)
using nccl_comm = void*;
enum : int { kNcclInt32 = 2, kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0 };
struct NcclApi {
    int (*all_gather)(const void*, void*, size_t, int, nccl_comm, cudaStream_t) = nullptr;
    int (*reduce_scatter)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
    int (*comm_count)(nccl_comm, int*) = nullptr;
    int (*comm_rank)(nccl_comm, int*) = nullptr;
    bool ok = false;
};

const NcclApi& nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // the library the process already uses (a Python host has loaded its own copy; RTLD_NOLOAD finds it by soname), else the
        // system's
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
        api.reduce_scatter = reinterpret_cast<decltype(api.reduce_scatter)>(dlsym(h, "ncclReduceScatter"));
        api.comm_count = reinterpret_cast<decltype(api.comm_count)>(dlsym(h, "ncclCommCount"));
        api.comm_rank = reinterpret_cast<decltype(api.comm_rank)>(dlsym(h, "ncclCommUserRank"));
        api.ok = api.all_gather && api.reduce_scatter && api.comm_count && api.comm_rank;
    });
    return api;
}

size_t al256e(size_t v) { return (v + 255) & ~(size_t) 255; }

struct EpCarve {
    uint8_t* x_all;          // [W T][H] rows of every rank
    float* logits;           // [T][E]
    int32_t* route;          // [ids T k | weight bits T k] of the rank's own tokens
    int32_t* route_all;      // the ranks' buffers, one after the other
    unsigned long long* ptr;
    int32_t *start, *n_groups, *ent_dst, *ent_tok;
    float *rows, *y_part;
    uint8_t* scratch;
    size_t bytes;
    int64_t cap_rows;
};

EpCarve ep_carve(const bsx_ep_layer_desc& d, int32_t T, int32_t W, void* ws) {
    EpCarve c;
    memset(&c, 0, sizeof c);
    const int64_t E = d.n_expert, k = d.top_k, H = d.layout.n_embd, n = (int64_t) W * T * k;
    c.cap_rows = n + (d.shared_blob ? T : 0);
    uint8_t* p = static_cast<uint8_t*>(ws);
    size_t at = 0;
    auto take = [&](size_t bytes) {
        uint8_t* r = p ? p + at : nullptr;
        at += al256e(bytes);
        return r;
    };
    c.x_all = take((size_t) W * T * H * 4);        // sized for fp32 rows; bf16 rows use half of it
    c.logits = reinterpret_cast<float*>(take((size_t) T * E * 4));
    c.route = reinterpret_cast<int32_t*>(take((size_t) 2 * T * k * 4));
    c.route_all = reinterpret_cast<int32_t*>(take((size_t) W * 2 * T * k * 4));
    c.ptr = reinterpret_cast<unsigned long long*>(take((size_t) (E + 3) * 8));
    c.start = reinterpret_cast<int32_t*>(take((size_t) (E + 3) * 4));
    c.n_groups = reinterpret_cast<int32_t*>(take(16));
    c.ent_dst = reinterpret_cast<int32_t*>(take((size_t) c.cap_rows * 4));
    c.ent_tok = reinterpret_cast<int32_t*>(take((size_t) c.cap_rows * 4));
    c.rows = reinterpret_cast<float*>(take((size_t) c.cap_rows * H * 4));
    c.y_part = reinterpret_cast<float*>(take((size_t) W * T * H * 4));
    c.scratch = take(d.packed ? bsx_experts_packed_scratch_bytes(&d.layout, c.cap_rows) : bsx_expert_scratch_bytes(&d.layout, c.cap_rows));
    c.bytes = at;
    return c;
}

int32_t ep_check(const bsx_ep_layer_desc* d, int32_t max_tokens, int32_t world) {
    if (!d) return BSX_E_POINTER;
    if (world < 1 || world > 64 || max_tokens < 1) return BSX_E_GEOMETRY;
    if (d->n_expert < 32 || d->n_expert % 32 || d->n_expert > 1024 || d->top_k < 1 || d->top_k > 32) return BSX_E_GEOMETRY;
    if (d->n_local < 0 || d->n_local > d->n_expert || d->e_lo < 0 || d->e_lo + d->n_local > d->n_expert || d->n_replicas < 0) return BSX_E_GEOMETRY;
    if ((int64_t) world * max_tokens * d->top_k > BSX_EP_PLAN_MAX_PAIRS) return BSX_E_LIMIT;
    if (!bsx_expert_supported(d->layout.gu_type, d->layout.d_type, d->layout.up_type, d->layout.n_embd, d->layout.n_ff)) return BSX_E_TYPE;
    if (d->packed && !bsx_expert_packed_bytes(&d->layout)) return BSX_E_TYPE;
    if (d->gate_kind < BSX_GATE_SQRT_SOFTPLUS || d->gate_kind > BSX_GATE_SOFTMAX_F64) return BSX_E_GEOMETRY;
    return BSX_OK;
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" int32_t bsx_ep_available(void) { return nccl_api().ok ? 1 : 0; }

extern "C" size_t bsx_ep_layer_workspace_bytes(const bsx_ep_layer_desc* d, int32_t max_tokens, int32_t world) {
    if (ep_check(d, max_tokens, world) != BSX_OK) return 0;
    return ep_carve(*d, max_tokens, world, nullptr).bytes + 256;
}

extern "C" int32_t bsx_ep_layer_views(const bsx_ep_layer_desc* d, int32_t max_tokens, int32_t world, void* workspace, bsx_moe_layer_views_t* v) {
    const int32_t rc = ep_check(d, max_tokens, world);
    if (rc != BSX_OK) return rc;
    if (!aligned(workspace, 256) || !v) return BSX_E_POINTER;
    const EpCarve c = ep_carve(*d, max_tokens, world, workspace);
    v->logits = c.logits;
    v->ids = c.route;
    v->weights = reinterpret_cast<float*>(c.route + (size_t) max_tokens * d->top_k);
    v->n_groups = c.n_groups;
    v->grp_start = c.start;
    v->ent_dst = c.ent_dst;
    v->ent_tok = c.ent_tok;
    v->rows = c.rows;
    return BSX_OK;
}

extern "C" int32_t bsx_ep_layer(const bsx_ep_layer_desc* d, void* comm, const void* x, int32_t x_kind, int32_t n_tokens, void* workspace, float* y,
                                int32_t* status, void* stream, void* side_stream, void* ev_fork, void* ev_join) {
    if (!stream) return BSX_E_STREAM;
    const NcclApi& nc = nccl_api();
    if (!nc.ok) return BSX_E_UNAVAILABLE;
    if (!comm) return BSX_E_POINTER;
    int W = 0, rank = -1;
    if (nc.comm_count(comm, &W) != 0 || nc.comm_rank(comm, &rank) != 0) return BSX_E_UNAVAILABLE;
    const int32_t T = n_tokens;
    int32_t rc = ep_check(d, T, W);
    if (rc != BSX_OK) return rc;
    if (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16) return BSX_E_GEOMETRY;
    if (!d->gate || !d->blob_table || !aligned(x, 16) || !aligned(workspace, 256) || !aligned(y, 16) || (d->packed && !status)) return BSX_E_POINTER;
    if (side_stream && (!ev_fork || !ev_join)) return BSX_E_POINTER;
    const cudaStream_t st = (cudaStream_t) stream;
    const cudaStream_t side = side_stream ? (cudaStream_t) side_stream : st;
    const bsx_expert_layout& L = d->layout;
    const EpCarve c = ep_carve(*d, T, W, workspace);
    const int32_t E = d->n_expert, k = d->top_k, H = (int32_t) L.n_embd;
    const int64_t n = (int64_t) W * T * k;
    const bool shared = d->shared_blob != 0ull;

    // 1. every rank's rows - beside the router
    if (side != st) {
        if (cudaEventRecord((cudaEvent_t) ev_fork, st) != cudaSuccess) return launch_status();
        if (cudaStreamWaitEvent(side, (cudaEvent_t) ev_fork, 0) != cudaSuccess) return launch_status();
    }
    if (nc.all_gather(x, c.x_all, (size_t) T * H, x_kind == BSX_X_BF16 ? kNcclBfloat16 : kNcclFloat32, comm, side) != 0) return BSX_E_UNAVAILABLE;
    if (side != st && cudaEventRecord((cudaEvent_t) ev_join, side) != cudaSuccess) return launch_status();
    // 2. the rank's own routing: ids, then weight bits, in one buffer
    int32_t* ids = c.route;
    float* w = reinterpret_cast<float*>(c.route + (size_t) T * k);
    {
        PdlScope pdl(true, 1);   // logits follow the caller's work; the selection is a programmatic dependent launch
        rc = bsx_router_x(x, x_kind, d->gate, d->bias, T, E, H, k, d->gate_kind, d->weight_scale, d->n_group, d->topk_group, 0.f, nullptr, 0, c.logits, ids, w,
                          stream);
    }
    if (rc != BSX_OK) return rc;
    // 3. everyone's routing
    if (nc.all_gather(c.route, c.route_all, (size_t) 2 * T * k, kNcclInt32, comm, st) != 0) return BSX_E_UNAVAILABLE;
    // 4. the gathered pairs -> this rank's groups
    const int32_t own_n = (shared || d->replicated) ? T : 0;
    rc = bsx_ep_plan(c.route_all, n, k, T * k, 2 * T * k, E, d->blob_table, d->shared_blob, rank * T, own_n, d->replicated, c.ptr, c.start, c.n_groups,
                     c.ent_dst, c.ent_tok, stream);
    if (rc != BSX_OK) return rc;
    if (side != st && cudaStreamWaitEvent(st, (cudaEvent_t) ev_join, 0) != cudaSuccess) return launch_status();
    // 5. the local experts over the gathered rows (a pair's output lands on row = its index; shared rows after them).  The first
    // kernel of the chain follows a collective and an event of another stream, so it is a plain launch; the ones behind it
    // (gate/up, SwiGLU images, down, partial combine) are programmatic dependent launches of each other.
    PdlScope pdl(true, 1);
    const int64_t cap_groups = (int64_t) d->n_local + d->n_replicas + (shared ? 1 : 0);
    if (d->packed) {
        rc = bsx_experts_grouped_packed(&L, c.ptr, c.start, c.n_groups, c.ent_dst, c.ent_tok, cap_groups, c.cap_rows, c.x_all, x_kind, W * T, c.scratch, c.rows,
                                        BSX_OUT_F32, status, stream);
    } else {
        rc = bsx_experts_grouped_rows(&L, c.ptr, c.start, c.n_groups, c.ent_dst, c.ent_tok, cap_groups, c.cap_rows, c.x_all, x_kind, W * T, c.scratch, c.rows,
                                      BSX_OUT_F32, stream);
    }
    if (rc != BSX_OK) return rc;
    // 6. each token's local pairs, 7. summed over the ranks onto the token's owner
    rc = bsx_combine_partial_ep(c.rows, reinterpret_cast<const float*>(c.route_all + (size_t) T * k), c.route_all, T, 2 * T * k, d->e_lo, d->e_lo + d->n_local,
                                W * T, k, H, shared ? c.rows + (size_t) n * H : nullptr, rank * T, own_n, d->replicated, c.y_part, stream);
    if (rc != BSX_OK) return rc;
    if (nc.reduce_scatter(c.y_part, y, (size_t) T * H, kNcclFloat32, kNcclSum, comm, st) != 0) return BSX_E_UNAVAILABLE;
    return launch_status();
}
