/* basalt_b200.h - C ABI of the B200 (sm_100a) mixture-of-experts layer: router, token-to-expert dispatch, grouped expert
 * gate-up / SwiGLU / down products over ggml block formats (NVFP4, Q6_K, IQ1_M), weighted combine with the shared expert.
 *
 * Every entry point is a drop-in for one operator of the Basalt engine's src/kernels / src/prefill layer; the comment above
 * each declaration cites the reference interface it replaces (paths inside the Basalt project).  basalt_shim.hpp wraps
 * these in inline C++ functions that carry the reference's exact signatures and exception behaviour.
 *
 * Conventions (the reference's, include/basalt/kernels/router.hpp:4-5, iq_kernels.hpp:77-95):
 *   - every data pointer is a DEVICE pointer; the caller owns all buffers including scratch, sized by the *_bytes helpers;
 *   - `stream` is a cudaStream_t passed as void*; nothing is allocated, no host read happens inside a call and, with a
 *     non-null stream, no synchronisation, so calls can be captured into a CUDA graph.  For the router family a null
 *     stream means "default stream, then synchronise" (router.cu:266); the expert, dispatch and combine family refuses
 *     a null stream (BSX_E_STREAM), as the reference's native family does (native_moe.cu:61);
 *   - a token's result does not depend on the number of tokens in the call or on its position;
 *   - return value: 0 = ok, negative = BSX_E_* argument error, positive = a cudaError_t from a launch.  Nothing exits
 *     or throws.  There is no CPU fallback: without a usable CUDA device every compute call fails with a CUDA error.
 */
#ifndef BASALT_B200_H
#define BASALT_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BSX_API __attribute__((visibility("default")))
#else
#define BSX_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
    BSX_OK = 0,
    BSX_E_GEOMETRY = -1,   /* unsupported shape (the reference throws std::invalid_argument / exits) */
    BSX_E_STREAM = -2,     /* null stream where the reference forbids it */
    BSX_E_TYPE = -3,       /* block format not supported */
    BSX_E_POINTER = -4,    /* null or misaligned pointer */
    BSX_E_LIMIT = -5,      /* a size beyond a documented fixed maximum */
    BSX_E_UNAVAILABLE = -6 /* the expert-parallel entries only: no NCCL library in the process, or NCCL refused the call */
};

/* gate functions of bsx_router_select */
enum {
    BSX_GATE_SQRT_SOFTPLUS = 0, /* RouterGate::SqrtSoftplus, router.hpp:14 */
    BSX_GATE_SIGMOID = 1,       /* RouterGate::Sigmoid */
    BSX_GATE_SOFTMAX = 2,       /* fp32 one-warp softmax top-k, src/models/qwen4exp/prefill/kernels.cu:351-390 */
    BSX_GATE_SOFTMAX_FAST = 3,  /* the same built with fast-math, src/models/qwen4exp/kernels/native_router.cu:44-99 */
    BSX_GATE_SOFTMAX_F64 = 4    /* fp64 exponentials and renormalisation, src/models/qwen4exp/kernels/router_top10.cu:57-174 */
};

/* ggml type ids of the block formats (include/basalt/ggml/ggml.h) */
enum { BSX_TYPE_Q5_0 = 6, BSX_TYPE_Q5_1 = 7, BSX_TYPE_Q8_0 = 8, BSX_TYPE_Q2_K = 10, BSX_TYPE_Q3_K = 11, BSX_TYPE_Q4_K = 12, BSX_TYPE_Q5_K = 13,
       BSX_TYPE_Q6_K = 14, BSX_TYPE_IQ2_XXS = 16, BSX_TYPE_IQ2_XS = 17, BSX_TYPE_IQ3_XXS = 18, BSX_TYPE_IQ1_S = 19, BSX_TYPE_IQ4_NL = 20,
       BSX_TYPE_IQ3_S = 21, BSX_TYPE_IQ2_S = 22, BSX_TYPE_IQ4_XS = 23, BSX_TYPE_IQ1_M = 29, BSX_TYPE_NVFP4 = 40, BSX_TYPE_Q2_0 = 42 };

/* activation / output element kinds */
enum { BSX_X_F32 = 0, BSX_X_BF16 = 1, BSX_X_Q8_1 = 2 };
enum { BSX_OUT_F32 = 0, BSX_OUT_BF16 = 1 };

#define BSX_MAX_HELD_TABS 4      /* ResidentTabs::kMax, include/basalt/kernels/route_lossy.hpp:20 */
#define BSX_TAIL_SKIP_MAX 128    /* kRouteTailSkipMax, route_lossy.hpp:33 */
#define BSX_PLAN_MAX_PAIRS 1024  /* moe_plan's limit, src/models/inkling2/kernels/ops.cu:493 */
#define BSX_PLAN_MAX_EXPERTS 2048 /* bsx_moe_plan[_shared]: the expert table lives in 48 KB of shared memory */

/* ---- a1: router logits.  Replaces the logits stage of basalt::kernels::router (include/basalt/kernels/router.hpp:30-32,
 * src/kernels/cuda/router.cu:49-146,233-253).  logits[t][e] = gate[e] . x[t]; x [T][H] fp32, gate [E][H] fp32 row-major,
 * logits [T][E] fp32.  Bit-identical to the reference: each sum runs as 256 column-strided fmaf chains, a 32-wide xor
 * butterfly per chain group, then the 8 partial sums in order.  E % 32 == 0, H % 128 == 0, H <= 8192. */
BSX_API int32_t bsx_router_logits(const float* x, const float* gate, int32_t T, int32_t E, int32_t H, float* logits, void* stream);

/* ---- a2-a4: selection and weights from logits.  Replaces basalt::kernels::router_select (router.hpp:36-37,
 * router.cu:170-229,255-267), qwen4exp::route / route_kernel (src/models/qwen4exp/prefill/kernels.cu:351-390,639-647),
 * native_router_top10[_multi] (include/basalt/models/qwen4exp/kernels/native_router.hpp:8-16) and router_top10
 * (src/models/qwen4exp/kernels/router_top10.cu:181-214).
 * Sigmoid / sqrt-softplus: s = gate(logit); the k largest s + bias (+ prior for experts a held table names, when
 * prior > 0) are chosen, the lower index winning a tie; ids come in rank order; weight = s / (sum of the chosen s + 1e-20)
 * * weight_scale.  Softmax kinds ignore bias, weight_scale, groups and prior: p = softmax over all experts, k argmax passes
 * (value desc, index asc), weight = p / max(sum of chosen p, 2^-14).
 * Group-limited selection (no counterpart in the reference; n_group <= 1 or topk_group >= n_group reduces to the plain
 * selection bit for bit): experts form n_group contiguous groups, a group scores the sum of its two largest s + bias, only
 * the topk_group best groups (lower index on a tie) can be chosen from.
 * E % 32 == 0, E <= 1024, 1 <= k <= 32 (k <= 16 for the non-softmax kinds, as the reference), n_group <= 32.
 * held_tabs: n_held (<= 4) device tables [E] of int32 (slot or -1), may be null. */
BSX_API int32_t bsx_router_select(const float* logits, const float* bias, int32_t T, int32_t E, int32_t k, int32_t gate_kind,
                          float weight_scale, int32_t n_group, int32_t topk_group, float prior,
                          const int32_t* const* held_tabs, int32_t n_held, int32_t* ids, float* weights, void* stream);

/* ---- a1+a2: basalt::kernels::router (router.hpp:30-32): bsx_router_logits then bsx_router_select on one stream. */
BSX_API int32_t bsx_router(const float* x, const float* gate, const float* bias, int32_t T, int32_t E, int32_t H, int32_t k,
                   int32_t gate_kind, float weight_scale, int32_t n_group, int32_t topk_group, float prior,
                   const int32_t* const* held_tabs, int32_t n_held, float* logits, int32_t* ids, float* weights, void* stream);

/* ---- a1 for prompt-sized batches: the gate product as a GEMM on the tcgen05 tensor cores.  Replaces the prompt path's router
 * GEMM (src/models/qwen4exp/prefill/routing.cpp:26, a cuBLAS bf16 product).  Same logits layout as bsx_router_logits; values
 * agree with it to ~1e-6 of |x||gate| (fp16 hi + lo operand images, fp32 accumulation), not bit for bit: use
 * bsx_router_logits where routing must not depend on the batch.  x fp32 or bf16 [T][H]; E % 32 == 0, H % 64 == 0.
 * scratch: bsx_router_logits_prefill_scratch_bytes(T, E, H), 256-byte aligned.  status: a device int32 the caller zeroes; bit 0
 * is set if a bounded wait inside the kernel ran out (the kernel then returns instead of hanging). */
BSX_API size_t bsx_router_logits_prefill_scratch_bytes(int64_t T, int32_t E, int32_t H);
BSX_API int32_t bsx_router_logits_prefill(const void* x, int32_t x_kind, const float* gate, int64_t T, int32_t E, int32_t H, float* logits,
                                          void* scratch, int32_t* status, void* stream);

/* ---- a1/a2 with bf16 activation rows (x_kind BSX_X_F32 or BSX_X_BF16; no counterpart in the reference, whose router reads
 * fp32 only: a bf16 row is widened exactly, then the same sums run, so the result equals bsx_router on the widened rows). */
BSX_API int32_t bsx_router_logits_x(const void* x, int32_t x_kind, const float* gate, int32_t T, int32_t E, int32_t H, float* logits,
                                    void* stream);
BSX_API int32_t bsx_router_x(const void* x, int32_t x_kind, const float* gate, const float* bias, int32_t T, int32_t E, int32_t H,
                             int32_t k, int32_t gate_kind, float weight_scale, int32_t n_group, int32_t topk_group, float prior,
                             const int32_t* const* held_tabs, int32_t n_held, float* logits, int32_t* ids, float* weights,
                             void* stream);

/* ---- a5: opt-in lossy tail skip.  Replaces basalt::kernels::route_tail_skip (include/basalt/kernels/route_lossy.hpp:58-59,
 * src/kernels/cuda/route_tail_skip.cu:14-53).  n_entries <= 128; rank outside 1..k-1 leaves the window untouched.
 * counts (optional, 3 x uint64 on the device): entries, entries no table holds, entries dropped (added to). */
BSX_API int32_t bsx_route_tail_skip(int32_t* ids, float* weights, const int32_t* const* held_tabs, int32_t n_held, int32_t n_entries,
                            int32_t k, int32_t rank, int32_t E, unsigned long long* counts, void* stream);

/* ---- a6: dispatch.  Replaces qwen4exp Group::group() (src/models/qwen4exp/prefill/routing.cpp:67-108), fused::group
 * (include/basalt/models/qwen4exp/prefill/moe_fused.hpp:46-50, moe_fused.cu:99-168,412-428), route_count
 * (prefill/kernels.cu:648-657) and the tile plans of fp4::plan / plan_blocks (include/basalt/prefill/moe_fp4.hpp:23-41).
 * ids [n_pairs] (pair i = token i / k, choice i % k) -> cnt [E], off [E+1] (exclusive prefix sum in expert-id order),
 * slot [n_pairs] (row of pair i; -1 for an id outside [0, E)), src [n_pairs] (token of each row).  The permutation is the
 * stable counting sort: pairs keep their order inside an expert (the host path's order; deterministic, no atomics on
 * row positions).  tiles (optional, with tile_rows > 0): int32 pairs {expert, first row} per tile of tile_rows rows,
 * experts ascending, n_tiles[0] = their number; capacity n_pairs / tile_rows + E entries.
 * scratch: bsx_dispatch_scratch_bytes(n_pairs, E).  E <= 1024. */
BSX_API size_t bsx_dispatch_scratch_bytes(int64_t n_pairs, int32_t E);
BSX_API int32_t bsx_dispatch(const int32_t* ids, int64_t n_pairs, int32_t k, int32_t E, int32_t* cnt, int32_t* off, int32_t* slot,
                     int32_t* src, int32_t tile_rows, int32_t* tiles, int32_t* n_tiles, void* scratch, void* stream);

/* ---- bsx_dispatch for callers that cannot hand over scratch memory.  (No counterpart in the reference.)
 * Some hosts of this library have given every byte of device memory to their own arenas before the first token, or run the
 * layer from a thread or a phase in which the CUDA allocator must not be entered; they have nowhere to get the count table
 * bsx_dispatch wants.  This entry point keeps that table inside the library instead: a 1 MiB array in device global memory
 * that every GPU holding the library carries until the process exits.  It allocates nothing, ever.
 * Limits: n_pairs <= 65536 and E <= 1024; a larger call is refused with BSX_E_LIMIT (use bsx_dispatch with your own scratch).
 * No tile list.  The first call on each device looks the array's address up (with that device current) and should be made
 * before any stream capture begins; later calls only launch (two host threads may make that first call at once).  All calls on a device share the one table, which keeps
 * whatever the previous call left (each call overwrites every entry it reads, so nothing has to start at zero): two calls
 * that overlap on the GPU - different streams, or a graph replayed while another call runs - race and give wrong rows.
 * Results are those of bsx_dispatch, bit for bit. */
BSX_API int32_t bsx_dispatch_static(const int32_t* ids, int64_t n_pairs, int32_t k, int32_t E, int32_t* cnt, int32_t* off,
                                    int32_t* slot, int32_t* src, void* stream);

/* ---- a6: apply the permutation.  out[r] = x[src[r]] for rows of row_bytes bytes (a multiple of 16); src < 0 gives a zero row.
 * Replaces gather_rows16 (src/models/qwen4exp/prefill/kernels.cu:430-437, :694-699). */
BSX_API int32_t bsx_gather_rows(const void* x, int64_t row_bytes, const int32_t* src, int64_t n_rows, void* out, void* stream);

/* ---- a6, decode-window form.  Replaces inkling2 moe_plan (src/models/inkling2/kernels/ops.cu:275-340,488-498): the experts
 * with pairs and a non-zero blob address become groups in ascending expert order (ptr[g], start[g]; start[n_groups] =
 * start[n_groups+1] = entries), entries inside a group in pair order, dst[entry] = pair index (the output row),
 * tok[entry] = pair / k.  T * k <= 1024 (BSX_E_LIMIT beyond), E <= 2048 (BSX_E_GEOMETRY beyond); ids outside [0, E) are skipped. */
BSX_API int32_t bsx_moe_plan(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table,
                     unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok, void* stream);

/* ---- a6 + a10: the decode-window plan with the shared expert as one more group.  Basalt runs a shared expert as a dense
 * gated MLP whose plan is "one group holding every token" (gated_mlp_plan_kernel, src/kernels/cuda/iq_kernels.cu:3414-3426);
 * here that group is appended to the routed groups so one bsx_experts_grouped call covers both: ptr[n_groups-1] =
 * shared_blob, its entries read token t and write output row T*k + t (t < T).  ptr / start need T*k + 3 slots, dst / tok
 * T*k + T.  shared_blob = 0 gives bsx_moe_plan.  The shared expert must have the routed experts' layout. */
BSX_API int32_t bsx_moe_plan_shared(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table,
                                    unsigned long long shared_blob, unsigned long long* ptr, int32_t* start, int32_t* n_groups,
                                    int32_t* dst, int32_t* tok, void* stream);

/* ---- a8: expert blob geometry.  Mirrors NativeExpertLayout / native_expert_layout / native_expert_supported /
 * native_expert_scratch_bytes (include/basalt/kernels/iq_kernels.hpp:51-75, src/kernels/cuda/iq_kernels.cu:3208-3242):
 * blob = [gate rows | up rows | down rows | NVFP4 only: fp32 {s_gate, s_up, s_down, 0}], raw ggml blocks. */
typedef struct bsx_expert_layout {
    int32_t gu_type, d_type, up_type;
    int32_t options;                   /* BSX_EXPERT_* bits below; 0 from bsx_expert_layout_init */
    int64_t n_embd, n_ff;
    uint64_t gu_row, d_row, up_row;    /* bytes per gate, down and up row */
    uint64_t up_off, down_off, bytes;  /* offsets inside the blob; its size */
    float swiglu_limit;                /* > 0: gate capped above at it, up clamped to +-it */
    float gate_softcap, up_softcap;    /* > 0 (both): h = cg tanh(g/cg) sigmoid(g) cu tanh(u/cu) */
    float reserved_f;
} bsx_expert_layout;

/* bsx_expert_layout.options, read by every bsx_experts_grouped* call that gets the layout (per call: nothing process-wide).
 * The stage bits mirror native_expert_set_mode's phase (include/basalt/kernels/iq_kernels.hpp:113-115), which the reference's
 * bench uses to time each half alone. */
enum {
    BSX_EXPERT_STAGE_ALL = 0,    /* gate/up + SwiGLU, then down */
    BSX_EXPERT_STAGE_GU = 1,     /* gate/up + SwiGLU only (h stays in the scratch) */
    BSX_EXPERT_STAGE_DOWN = 2,   /* down only, over the h a GU call left */
    BSX_EXPERT_STAGE_MASK = 3,
    BSX_EXPERT_PLAIN = 4         /* the warp-per-row kernels whatever the format (the second opinion of the parity tests) */
};

BSX_API int32_t bsx_expert_layout_init(int32_t gu_type, int32_t d_type, int32_t up_type, int64_t n_embd, int64_t n_ff,
                               float swiglu_limit, float gate_softcap, float up_softcap, bsx_expert_layout* layout);
BSX_API int32_t bsx_expert_supported(int32_t gu_type, int32_t d_type, int32_t up_type, int64_t n_embd, int64_t n_ff);
/* scratch for bsx_experts_grouped with up to cap_entries entries: the SwiGLU buffer plus the fp16 activation images of the
 * tensor-core path (the reference's helper takes (cap_entries, n_ff) only; this one needs n_embd as well, hence the layout) */
BSX_API size_t bsx_expert_scratch_bytes(const bsx_expert_layout* layout, int64_t cap_entries);

/* ---- a7: q8_1 activation rows.  Replaces basalt::kernels::quantize_q8_1_rows (iq_kernels.hpp:23, iq_kernels.cu:2471-2503):
 * per 32 values fp16 d = amax / 127, fp16 sum, 32 int8 codes.  n_cols % 32 == 0.  Bit-identical to the reference. */
BSX_API int32_t bsx_quantize_q8_1_rows(const float* x, int64_t n_rows, int64_t n_cols, void* y, void* stream);

/* ---- a9/a10: grouped decode experts.  Replaces native_expert_grouped / native_expert_grouped_clamped / gated_mlp_clamped
 * (iq_kernels.hpp:77-98, iq_kernels.cu:3304-3447).  Group g's blob is at device address grp_ptr[g]; its entries
 * [grp_start[g], grp_start[g+1]) read activation row ent_tok[e] of x and write row ent_dst[e] of out (n_embd values,
 * unweighted): out = s_down W_down ( silu(s_gate W_gate x) * (s_up W_up x) ).  n_groups is read on the device;
 * cap_groups / cap_entries bound the launch.  x_kind: BSX_X_F32 ([rows][n_embd] floats), BSX_X_BF16, or BSX_X_Q8_1 (the
 * reference's activation blocks, decoded as d * q).  Unlike the reference, activations and the SwiGLU output are NOT
 * re-quantised to int8: products accumulate in fp32 on exactly decoded weights, so results sit within ~1e-5 relative
 * of the dequantised fp32 reference instead of the reference kernels' ~1e-2.
 * scratch: bsx_expert_scratch_bytes(layout, cap_entries).  A shared expert is one group holding every token. */
BSX_API int32_t bsx_experts_grouped(const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                            const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                            int64_t cap_entries, const void* x, int32_t x_kind, void* scratch, void* out, int32_t out_kind,
                            void* stream);

/* bsx_experts_grouped for a caller that knows how many rows x has (every ent_tok value is below n_x_rows): the fp16 images
 * the tensor-core path makes of the activations are then built once per row instead of once per entry.  Same results.
 * No counterpart in the reference (its q8_1 rows are made by the caller, once per token, for the same reason). */
BSX_API int32_t bsx_experts_grouped_rows(const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                         const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                         int64_t cap_entries, const void* x, int32_t x_kind, int32_t n_x_rows, void* scratch, void* out,
                                         int32_t out_kind, void* stream);

/* ---- a10: a dense gated MLP (a shared expert) on n_tok rows: row t of out is token t's unweighted output.  Replaces
 * gated_mlp_clamped / gated_mlp_scratch_bytes (iq_kernels.hpp:93-98, iq_kernels.cu:3413-3447): the one-group plan is built on
 * the device, then the grouped experts run.  The SwiGLU limit rides in the layout.  scratch: bsx_gated_mlp_scratch_bytes. */
BSX_API size_t bsx_gated_mlp_scratch_bytes(const bsx_expert_layout* layout, int64_t cap_tok);
BSX_API int32_t bsx_gated_mlp(const bsx_expert_layout* layout, const void* blob, int32_t n_tok, int64_t cap_tok, const void* x,
                              int32_t x_kind, void* scratch, void* out, int32_t out_kind, void* stream);

/* ---- a9 on the block-scaled FP4 tensor cores (tcgen05.mma kind::mxf4nvf4): the weight stream with no decode arithmetic.
 * bsx_expert_pack rewrites one all-NVFP4 blob (n_embd % 256 == 0, n_ff % 256 == 0), once, into planes - codes row-major,
 * UE4M3 scales in the order the tensor core's scale copy reads, the fp32 tail - the same bytes in another order
 * (cf. Basalt's own load-time planes, include/basalt/kernels/nvfp4_planes.hpp:6-20); bsx_expert_packed_bytes gives the size
 * (0: layout not covered), packed must be 256-byte aligned.  bsx_experts_grouped_packed is bsx_experts_grouped_rows over
 * packed blobs (grp_ptr[g] = a packed blob): activations enter as four FP4 terms per row (relative error ~1e-4, against
 * the 2e-3 bar and the ~1e-2 of the reference's int8 rounding), accumulation is fp32 in tensor memory.
 * scratch: bsx_experts_packed_scratch_bytes(layout, cap_entries), 256-byte aligned.  status: a device int32 the caller
 * zeroes; bit 0 is set if a bounded wait inside a kernel ran out (the kernel returns instead of hanging). */
BSX_API size_t bsx_expert_packed_bytes(const bsx_expert_layout* layout);
BSX_API int32_t bsx_expert_pack(const bsx_expert_layout* layout, const void* blob, void* packed, void* stream);
BSX_API size_t bsx_experts_packed_scratch_bytes(const bsx_expert_layout* layout, int64_t cap_entries);
/* The x images of bsx_experts_grouped_packed made ahead of the call - they need only x, not the routing, so a caller can run
 * them on another stream beside router and plan: rows 0 .. n_x_rows - 1 of x into `scratch` (the same scratch and
 * cap_entries the grouped call will get).  The grouped call is then told so by a NEGATIVE n_x_rows (-n_x_rows). */
BSX_API int32_t bsx_experts_packed_x_images(const bsx_expert_layout* layout, const void* x, int32_t x_kind, int32_t n_x_rows, int64_t cap_entries,
                                            void* scratch, void* stream);
BSX_API int32_t bsx_experts_grouped_packed(const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                           const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                           int64_t cap_entries, const void* x, int32_t x_kind, int32_t n_x_rows, void* scratch, void* out,
                                           int32_t out_kind, int32_t* status, void* stream);

/* ---- a11 / a12: prompt-sized grouped experts on the tcgen05 tensor cores, ggml blobs in place: NVFP4 (replaces fp4::run_group /
 * run_experts, include/basalt/prefill/moe_fp4.hpp:43-113, src/prefill/moe_fp4.cu:604-687) and the K- / I-quant formats Q6_K and
 * IQ1_M (replaces the int8 MMQ path mmq::quantize -> Context::run -> swiglu -> Context::run, include/basalt/prefill/moe_mmq.hpp:37-125,
 * src/prefill/moe_mmq.cu:246-356; gate and up of one format, n_embd and n_ff multiples of 256): for the expert-sorted rows of a bsx_dispatch
 * (off, src, and its tile list with tile_rows = 128), gate/up through the rows' tokens, SwiGLU, down; dm[row] (fp32,
 * unweighted, row = dispatch slot) is what bsx_combine reads.  blob_table[e] = device address of expert e's blob.
 * x: fp32 or bf16 [n_tokens][n_embd].  Weights are decoded exactly to fp16 and multiplied by fp16 activations with fp32
 * accumulation (kind::f16), so results sit ~2e-4 from the dequantised fp32 reference.  n_embd % 128 == 0, n_ff % 64 == 0.
 * status: a device int32 the caller zeroes; a kernel that gives up on a bounded wait sets bit 0 there instead of hanging.
 * scratch: bsx_experts_prefill_scratch_bytes(layout, n_tokens, cap_rows); cap_tiles >= the tile count, <= 65535. */
BSX_API size_t bsx_experts_prefill_scratch_bytes(const bsx_expert_layout* layout, int64_t n_tokens, int64_t cap_rows);
BSX_API int32_t bsx_experts_prefill(const bsx_expert_layout* layout, const unsigned long long* blob_table, const int32_t* off,
                                    const int32_t* src, const int32_t* tiles, const int32_t* n_tiles, int64_t cap_tiles, int64_t cap_rows,
                                    const void* x, int32_t x_kind, int64_t n_tokens, void* scratch, float* dm, int32_t* status, void* stream);

/* The tile list bsx_dispatch makes, from row bounds alone - for a caller that grouped its rows itself (Group::group(),
 * src/models/qwen4exp/prefill/routing.cpp:67-108, fp4::plan_blocks, include/basalt/prefill/moe_fp4.hpp:38-41): off[E + 1]
 * expert row bounds on the device -> tiles {expert, first row} per tile_rows rows of an expert, in expert order, and their
 * count.  tiles must hold off[E] / tile_rows + E entries.  E <= 1024. */
BSX_API int32_t bsx_tiles_from_bounds(const int32_t* off, int32_t E, int32_t tile_rows, int32_t* tiles, int32_t* n_tiles, void* stream);

/* ---- a11 / a12 as the engine's prompt path drives them: a group of up to 16 consecutive experts of a layer, each given by its
 * blob's address on the HOST side (blobs[i], i < n), over rows the caller grouped by expert.  Replaces fp4::run_group /
 * run_experts and the Group they take (include/basalt/prefill/moe_fp4.hpp:82-113; call site
 * src/models/qwen4exp/prefill/expert_fp4.cpp:10-30).  bounds: n + 1 ABSOLUTE row bounds on the device (expert i's rows are
 * [bounds[i], bounds[i+1]) of dm and of row_token); row_token[row] = the row's token; cap_rows >= the layer's row count (the
 * largest bound any group of the layer has); x, dm, status as for bsx_experts_prefill.  The blob addresses travel as kernel
 * arguments: no copy, no synchronisation, capturable.  scratch: bsx_experts_prefill_group_scratch_bytes, 256-byte aligned.
 * bsx_unit_offsets: out[0] = 0, out[j+1] = sum over i <= j of ceil(rows_i / unit_rows) for n <= 1024 segments of `bounds` -
 * fp4::plan (unit 64) and plan_blocks (units 64 and 128), moe_fp4.hpp:23-41.  bsx_rebase_bounds: out[i] = bounds[i] - bounds[0],
 * i <= n (fp4::rebase). */
BSX_API size_t bsx_experts_prefill_group_scratch_bytes(const bsx_expert_layout* layout, int64_t n_tokens, int64_t cap_rows);
BSX_API int32_t bsx_experts_prefill_group(const bsx_expert_layout* layout, const void* const* blobs, int32_t n, const int32_t* bounds,
                                          const int32_t* row_token, int64_t cap_rows, const void* x, int32_t x_kind, int64_t n_tokens,
                                          void* scratch, float* dm, int32_t* status, void* stream);
BSX_API int32_t bsx_unit_offsets(const int32_t* bounds, int32_t n, int32_t unit_rows, int32_t* out, void* stream);
BSX_API int32_t bsx_rebase_bounds(const int32_t* bounds, int32_t n, int32_t* out, void* stream);

/* ---- a11 on the block-scaled FP4 tensor cores: bsx_experts_prefill over blobs packed by bsx_expert_pack (blob_table[e] = a
 * packed blob, 0 = held elsewhere).  Activations enter as four FP4 terms per row (x rows and the SwiGLU rows alike), so the
 * rows sit ~2e-4 from the dequantised fp32 reference; nothing is decoded on the way to the tensor core.  n_expert = the
 * length of off minus one.  scratch: bsx_experts_prefill_packed_scratch_bytes(layout, n_tokens, cap_rows), 256-byte aligned.
 * Tiles as for bsx_experts_prefill (bsx_dispatch with tile_rows = 128). */
BSX_API size_t bsx_experts_prefill_packed_scratch_bytes(const bsx_expert_layout* layout, int64_t n_tokens, int64_t cap_rows);
BSX_API int32_t bsx_experts_prefill_packed(const bsx_expert_layout* layout, const unsigned long long* blob_table, const int32_t* off,
                                           const int32_t* src, const int32_t* tiles, const int32_t* n_tiles, int64_t cap_tiles, int64_t cap_rows,
                                           const void* x, int32_t x_kind, int64_t n_tokens, int32_t n_expert, void* scratch, float* dm,
                                           int32_t* status, void* stream);

/* ---- a13: weighted combine.  Replaces native_moe_combine[_multi] (include/basalt/models/qwen4exp/kernels/native_moe.hpp:5-15,
 * native_moe.cu:36-85), moe_combine (src/models/qwen4exp/prefill/kernels.cu:438-449,705-709) and weighted_sum_tokens
 * (src/models/deepseek41/prefill_ffn.cu:33-50).  y[t] = fma chain over j < k of weights[t][j] * rows[slot[t*k+j]] in j
 * order starting from 0, then + shared[t] (as one more fma with sigmoid(shared_gate[t]) when shared_gate is given).
 * slot may be null (row = t*k+j, the decode form); a slot < 0 contributes nothing.  A gather, never a scatter-add:
 * bit-stable from run to run.  rows [n_rows][H] fp32, y [T][H] fp32, H % 4 == 0. */
BSX_API int32_t bsx_combine(const float* rows, const int32_t* slot, const float* weights, const float* shared, const float* shared_gate,
                    int32_t T, int32_t k, int32_t H, float* y, void* stream);

/* ---- a13 + the step after the layer: bsx_combine with the residual stream's row added last, y[t] = (combine) + residual[t] as one
 * more rounded fp32 add - the weighted sum and the residual write in one pass over the rows instead of a T x H round trip
 * through HBM (Basalt fuses the same pair in its per-model finish kernels: moe_finish, src/models/inkling2/kernels/glue.cu:507-546
 * called at src/models/inkling2/session.cpp:706-716).  residual [T][H] fp32, may be null (= bsx_combine); y may alias it. */
BSX_API int32_t bsx_combine_residual(const float* rows, const int32_t* slot, const float* weights, const float* shared, const float* shared_gate,
                                     const float* residual, int32_t T, int32_t k, int32_t H, float* y, void* stream);

/* ---- a2-a4 + a6 together: bsx_router_select followed by bsx_moe_plan_shared (shared_blob = 0: bsx_moe_plan), for decode
 * windows (T * k <= 1024).  Up to 16 tokens it is one launch: one block chooses every token's experts and goes straight on to
 * the plan, the ids never leaving shared memory in between; wider windows keep the selection spread over the SMs and take two
 * launches.  Either way ids, weights, groups and entries carry the bits of the two separate calls.  Gate kinds SOFTMAX,
 * SIGMOID and SQRT_SOFTPLUS (with groups); BSX_E_TYPE for the others (use the separate calls); no held tables / prior. */
BSX_API int32_t bsx_route_plan(const float* logits, const float* bias, int32_t T, int32_t E, int32_t k, int32_t gate_kind, float weight_scale,
                               int32_t n_group, int32_t topk_group, const unsigned long long* blob_table, unsigned long long shared_blob,
                               int32_t* ids, float* weights, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok,
                               void* stream);

/* ---- a1-a13 in one call: the whole decode-window step of a resident layer - (input RMS norm,) router logits, selection,
 * plan, grouped experts with the shared expert, weighted combine, (+ residual row).  It is the sequence Basalt's layer loop
 * issues call by call (src/models/inkling2/session.cpp:680-716; src/models/deepseek41/ops_kernels.cpp:797,931,964), for a C or
 * C++ caller that wants the step without a host layer of its own.  Every kernel after the first is a programmatic dependent
 * launch (as Basalt's decode chain: include/basalt/kernels/pdl.hpp:20-32), selection + plan (+ the packed kernels' pass list)
 * are one kernel for windows of up to 16 tokens.  Nothing is allocated or read back; the call can be captured into a CUDA graph.
 * desc: layout = the routed experts' (and, with `packed`, the shared expert's); shared_layout = the shared expert's when its
 * ggml blob has another layout (n_embd = 0: same as layout); packed = blobs are bsx_expert_pack planes (all-NVFP4).
 * x [n_tokens][n_embd] fp32 or bf16; y [n_tokens][n_embd] fp32; residual [n_tokens][n_embd] fp32 or null; n_tokens <= max_tokens,
 * max_tokens * top_k <= 1024.  workspace: bsx_moe_layer_workspace_bytes(desc, max_tokens), 256-byte aligned, the same max_tokens
 * on every call.  status: a device int32 the caller zeroes (bit 0: a bounded wait inside a kernel ran out); required with packed.
 * bsx_moe_layer_views: where the step leaves its routing inside the workspace (logits, ids, weights, groups), for a caller that
 * wants to look at them. */
enum { BSX_LAYER_NO_PDL = 1 };   /* flags: plain launches (for comparison) */
typedef struct bsx_moe_layer_desc {
    bsx_expert_layout layout, shared_layout;
    int32_t n_expert, top_k, gate_kind, n_group, topk_group, packed, flags;
    float weight_scale, norm_eps;
    const float* gate;                     /* [n_expert][n_embd] fp32 */
    const float* bias;                     /* [n_expert] fp32 or null */
    const unsigned long long* blob_table;  /* [n_expert] device addresses of the experts' blobs; 0 = not held here */
    unsigned long long shared_blob;        /* 0 = no shared expert */
    const float* norm_w;                   /* [n_embd] fp32: the layer's input RMS norm weights, or null (rows arrive normed) */
} bsx_moe_layer_desc;
typedef struct bsx_moe_layer_views_t {
    float* logits;
    int32_t* ids;
    float* weights;
    int32_t *n_groups, *grp_start, *ent_dst, *ent_tok;
    float* rows;
} bsx_moe_layer_views_t;
BSX_API size_t bsx_moe_layer_workspace_bytes(const bsx_moe_layer_desc* desc, int32_t max_tokens);
BSX_API int32_t bsx_moe_layer_views(const bsx_moe_layer_desc* desc, int32_t max_tokens, void* workspace, bsx_moe_layer_views_t* views);
BSX_API int32_t bsx_moe_layer(const bsx_moe_layer_desc* desc, const void* x, int32_t x_kind, int32_t n_tokens, int32_t max_tokens,
                              const float* residual, void* workspace, float* y, int32_t* status, void* stream);

/* ---- expert parallelism (no counterpart in the reference, which moves rows between cards through host memory:
 * include/basalt/models/qwen4exp/kernels/dec_moe.hpp:1-11).  bsx_plan_groups turns a dispatch (cnt, off, src over ALL experts)
 * into the groups of the experts this device holds (blob_table[e] != 0): ptr/start/n_groups as bsx_moe_plan makes them,
 * ent_dst[entry] = the entry's dispatch row, ent_tok[entry] = its token; arrays sized for every row.  E <= 1024.
 * bsx_combine_partial is bsx_combine restricted to the pairs whose expert id lies in [e_lo, e_hi) - one rank's share of
 * y, to be summed across ranks (reduce-scatter). */
BSX_API int32_t bsx_plan_groups(const int32_t* cnt, const int32_t* off, const int32_t* src, int32_t E, const unsigned long long* blob_table,
                                unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* ent_dst, int32_t* ent_tok, void* stream);
/* bsx_plan_groups plus one more group for a shared expert every device holds: its entries are tokens tok_lo .. tok_lo +
 * tok_n - 1 (this device's own tokens), their rows follow the dispatch's rows (row off[E] + t); arrays sized for that. */
BSX_API int32_t bsx_plan_groups_shared(const int32_t* cnt, const int32_t* off, const int32_t* src, int32_t E, const unsigned long long* blob_table,
                                       unsigned long long shared_blob, int32_t tok_lo, int32_t tok_n, unsigned long long* ptr, int32_t* start,
                                       int32_t* n_groups, int32_t* ent_dst, int32_t* ent_tok, void* stream);
BSX_API int32_t bsx_combine_partial(const float* rows, const int32_t* slot, const float* weights, const int32_t* ids, int32_t e_lo,
                                    int32_t e_hi, int32_t T, int32_t k, int32_t H, float* y, void* stream);
/* The decode-sized expert-parallel step in two launches around the experts.  bsx_ep_plan: from every gathered token's routing
 * (n_pairs ids in pair order; or in per-rank blocks of pairs_per_block ids, block_stride values apart - what an all-gather of
 * [ids | weights] buffers leaves - with pairs_per_block > 0) straight to the groups of the experts held here (blob_table[e] != 0):
 * ptr / start / n_groups as bsx_moe_plan, ent_dst[entry] = the pair's index (its row), ent_tok[entry] = pair / k; plus, with
 * shared_blob, one group over tokens tok_lo .. tok_lo + tok_n - 1 whose rows follow the pairs' rows (row n_pairs + i).  The
 * order of the entries inside a group is not fixed (every entry writes its own row, so results do not depend on it).
 * n_pairs <= BSX_EP_PLAN_MAX_PAIRS.  bsx_combine_partial_ep: bsx_combine_partial over that layout (row = pair index) with the
 * shared rows of tokens tok_lo .. added on their owner, so that the reduce-scatter that follows yields finished rows.
 * replicated (optional, [E] bytes on the device, the same table on every rank): hot experts of which EVERY rank holds a copy
 * (blob_table[e] != 0 everywhere) - the B200 form of Basalt's expert residency tiers (include/basalt/core/expert_tier.hpp:1-10:
 * experts never leave HBM here, the popular ones are simply held more than once).  A pair naming a replicated expert is run
 * by the rank that owns its token (tokens tok_lo .. tok_lo + tok_n - 1), so popular experts stop loading one rank with
 * everybody's rows; every pair still has exactly one rank in the plan and in the partial sums. */
#define BSX_EP_PLAN_MAX_PAIRS 8192
BSX_API int32_t bsx_ep_plan(const int32_t* ids, int64_t n_pairs, int32_t k, int32_t pairs_per_block, int32_t block_stride, int32_t E,
                            const unsigned long long* blob_table, unsigned long long shared_blob, int32_t tok_lo, int32_t tok_n,
                            const uint8_t* replicated, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* ent_dst,
                            int32_t* ent_tok, void* stream);
BSX_API int32_t bsx_combine_partial_ep(const float* rows, const float* weights, const int32_t* ids, int32_t tokens_per_block, int32_t block_stride,
                                       int32_t e_lo, int32_t e_hi, int32_t T, int32_t k, int32_t H, const float* shared, int32_t tok_lo, int32_t tok_n,
                                       const uint8_t* replicated, float* y, void* stream);

/* The whole decode-window step of an expert-parallel layer in one call, on the caller's NCCL communicator (one process per GPU;
 * no counterpart in the reference, see above).  Rank r of the communicator holds the layer's experts e_lo .. e_lo + n_local - 1
 * (blob_table[e] != 0 for those, for the replicated ones and for nothing else), the router weights and the shared expert; every
 * rank calls with the same n_tokens rows of its own.  Sequence: all-gather of the rows (on side_stream when given, beside the
 * router; ev_fork / ev_join are two events of the caller's that order the two streams), router, all-gather of [ids | weights],
 * bsx_ep_plan, grouped experts, bsx_combine_partial_ep, reduce-scatter.  y [n_tokens][n_embd] fp32: this rank's tokens, equal to
 * bsx_moe_layer on one GPU holding every expert up to the order of the fp32 sum over the ranks.
 * comm: an ncclComm_t.  NCCL is looked up at run time in the process (libnccl.so.2), never linked: bsx_ep_available() says
 * whether it was found; without it the call returns BSX_E_UNAVAILABLE.  n_tokens is the same on every rank and on every call
 * with one workspace (fixed-size collectives), world * n_tokens * top_k <= BSX_EP_PLAN_MAX_PAIRS.  Nothing is allocated or read
 * back; the call can be captured into a CUDA graph (NCCL's kernels included).  No kernel waits on another rank: a rank that
 * does not call shows up as NCCL's timeout on the host. */
typedef struct bsx_ep_layer_desc {
    bsx_expert_layout layout;
    int32_t n_expert, top_k, gate_kind, n_group, topk_group, packed;
    int32_t e_lo, n_local, n_replicas, reserved;
    float weight_scale, reserved_f;
    const float* gate;                     /* [n_expert][n_embd] fp32 */
    const float* bias;                     /* [n_expert] fp32 or null */
    const unsigned long long* blob_table;  /* [n_expert] device addresses; 0 = held by another rank */
    unsigned long long shared_blob;        /* 0 = no shared expert */
    const uint8_t* replicated;             /* [n_expert] device bytes, 1 = every rank holds a copy; or null */
} bsx_ep_layer_desc;
BSX_API int32_t bsx_ep_available(void);
BSX_API size_t bsx_ep_layer_workspace_bytes(const bsx_ep_layer_desc* desc, int32_t n_tokens, int32_t world);
BSX_API int32_t bsx_ep_layer_views(const bsx_ep_layer_desc* desc, int32_t n_tokens, int32_t world, void* workspace, bsx_moe_layer_views_t* views);
BSX_API int32_t bsx_ep_layer(const bsx_ep_layer_desc* desc, void* comm, const void* x, int32_t x_kind, int32_t n_tokens, void* workspace, float* y,
                             int32_t* status, void* stream, void* side_stream, void* ev_fork, void* ev_join);

/* ---- the step before the layer: the RMS norm of the layer's input rows (weights w, any offset folded), as fp32 rows xn (what
 * the router reads) and / or bf16 rows act; either may be null, not both.  Replaces wgemm::norm_pack
 * (include/basalt/kernels/window_gemm.hpp:36-40, src/kernels/cuda/window_gemm.cu:75-112) with its summation order, so the rows
 * carry the reference's bits.  x [T][K] fp32 or bf16 (x_kind BSX_X_F32 / BSX_X_BF16).
 * bsx_norm_pack_images: the same norm plus the FP4 images bsx_experts_grouped_packed reads, in one launch - rows 0 ..
 * n_x_rows - 1 into `scratch` exactly as bsx_experts_packed_x_images(xn) would leave them (the grouped call is then given
 * -n_x_rows); xn is required, act optional. */
BSX_API int32_t bsx_norm_pack(const void* x, int32_t x_kind, const float* w, float eps, int64_t K, int32_t T, void* act, float* xn,
                              void* stream);
BSX_API int32_t bsx_norm_pack_images(const bsx_expert_layout* layout, const void* x, int32_t x_kind, const float* w, float eps,
                                     int32_t n_x_rows, int64_t cap_entries, void* scratch, float* xn, void* act, void* stream);

/* ---- the model file's `experts.layout` text (host only): which ggml types each layer's expert blobs have, how large a blob is
 * and where the layer's n_expert blobs start inside the `experts` section.  Replaces expert_layout_load_text / ExpertLayout
 * (include/basalt/kernels/cpu/expert_layout.hpp:17-35,60-67; src/kernels/cpu/expert_layout.cpp:133-203) with the same rules:
 * a "# experts vN: ... (n_expert E, total B)" header (a version above 7 is refused; E replaces the caller's n_expert), one
 * "layer gu_type d_type offset blob_bytes [up_type from v7]" line per layer, further columns ignored, blob_bytes checked
 * against the formats' geometry at (n_embd, n_ff), layers contiguous from offset 0.  rows: n_layers entries, filled by layer
 * id.  Every ggml format the reference's loader takes parses (its block geometry is known here), also those this library
 * has no kernels for yet: rows[l].kernels says which layers can run.  err (may be null): the reason in words.  Returns
 * BSX_OK, or BSX_E_TYPE (newer version, a type without a dot product, a gate / up / down mix the loader refuses) /
 * BSX_E_GEOMETRY (empty text, malformed line, rows that are not whole blocks, size mismatch, a missing layer). */
typedef struct bsx_layout_row {
    int32_t gu_type, d_type, up_type;
    int32_t kernels;                 /* 1: this library has kernels for the layer's formats (bsx_expert_supported) */
    uint64_t offset, blob_bytes;     /* of the layer's first blob inside the experts section; bytes per blob */
} bsx_layout_row;
typedef struct bsx_layout_info {
    int32_t version, reserved;       /* the header's version (0: none given) */
    int64_t n_layers, n_expert;
    uint64_t max_blob, total;        /* the largest blob; the experts section's size */
} bsx_layout_info;
BSX_API int32_t bsx_layout_parse(const char* text, size_t len, int64_t n_layers, int64_t n_expert, int64_t n_embd, int64_t n_ff,
                                 float swiglu_limit, bsx_layout_row* rows, bsx_layout_info* info, char* err, size_t err_cap);

/* ---- device self-check helpers (host-side; no GPU needed): the block decoders compiled for the host, for tests. */
BSX_API int32_t bsx_host_decode_row(int32_t type, const void* row, float* y, int64_t n);
BSX_API size_t bsx_row_bytes(int32_t type, int64_t n);
BSX_API const char* bsx_version(void);

#ifdef __cplusplus
}
#endif
#endif /* BASALT_B200_H */
