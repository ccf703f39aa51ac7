// experts_nvf4.cu - decode-sized grouped experts on the block-scaled FP4 tensor cores: tcgen05.mma kind::mxf4nvf4 reads the
// NVFP4 codes and their UE4M3 block scales exactly as they are stored, so the weight stream needs no arithmetic at all and
// the kernel is what the workload is: a copy from HBM into shared memory at the pace of the memory system.
//
// What makes that possible:
//  * An NVFP4 block IS the tensor core's operand: 16 E2M1 codes share one UE4M3 scale (scale_vec::4X), element 2i of a
//    16-value sub-block in the low nibble of byte i and element 2i + 1 in the high nibble.  ggml stores value b and value
//    b + 8 in byte b (include/basalt/ggml/ggml_common.h:146-156), i.e. the same thing up to a fixed permutation inside the
//    sub-block, which the activation side simply shares.  ggml's decode (value = doubled-E2M1 x scale / 2,
//    src/kernels/cpu/ggml/ggml_quants.c:1397-1422) equals E2M1 x UE4M3, the product the hardware forms.
//  * The only thing in the way is the layout: ggml interleaves 4 scale bytes with 32 code bytes (36-byte blocks), which
//    no 16-byte copy can split.  bsx_expert_pack rewrites a blob once, at load time, into 18 KB blocks (the codes of 128 rows x
//    256 columns as the swizzled image of a stage, then their scales in the 32-lane x 4-word order tcgen05.cp wants:
//    nvf4.cuh), the same bytes in another order - Basalt does the like for its own
//    FP4 kernels (include/basalt/kernels/nvfp4_planes.hpp:6-20).
//  * Activations must be FP4 too.  One FP4 term is worth ~3.3 bits, far from the 2e-3 bar; so a row goes in as FOUR terms
//    (each term quantises the residual the terms before it left, with its own block scales): relative error ~1e-4.  The
//    terms are extra columns of the small operand - 8 entries x 4 terms = 32 columns - which costs nothing here because
//    the tensor core idles anyway: the kernel is bound by the weight stream.
//
// Kernel: persistent CTAs, one per SM, static round-robin over work units (pass of <= 8 entries of one expert, block of
// 2 x 128 weight rows: 128 gate rows with their 128 up rows, or 256 down rows).  Warp 0 issues tcgen05.cp (scales ->
// tensor memory) and the MMAs (M = 128 weight rows, N = 32 columns, K = 64 per instruction); warp 1 streams the weights (one
// lane, two 18 KB bulk copies a stage, completion in bytes on the stage's mbarrier), warp 2 the activation images (cp.async)
// into stages of 256 columns (5-stage ring, continuous across units); warps 3-6 are the
// epilogue (thread = TMEM lane = weight row: sums each entry's four term columns, applies row and tail scales, SwiGLU for
// gate/up, stores coalesced).  Two accumulator sets in tensor memory let the epilogue of one unit overlap the stream of
// the next.  Every mbarrier wait is time-bounded and reports through a status word.
//
// Semantics: Basalt's native_expert_grouped (include/basalt/kernels/iq_kernels.hpp:77-92) without its int8 rounding of x, h.
#include <atomic>
#include <cuda_fp16.h>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"
#include "norm.cuh"
#include "nvf4.cuh"
#include "pdl.cuh"
#include "plan.cuh"
#include "tc5.cuh"

namespace bsx {
namespace {

constexpr int kATile = 128 * 128;          // one operand tile of a stage: 128 rows x 128 bytes (256 columns of codes)
constexpr int kSFTile = 4 * 512;           // 4 K-steps x (32 lanes x 4 words)
constexpr int kThreadsF = 32 * 7;          // MMA warp, weight loader warp, activation loader warp, four epilogue warps
constexpr uint32_t kTmemCols = 512;
constexpr int kOffSFA0 = kATile, kOffA1 = kATile + kSFTile, kOffSFA1 = kOffA1 + kATile, kOffB = kOffSFA1 + kSFTile;
constexpr int kEntNarrow = kPassEntries, kEntWide = 2 * kPassEntries;

// The kernel in two widths.  ENT = entries per pass: 8 (the MMA's N = 32 columns; what a decode window on one GPU needs, where an
// expert sees a handful of tokens) or 16 (N = 64; for expert-parallel steps, where the gathered tokens of all ranks give every local
// expert tens of entries and each pass streams the expert's blocks again - from L2 after the first, but at half the passes).
template <int ENT>
struct FG {
    static constexpr int kCols = kTermsF * ENT;         // MMA N
    static constexpr int kBTile = kCols * 128;
    // a stage: [tile 0 codes | tile 0 scales | tile 1 codes | tile 1 scales | activation codes | activation scales]
    static constexpr int kOffSFB = kOffB + kBTile;
    static constexpr int kStage = kOffSFB + kSFTile;    // 43,008 or 47,104 bytes: multiples of 1024
    static constexpr int kStages = ENT == kEntNarrow ? 5 : 4;
    static constexpr size_t kSmem = 1024 + (size_t) kStages * kStage + 256;
    // tensor-memory columns: two accumulator sets of (D0, D1) x kCols columns, then per stage 16 columns each for SFA0, SFA1, SFB
    static constexpr uint32_t kAccCols = 2 * kCols, kTmemSF = 2 * kAccCols;
    // kind::mxf4nvf4, scale_vec::4X: E2M1 x E2M1, UE4M3 scales (bit 23 = 0), both K-major, N = kCols, M = 128
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t) (kCols >> 3) << 17) | ((uint32_t) (128 >> 4) << 24);
    static_assert(kStage % 1024 == 0 && kSmem <= 227 * 1024 && kTmemSF + kStages * 48 <= kTmemCols, "stage geometry");
};

enum { FMODE_GU = 0, FMODE_DOWN = 1 };

// a pass (PassRec, plan.cuh): up to ENT consecutive entries [eb, eb + ntok) of one group, with the group's blob - everything a
// stream kernel needs about it in one 16-byte load

size_t al256f(size_t v) { return (v + 255) & ~(size_t) 255; }

// ---------------------------------------------------------------- packing
// One thread per (matrix row, 64-column block): 36 bytes in, 32 code bytes and one scale word out.  A scale byte keeps its
// low 7 bits and 0x7F becomes 0, which is what the ggml decoder does with them (ggml_quants.c:1397-1406).
__global__ void __launch_bounds__(256) pack_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, bsx_expert_layout L) {
    const int64_t H = L.n_embd, I = L.n_ff;
    const PackedGeom g = packed_geom(H, I);
    const int64_t n_gu = I * (H / 64), n_d = H * (I / 64);
    const int64_t i = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (i == 0) {
        for (int k = 0; k < 4; ++k) reinterpret_cast<float*>(out + g.tail)[k] = reinterpret_cast<const float*>(in + L.bytes - 16)[k];
    }
    if (i >= 2 * n_gu + n_d) return;
    const int mat = i < n_gu ? 0 : (i < 2 * n_gu ? 1 : 2);
    const int64_t j = i - (mat == 0 ? 0 : (mat == 1 ? n_gu : 2 * n_gu));
    const int64_t K = mat == 2 ? I : H;
    const int64_t nb = K / 64, row = j / nb, blk = j - row * nb;
    const uint8_t* src = in + (mat == 0 ? 0 : (mat == 1 ? (size_t) L.up_off : (size_t) L.down_off)) +
                         (size_t) row * (mat == 0 ? L.gu_row : (mat == 1 ? L.up_row : L.d_row)) + (size_t) blk * 36;
    const uint32_t* w = reinterpret_cast<const uint32_t*>(src);
    uint32_t sc = w[0] & 0x7F7F7F7Fu;
#pragma unroll
    for (int b = 0; b < 4; ++b)
        if (((sc >> (8 * b)) & 0xFFu) == 0x7Fu) sc &= ~(0xFFu << (8 * b));
    const int64_t tile = row >> 7, chunk = blk >> 2;
    const int r = (int) (row & 127), step = (int) (blk & 3);
    uint8_t* block = out + (mat == 0 ? g.gate : (mat == 1 ? g.up : g.down)) + (size_t) (tile * (K / 256) + chunk) * kBlockF;
    // the K-step's 32 code bytes are 16-byte pieces 2 step and 2 step + 1 of the row's 128 bytes
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int piece = 2 * step + h;
        uint32_t* dst = reinterpret_cast<uint32_t*>(block + (r >> 3) * 1024 + (r & 7) * 128 + ((piece ^ (r & 7)) << 4));
#pragma unroll
        for (int k = 0; k < 4; ++k) dst[k] = w[1 + 4 * h + k];
    }
    reinterpret_cast<uint32_t*>(block + 128 * 128 + step * 512)[(r & 31) * 4 + (r >> 5)] = sc;
}

// ---------------------------------------------------------------- FP4 activation images
// TPR threads per activation row (32, 128 or 256: a thread per 16-value sub-block where the row allows): the row times a
// power of two (largest magnitude into [2^7, 2^8), so block scales sit well inside UE4M3's range) as kTermsF FP4 terms.
// Term t of a sub-block: scale = the smallest UE4M3 value s with 6 s >= the largest residual, codes = rn(residual / s),
// residual -= code value x s.  Layout: codes [row][term][K / 2] bytes with ggml's nibble order (byte b of a sub-block =
// values b and b + 8), scales [row][term][K / 16] bytes, inv[row].  FROM_H = false: rows of x (kind x_kind) - row i of x
// when the caller gave the number of x rows, else the row of entry i; true: row e of the SwiGLU output h.  The last block
// lists the passes (up to pass_entries consecutive entries of one group).
template <bool FROM_H, int TPR>
__global__ void __launch_bounds__(256) prep_fp4_kernel(ExpertArgs a, uint8_t* __restrict__ codes, uint8_t* __restrict__ sfs, float* __restrict__ inv,
                                                        PassRec* __restrict__ items, int* __restrict__ n_items, int pass_entries) {
    // pass_entries = 0: the pass list exists already (and a kernel launched after this one may be reading it): leave it alone
    if (pass_entries == 0 && blockIdx.x == gridDim.x - 1) return;
    // The kernel after the h images is the down stage, whose weight loader may run ahead (it reads constants): letting it be
    // scheduled before this kernel's own wait means its blocks start on each SM as the gate/up stage's block there exits.
    if (FROM_H) pdl_launch_dependents();
    pdl_wait();
    if (!FROM_H) pdl_launch_dependents();
    const int ng = min(*a.n_groups, (int) a.cap_groups);
    const int total = min(a.grp_start[ng], (int) a.cap_entries);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int sh[8];
    __shared__ float shf[8];
    if (blockIdx.x == gridDim.x - 1) {
        __shared__ int s_base;
        if (threadIdx.x == 0) s_base = 0;
        __syncthreads();
        for (int g0 = 0; g0 < ng; g0 += 256) {
            const int g = g0 + threadIdx.x;
            const int s0 = g < ng ? a.grp_start[g] : 0;
            const int cnt = g < ng ? max(0, min(a.grp_start[g + 1], (int) a.cap_entries) - s0) : 0;
            const int np = (cnt + pass_entries - 1) / pass_entries;
            int x = np;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(kFull, x, o);
                if (lane >= o) x += y;
            }
            if (lane == 31) sh[warp] = x;
            __syncthreads();
            int before = s_base;
            for (int w = 0; w < warp; ++w) before += sh[w];
            for (int p = 0; p < np; ++p) {
                PassRec r;
                r.blob = a.grp_ptr[g];
                r.eb = s0 + p * pass_entries;
                r.ntok = min(pass_entries, cnt - p * pass_entries);
                items[before + x - np + p] = r;
            }
            __syncthreads();
            if (threadIdx.x == 255) s_base = before + x;
            __syncthreads();
        }
        if (threadIdx.x == 0) n_items[0] = s_base;
        return;
    }
    constexpr int kRowsPerBlock = 256 / TPR;
    const int i = blockIdx.x * kRowsPerBlock + (int) threadIdx.x / TPR;   // image row
    const int n_img = FROM_H ? total : (a.n_x_rows > 0 ? a.n_x_rows : total);
    const bool live = i < n_img;
    const int64_t K = FROM_H ? a.L.n_ff : a.L.n_embd;
    const int64_t row = !live ? 0 : (FROM_H ? (int64_t) i : (a.n_x_rows > 0 ? (int64_t) i : (int64_t) a.ent_tok[i]));
    fp4_image_row<TPR>(FROM_H ? (const void*) a.h : a.x, FROM_H ? BSX_X_F32 : a.x_kind, row, K, live, i, codes, sfs, inv, shf);
}

// rows 0 .. n_rows - 1 of x alone (no plan needed): for a caller that makes the images beside the routing
template <int TPR>
__global__ void __launch_bounds__(256) x_images_kernel(const void* __restrict__ x, int kind, int n_rows, int64_t K, uint8_t* __restrict__ codes,
                                                        uint8_t* __restrict__ sfs, float* __restrict__ inv) {
    __shared__ float shf[8];
    pdl_wait();
    pdl_launch_dependents();
    const int i = blockIdx.x * (256 / TPR) + (int) threadIdx.x / TPR;
    fp4_image_row<TPR>(x, kind, i < n_rows ? i : 0, K, i < n_rows, i, codes, sfs, inv, shf);
}

// The RMS norm of row blockIdx.x (norm.cuh: the reference's order, so xn carries its bits) and the FP4 images of the normed
// row, one launch: the block reads back the fp32 row it has just written (still in L1 / L2) instead of a second kernel
// fetching it from HBM.
template <bool BF16>
__global__ void __launch_bounds__(kNormThreads) norm_images_kernel(const void* __restrict__ x, const float* __restrict__ w, float eps, int64_t K,
                                                                   uint16_t* act, float* xn, uint8_t* __restrict__ codes,
                                                                   uint8_t* __restrict__ sfs, float* __restrict__ inv) {
    __shared__ float red[kNormThreads / 32];
    __shared__ float shf[kNormThreads / 32];
    pdl_wait();
    pdl_launch_dependents();
    norm_row<BF16>(x, w, eps, K, blockIdx.x, act, xn, red);
    fp4_image_row<kNormThreads>(xn, BSX_X_F32, blockIdx.x, K, true, (int) blockIdx.x, codes, sfs, inv, shf);
}

template <bool FROM_H>
void launch_prep(const ExpertArgs& a, int64_t rows, int64_t K, uint8_t* codes, uint8_t* sfs, float* inv, PassRec* items, int* n_items, int pass_entries,
                 cudaStream_t st) {
    const int64_t n_sb = K / 16;
    if (n_sb <= 32) launch_k(prep_fp4_kernel<FROM_H, 32>, dim3((unsigned) ((rows + 7) / 8 + 1)), dim3(256), 0, st, a, codes, sfs, inv, items, n_items, pass_entries);
    else if (n_sb <= 128) launch_k(prep_fp4_kernel<FROM_H, 128>, dim3((unsigned) ((rows + 1) / 2 + 1)), dim3(256), 0, st, a, codes, sfs, inv, items, n_items, pass_entries);
    else launch_k(prep_fp4_kernel<FROM_H, 256>, dim3((unsigned) (rows + 1)), dim3(256), 0, st, a, codes, sfs, inv, items, n_items, pass_entries);
}

// ---------------------------------------------------------------- the stream kernel
struct StreamArgs {
    ExpertArgs e;
    const uint8_t* codes;     // activation images
    const uint8_t* sfs;
    const float* inv;
    const PassRec* items;
    const int* n_items;
    int32_t* status;
    int early_weights;        // the pass list was complete before the kernel ahead of this one started: the weight loader need not wait
};

__device__ __forceinline__ uint64_t sf_desc(uint32_t addr) {   // 32 rows x 16 bytes, 8-row groups 128 bytes apart, no swizzle
    return (uint64_t) ((addr & 0x3FFFFu) >> 4) | ((uint64_t) (128 >> 4) << 16) | ((uint64_t) (128 >> 4) << 32) | ((uint64_t) 1 << 46);
}

template <int MODE, int ENT>
__global__ void __launch_bounds__(kThreadsF, 1) nvf4_stream_kernel(StreamArgs sa) {
    using G = FG<ENT>;
    constexpr int kStagesF = G::kStages, kStageF = G::kStage, kOffSFB = G::kOffSFB;
    constexpr uint32_t kTmemSF = G::kTmemSF, kIdescF = G::kIdesc;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStagesF * kStageF);
    uint64_t* empty = full + kStagesF;
    uint64_t* acc_full = empty + kStagesF;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const ExpertArgs& a = sa.e;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t K = MODE == FMODE_GU ? a.L.n_embd : a.L.n_ff;
    const int64_t R = MODE == FMODE_GU ? a.L.n_ff : a.L.n_embd;       // rows of each weight matrix
    const int n_chunk = (int) (K >> 8);                                 // stages (256 columns) per unit
    constexpr int kRowsPerBlock = MODE == FMODE_GU ? 128 : 256;         // weight rows of the two tiles of one accumulator set
    const int n_rb = (int) ((R + kRowsPerBlock - 1) / kRowsPerBlock);
    // a unit = one pass x n_sub consecutive row blocks, sized to at least 4 stages so that the per-unit bookkeeping (the
    // pass record, the entries' rows and scales) is amortised and its loads hide behind the stream
    const int n_sub_full = max(1, min(n_rb, (4 + n_chunk - 1) / n_chunk));
    const PackedGeom geo = packed_geom(a.L.n_embd, a.L.n_ff);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesF; ++s) {
            mbar_init(&full[s], 33);     // the weight loader's expect_tx arrival + the 32 lanes of the activation loader
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;
    // barriers and tensor memory are set up; from here on the kernel reads what the kernels before it wrote (the pass list,
    // the activation images), so a programmatic launch waits here for them to finish.  Except the weight loader of the down
    // stage: the pass list it follows was written before the gate/up stage ran and the blobs are constants, so it fills the
    // stages while the SwiGLU rows' images are still being made - the stream is in flight when the first image arrives.
    if (!(sa.early_weights && warp == 1)) pdl_wait();
    pdl_launch_dependents();
    // ... unless the window is so small that such units would not go round the SMs three times: then one row block a unit, so that
    // the last, partial round of the static schedule costs half as much (a window of 8 tokens has ~80 passes)
    const int n_pass = sa.n_items[0];
    const int n_sub = (n_sub_full > 1 && n_pass * ((n_rb + n_sub_full - 1) / n_sub_full) < 3 * (int) gridDim.x) ? 1 : n_sub_full;
    const int n_upp = (n_rb + n_sub - 1) / n_sub;                        // units per pass
    const int n_units = n_pass * n_upp;

    // unit -> its pass record and its row blocks [rb0, rb1).  Tile 0 / tile 1 of a row block: the 128 gate rows r0.. and the
    // 128 up rows r0.. (gate/up), or down rows r0.. and r0 + 128.. (down).
    auto unit_blocks = [&](int unit, int& rb0, int& rb1) {
        const int pass = unit / n_upp;
        rb0 = (unit - pass * n_upp) * n_sub;
        rb1 = min(n_rb, rb0 + n_sub);
        return pass;
    };

    if (warp == 0) {
        // ---- MMA issuer: per 64-column K-step the three scale copies (smem -> tensor memory), then one MMA per tile
        if (lane == 0) {
            uint32_t kc = 0, ti = 0;
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                int rb0, rb1;
                unit_blocks(unit, rb0, rb1);
                for (int rb = rb0; rb < rb1 && ok; ++rb) {
                    const uint32_t acc = ti & 1u;
                    ok = mbar_wait(&acc_empty[acc], ((ti >> 1) & 1u) ^ 1u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t d0 = tmem + acc * G::kAccCols, d1 = d0 + G::kCols;
                    for (int c = 0; c < n_chunk; ++c, ++kc) {
                        const uint32_t s = kc % kStagesF;
                        ok = mbar_wait(&full[s], (kc / kStagesF) & 1u);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                        const uint32_t st = smem_u32(smem + s * kStageF);
                        const uint32_t tsf = tmem + kTmemSF + s * 48;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tsf + 4 * k), "l"(sf_desc(st + kOffSFA0 + k * 512)) : "memory");
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tsf + 16 + 4 * k), "l"(sf_desc(st + kOffSFA1 + k * 512)) : "memory");
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tsf + 32 + 4 * k), "l"(sf_desc(st + kOffSFB + k * 512)) : "memory");
                            const uint64_t bd = smem_desc_sw128(st + kOffB + k * 32);
                            const uint32_t accum = (c | k) ? 1u : 0u;
                            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
                                         "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::"r"(d0),
                                         "l"(smem_desc_sw128(st + k * 32)), "l"(bd), "r"(kIdescF), "r"(tsf + 4 * k), "r"(tsf + 32 + 4 * k), "r"(accum)
                                         : "memory");
                            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
                                         "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::"r"(d1),
                                         "l"(smem_desc_sw128(st + kOffA1 + k * 32)), "l"(bd), "r"(kIdescF), "r"(tsf + 16 + 4 * k), "r"(tsf + 32 + 4 * k), "r"(accum)
                                         : "memory");
                        }
                        umma_commit(&empty[s]);
                    }
                    if (!ok) break;
                    umma_commit(&acc_full[acc]);
                    ++ti;
                }
            }
            if (!ok) atomicOr(sa.status, 1);
        }
    } else if (warp == 1) {
        // ---- weight loader: one lane, two bulk copies a stage (each a whole block of the packed blob: 16 KB of codes already
        // in the stage's swizzled order + 2 KB of scales), completion counted in bytes on the stage's mbarrier.  The next
        // unit's pass record is requested while this unit streams.
        if (lane == 0) {
            uint32_t issued = 0;
            PassRec nxt;
            nxt.blob = 0ull; nxt.eb = 0; nxt.ntok = 0;
            if ((int) blockIdx.x < n_units) nxt = sa.items[blockIdx.x / n_upp];
            for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
                const PassRec u = nxt;
                if (unit + (int) gridDim.x < n_units) nxt = sa.items[(unit + gridDim.x) / n_upp];
                int rb0, rb1;
                unit_blocks(unit, rb0, rb1);
                const uint8_t* blob = reinterpret_cast<const uint8_t*>(u.blob);
                for (int rb = rb0; rb < rb1 && ok; ++rb) {
                    const uint8_t* b0 = MODE == FMODE_GU ? blob + geo.gate + (size_t) rb * n_chunk * kBlockF : blob + geo.down + (size_t) (2 * rb) * n_chunk * kBlockF;
                    const uint8_t* b1 = MODE == FMODE_GU ? blob + geo.up + (size_t) rb * n_chunk * kBlockF : b0 + (size_t) n_chunk * kBlockF;
                    for (int c = 0; c < n_chunk; ++c, ++issued) {
                        const uint32_t s = issued % kStagesF;
                        ok = mbar_wait(&empty[s], ((issued / kStagesF) & 1u) ^ 1u);
                        if (!ok) break;
                        const uint32_t st = smem_u32(smem + s * kStageF), bar = smem_u32(&full[s]);
                        asm volatile("{\n.reg .b64 t;\nmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n}\n" ::"r"(bar), "r"(2u * kBlockF) : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(st),
                                     "l"(b0 + (size_t) c * kBlockF), "r"((uint32_t) kBlockF), "r"(bar)
                                     : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(st + (uint32_t) kOffA1),
                                     "l"(b1 + (size_t) c * kBlockF), "r"((uint32_t) kBlockF), "r"(bar)
                                     : "memory");
                    }
                }
            }
            if (!ok) atomicOr(sa.status, 1);
        }
    } else if (warp == 2) {
        // ---- activation loader: the pass's FP4 images, 256 columns a stage.  Codes: column n = 4 j + t is term t of entry j;
        // lane l copies 16-byte piece l % 8 of rows l / 8 + 4 i (row 4 i + r4 -> entry i, term r4).  Scales: lane = column n,
        // its scale word of K-step k goes to word (n, 0) of that step's 512-byte block.  A lane runs up to two stages ahead of
        // its own landed copies and arrives on a stage once its copies there are visible to the tensor core.
        const int c8 = lane & 7, r4 = lane >> 3;
        uint32_t dsto[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r7 = 4 * h + r4;
            dsto[h] = (uint32_t) (kOffB + r7 * 128 + ((c8 ^ r7) << 4));
        }
        uint32_t issued = 0, arrived = 0;
        PassRec nxt;
        nxt.blob = 0ull; nxt.eb = 0; nxt.ntok = 0;
        if ((int) blockIdx.x < n_units) nxt = sa.items[blockIdx.x / n_upp];
        for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
            const PassRec u = nxt;
            if (unit + (int) gridDim.x < n_units) nxt = sa.items[(unit + gridDim.x) / n_upp];
            int rb0, rb1;
            unit_blocks(unit, rb0, rb1);
            const uint8_t* crow[ENT];
#pragma unroll
            for (int j = 0; j < ENT; ++j) {
                const int e = u.eb + (j < u.ntok ? j : 0);
                const int ir = (MODE == FMODE_GU && a.n_x_rows > 0) ? a.ent_tok[e] : e;
                crow[j] = sa.codes + ((size_t) ir * kTermsF + r4) * (size_t) (K >> 1) + c8 * 16;
            }
            // scales: column n = 4 entry + term is row n of the B operand; its word of a K-step sits at lane n % 32, word n / 32 of
            // the step's 512-byte block.  A lane serves columns lane, lane + 32, ...
            const uint8_t* srow[ENT / 8];
#pragma unroll
            for (int h = 0; h < ENT / 8; ++h) {
                const int j = 8 * h + (lane >> 2);
                const int e = u.eb + (j < u.ntok ? j : 0);
                const int ir = (MODE == FMODE_GU && a.n_x_rows > 0) ? a.ent_tok[e] : e;
                srow[h] = sa.sfs + ((size_t) ir * kTermsF + (lane & 3)) * (size_t) (K >> 4);
            }
            for (int rb = rb0; rb < rb1 && ok; ++rb) {
                for (int c = 0; c < n_chunk; ++c) {
                    const uint32_t s = issued % kStagesF;
                    ok = mbar_wait(&empty[s], ((issued / kStagesF) & 1u) ^ 1u);
                    if (!ok) break;
                    const uint32_t st = smem_u32(smem + s * kStageF);
#pragma unroll
                    for (int i = 0; i < ENT; ++i)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(st + (uint32_t) ((i >> 1) * 1024) + dsto[i & 1]), "l"(crow[i] + (size_t) c * 128)
                                     : "memory");
#pragma unroll
                    for (int h = 0; h < ENT / 8; ++h)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(st + (uint32_t) kOffSFB + k * 512 + lane * 16 + h * 4),
                                         "l"(srow[h] + (size_t) c * 16 + 4 * k)
                                         : "memory");
                    asm volatile("cp.async.commit_group;\n" ::: "memory");
                    ++issued;
                    if (issued - arrived > 2) {
                        asm volatile("cp.async.wait_group 2;\n" ::: "memory");
                        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                        mbar_arrive(&full[arrived % kStagesF]);
                        ++arrived;
                    }
                }
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (; arrived < issued; ++arrived) mbar_arrive(&full[arrived % kStagesF]);
        if (!ok) atomicOr(sa.status, 1);
    } else {
        // ---- epilogue: thread = TMEM lane = weight row of both tiles.  A warp may only read lanes 32 (warp % 4) .. + 31.
        // The unit's entries (rows, scales, destinations) are fetched before the wait for its first accumulator, so those
        // loads ride under the stream; the next unit's pass record is requested one unit ahead.
        const int q = warp & 3;
        const int rl = q * 32 + lane;
        const uint32_t lane_base = (uint32_t) (q * 32) << 16;
        uint32_t ti = 0;
        PassRec nxt;
        nxt.blob = 0ull; nxt.eb = 0; nxt.ntok = 0;
        if ((int) blockIdx.x < n_units) nxt = sa.items[blockIdx.x / n_upp];
        for (int unit = blockIdx.x; unit < n_units && ok; unit += gridDim.x) {
            const PassRec u = nxt;
            if (unit + (int) gridDim.x < n_units) nxt = sa.items[(unit + gridDim.x) / n_upp];
            int rb0, rb1;
            unit_blocks(unit, rb0, rb1);
            const float* tail = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(u.blob) + geo.tail);
            const float sg = tail[0], su = tail[1], sd = tail[2];
            float f[ENT];
            int64_t orow[ENT];
#pragma unroll
            for (int j = 0; j < ENT; ++j) {
                const int e = u.eb + (j < u.ntok ? j : 0);
                const int ir = (MODE == FMODE_GU && a.n_x_rows > 0) ? a.ent_tok[e] : e;
                f[j] = sa.inv[ir];
                orow[j] = MODE == FMODE_GU ? (int64_t) e * a.L.n_ff : (int64_t) a.ent_dst[e] * a.L.n_embd;
            }
            for (int rb = rb0; rb < rb1; ++rb) {
                const int r0 = rb * kRowsPerBlock;
                const uint32_t acc = ti & 1u;
                ok = __all_sync(kFull, mbar_wait(&acc_full[acc], (ti >> 1) & 1u));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // 8 entries (32 accumulator columns of each tile) at a time
#pragma unroll
                for (int hb = 0; hb < ENT / 8; ++hb) {
                    uint32_t d0[32], d1[32];
                    tmem_ld32(tmem + lane_base + acc * G::kAccCols + 32 * hb, d0);
                    tmem_ld32(tmem + lane_base + acc * G::kAccCols + G::kCols + 32 * hb, d1);
                    if (hb == ENT / 8 - 1) {
                        // the accumulators are in registers: the MMA warp may start the next row block on this set
                        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                        mbar_arrive(&acc_empty[acc]);
                        ++ti;
                    }
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                        const int j = 8 * hb + jj;
                        if (j < u.ntok) {
                            const float v0 = ((__uint_as_float(d0[4 * jj]) + __uint_as_float(d0[4 * jj + 1])) + __uint_as_float(d0[4 * jj + 2])) + __uint_as_float(d0[4 * jj + 3]);
                            const float v1 = ((__uint_as_float(d1[4 * jj]) + __uint_as_float(d1[4 * jj + 1])) + __uint_as_float(d1[4 * jj + 2])) + __uint_as_float(d1[4 * jj + 3]);
                            if (MODE == FMODE_GU) {
                                a.h[orow[j] + r0 + rl] = swiglu(v0 * f[j] * sg, v1 * f[j] * su, a.L);
                            } else {
                                store_out(a.out, a.out_kind, orow[j] + r0 + rl, v0 * f[j] * sd);
                                store_out(a.out, a.out_kind, orow[j] + r0 + 128 + rl, v1 * f[j] * sd);
                            }
                        }
                    }
                }
            }
        }
        if (!ok && lane == 0) atomicOr(sa.status, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template <int MODE, int ENT>
int32_t launch_stream(const StreamArgs& sa, cudaStream_t st) {
    static std::atomic<bool> configured[64];   // per device; threads of different devices call concurrently
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(nvf4_stream_kernel<MODE, ENT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) FG<ENT>::kSmem);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    launch_k(nvf4_stream_kernel<MODE, ENT>, dim3((unsigned) sm_count()), dim3(kThreadsF), FG<ENT>::kSmem, st, sa);
    return launch_status();
}

}  // namespace

// scratch beyond the SwiGLU buffer: x images (codes, scales), h images, inverse row scales, the pass list
size_t experts_packed_scratch_bytes(int64_t cap, int64_t H, int64_t I) {
    return al256f((size_t) cap * kTermsF * H / 2) + al256f((size_t) cap * kTermsF * H / 16) + al256f((size_t) cap * kTermsF * I / 2) +
           al256f((size_t) cap * kTermsF * I / 16) + 2 * al256f((size_t) cap * 4) + al256f((size_t) (cap + 1) * 16 + 16);
}

// the scratch regions behind the SwiGLU buffer
struct PackedScratch {
    uint8_t *xcodes, *xsf, *hcodes, *hsf;
    float *xinv, *hinv;
    int* n_items;
    PassRec* items;
};
static PackedScratch carve_scratch(void* scratch, int64_t cap, int64_t H, int64_t I) {
    PackedScratch r;
    uint8_t* p = static_cast<uint8_t*>(scratch) + al256f((size_t) cap * I * 4);
    r.xcodes = p;
    p += al256f((size_t) cap * kTermsF * H / 2);
    r.xsf = p;
    p += al256f((size_t) cap * kTermsF * H / 16);
    r.hcodes = p;
    p += al256f((size_t) cap * kTermsF * I / 2);
    r.hsf = p;
    p += al256f((size_t) cap * kTermsF * I / 16);
    r.xinv = reinterpret_cast<float*>(p);
    p += al256f((size_t) cap * 4);
    r.hinv = reinterpret_cast<float*>(p);
    p += al256f((size_t) cap * 4);
    r.n_items = reinterpret_cast<int*>(p);
    r.items = reinterpret_cast<PassRec*>(r.n_items + 4);
    return r;
}

int32_t experts_packed_x_images(const bsx_expert_layout& L, const void* x, int32_t x_kind, int32_t n_x_rows, int64_t cap, void* scratch, cudaStream_t st) {
    const PackedScratch sc = carve_scratch(scratch, cap, L.n_embd, L.n_ff);
    const int64_t n_sb = L.n_embd / 16;
    if (n_sb <= 32) launch_k(x_images_kernel<32>, dim3((unsigned) ((n_x_rows + 7) / 8)), dim3(256), 0, st, x, (int) x_kind, (int) n_x_rows, L.n_embd, sc.xcodes, sc.xsf, sc.xinv);
    else if (n_sb <= 128) launch_k(x_images_kernel<128>, dim3((unsigned) ((n_x_rows + 1) / 2)), dim3(256), 0, st, x, (int) x_kind, (int) n_x_rows, L.n_embd, sc.xcodes, sc.xsf, sc.xinv);
    else launch_k(x_images_kernel<256>, dim3((unsigned) n_x_rows), dim3(256), 0, st, x, (int) x_kind, (int) n_x_rows, L.n_embd, sc.xcodes, sc.xsf, sc.xinv);
    return launch_status();
}

void experts_packed_pass_list(void* scratch, int64_t cap, int64_t H, int64_t I, PassRec** items, int** n_items) {
    const PackedScratch sc = carve_scratch(scratch, cap, H, I);
    *items = sc.items;
    *n_items = sc.n_items;
}

int32_t experts_grouped_packed(const ExpertArgs& a, int32_t* status, cudaStream_t st, bool x_images_ready, bool pass_list_ready) {
    const bsx_expert_layout& L = a.L;
    if (L.gu_type != kTypeNVFP4 || L.up_type != kTypeNVFP4 || L.d_type != kTypeNVFP4) return BSX_E_TYPE;
    if (L.n_embd % 256 || L.n_ff % 256) return BSX_E_TYPE;       // whole 256-column stages, whole 128-row tiles
    const int64_t cap = a.cap_entries, H = L.n_embd, I = L.n_ff;
    const PackedScratch sc = carve_scratch(a.h, cap, H, I);
    uint8_t *xcodes = sc.xcodes, *xsf = sc.xsf, *hcodes = sc.hcodes, *hsf = sc.hsf;
    float *xinv = sc.xinv, *hinv = sc.hinv;
    int* n_items = sc.n_items;
    PassRec* items = sc.items;
    const int phase = experts_phase(a.L);
    const int64_t x_rows = a.n_x_rows > 0 ? a.n_x_rows : cap;
    StreamArgs sa;
    sa.e = a;
    sa.items = items;
    sa.n_items = n_items;
    sa.status = status;
    sa.early_weights = 0;
    int32_t rc = BSX_OK;
    // Passes of 16 entries where the groups are deep: the capacities say how many entries a group gets on average (an expert-parallel
    // rank sees every rank's tokens on its share of the experts).  A pass list that came with the plan has passes of 8.
    const bool wide = !pass_list_ready && a.cap_groups > 0 && cap >= 12 * a.cap_groups;
    const int pass_entries = wide ? kEntWide : kEntNarrow;
    if (phase != 2) {
        if (x_images_ready && !pass_list_ready)
            launch_k(prep_fp4_kernel<false, 32>, dim3(1), dim3(256), 0, st, a, xcodes, xsf, xinv, items, n_items, pass_entries);   // the pass list alone
        else if (!x_images_ready) launch_prep<false>(a, x_rows, H, xcodes, xsf, xinv, items, n_items, pass_entries, st);
        sa.codes = xcodes;
        sa.sfs = xsf;
        sa.inv = xinv;
        rc = wide ? launch_stream<FMODE_GU, kEntWide>(sa, st) : launch_stream<FMODE_GU, kEntNarrow>(sa, st);
    }
    if (rc != BSX_OK || phase == 1) return rc;
    launch_prep<true>(a, cap, I, hcodes, hsf, hinv, items, n_items, 0, st);   // the pass list is the gate/up stage's
    sa.codes = hcodes;
    sa.sfs = hsf;
    sa.inv = hinv;
    sa.early_weights = 1;
    return wide ? launch_stream<FMODE_DOWN, kEntWide>(sa, st) : launch_stream<FMODE_DOWN, kEntNarrow>(sa, st);
}

}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_expert_packed_bytes(const bsx_expert_layout* L) {
    if (!L || L->gu_type != kTypeNVFP4 || L->up_type != kTypeNVFP4 || L->d_type != kTypeNVFP4 || L->n_embd % 256 || L->n_ff % 256) return 0;
    return (packed_geom(L->n_embd, L->n_ff).bytes + 255) & ~(size_t) 255;
}

extern "C" int32_t bsx_expert_pack(const bsx_expert_layout* L, const void* blob, void* packed, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!L || !aligned(blob, 16) || !aligned(packed, 256)) return BSX_E_POINTER;
    if (!bsx_expert_packed_bytes(L)) return BSX_E_TYPE;
    const int64_t n = 2 * L->n_ff * (L->n_embd / 64) + L->n_embd * (L->n_ff / 64);
    pack_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(static_cast<const uint8_t*>(blob), static_cast<uint8_t*>(packed), *L);
    return launch_status();
}

extern "C" size_t bsx_experts_packed_scratch_bytes(const bsx_expert_layout* L, int64_t cap_entries) {
    if (!L || cap_entries < 0 || !bsx_expert_packed_bytes(L)) return 0;
    return al256f((size_t) cap_entries * L->n_ff * 4) + experts_packed_scratch_bytes(cap_entries, L->n_embd, L->n_ff) + 4096;
}

extern "C" int32_t bsx_experts_grouped_packed(const bsx_expert_layout* layout, const unsigned long long* grp_ptr, const int32_t* grp_start,
                                              const int32_t* n_groups, const int32_t* ent_dst, const int32_t* ent_tok, int64_t cap_groups,
                                              int64_t cap_entries, const void* x, int32_t x_kind, int32_t n_x_rows, void* scratch, void* out,
                                              int32_t out_kind, int32_t* status, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout || !status) return BSX_E_POINTER;
    if (!bsx_expert_packed_bytes(layout)) return BSX_E_TYPE;
    if (x_kind < BSX_X_F32 || x_kind > BSX_X_Q8_1 || (out_kind != BSX_OUT_F32 && out_kind != BSX_OUT_BF16)) return BSX_E_GEOMETRY;
    if (cap_groups < 0 || cap_entries < 0 || cap_entries > (int64_t) 1 << 30) return BSX_E_GEOMETRY;
    if (cap_groups == 0 || cap_entries == 0) return BSX_OK;
    if (!grp_ptr || !grp_start || !n_groups || !ent_dst || !ent_tok || !aligned(x, 16) || !aligned(scratch, 256) || !aligned(out, 16)) return BSX_E_POINTER;
    // n_x_rows < 0: the images of -n_x_rows rows of x are already in this scratch (bsx_experts_packed_x_images)
    const bool ready = n_x_rows < 0;
    if (ready) n_x_rows = -n_x_rows;
    if (n_x_rows > cap_entries) {
        if (ready) return BSX_E_GEOMETRY;
        n_x_rows = 0;
    }
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
    a.n_x_rows = n_x_rows;
    a.grid = nullptr;
    return experts_grouped_packed(a, status, (cudaStream_t) stream, ready, false);
}

extern "C" int32_t bsx_norm_pack_images(const bsx_expert_layout* layout, const void* x, int32_t x_kind, const float* w, float eps,
                                        int32_t n_x_rows, int64_t cap_entries, void* scratch, float* xn, void* act, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout || !aligned(x, 16) || !aligned(scratch, 256) || !aligned(xn, 16) || !w) return BSX_E_POINTER;
    if (!bsx_expert_packed_bytes(layout)) return BSX_E_TYPE;
    if (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16) return BSX_E_TYPE;
    if (n_x_rows < 0 || n_x_rows > cap_entries) return BSX_E_GEOMETRY;
    if (n_x_rows == 0) return BSX_OK;
    const PackedScratch sc = carve_scratch(scratch, cap_entries, layout->n_embd, layout->n_ff);
    cudaStream_t st = (cudaStream_t) stream;
    if (x_kind == BSX_X_BF16)
        launch_k(norm_images_kernel<true>, dim3((unsigned) n_x_rows), dim3(kNormThreads), 0, st, x, w, eps, layout->n_embd, static_cast<uint16_t*>(act), xn, sc.xcodes,
                 sc.xsf, sc.xinv);
    else
        launch_k(norm_images_kernel<false>, dim3((unsigned) n_x_rows), dim3(kNormThreads), 0, st, x, w, eps, layout->n_embd, static_cast<uint16_t*>(act), xn, sc.xcodes,
                 sc.xsf, sc.xinv);
    return launch_status();
}

extern "C" int32_t bsx_experts_packed_x_images(const bsx_expert_layout* layout, const void* x, int32_t x_kind, int32_t n_x_rows, int64_t cap_entries,
                                               void* scratch, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout || !aligned(x, 16) || !aligned(scratch, 256)) return BSX_E_POINTER;
    if (!bsx_expert_packed_bytes(layout)) return BSX_E_TYPE;
    if (x_kind < BSX_X_F32 || x_kind > BSX_X_Q8_1 || n_x_rows < 0 || n_x_rows > cap_entries) return BSX_E_GEOMETRY;
    if (n_x_rows == 0) return BSX_OK;
    return experts_packed_x_images(*layout, x, x_kind, n_x_rows, cap_entries, scratch, (cudaStream_t) stream);
}
