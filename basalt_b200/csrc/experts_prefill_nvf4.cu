// experts_prefill_nvf4.cu - prompt-sized grouped experts on the block-scaled FP4 tensor cores (tcgen05 kind::mxf4nvf4), over
// blobs packed by bsx_expert_pack.
//
// The same ragged grouped GEMM as experts_prefill.cu (Basalt's fp4::run_group, include/basalt/prefill/moe_fp4.hpp:43-113):
//   gate/up:  [128 rows x H] . [H x 2I]  -> SwiGLU ->  h [rows x I]       (fp32, in scratch)
//   down:     [128 rows x I] . [I x H]   ->             dm [rows x H]      (fp32, unweighted, row = dispatch slot)
// but nothing is decoded: a packed block (128 weight rows x 256 columns: 16 KB of codes in the swizzled order of a stage,
// 2 KB of UE4M3 scale words) is one bulk copy into shared memory and the tensor core reads it as it is.  Activations enter
// as four FP4 terms per row (nvf4.cuh; relative error ~1e-4), i.e. four MMAs per 64-column K-step into one accumulator.
// That is what Basalt's sm_120 kernel does with ONE term (and an optional second) at ~1e-1 .. 1e-2; four terms cost the
// tensor time of an fp16 product and meet the 2e-3 bar.
//
// Persistent CTAs, one per SM, static round-robin over work items (128-row tile of one expert, N weight rows):
//   gate/up: N = 256 = the tile's 128 gate rows and their 128 up rows (two packed blocks), one accumulator of 256 columns;
//   down:    N = 128 (one packed block), two accumulators, so the epilogue of one item overlaps the next item's stream.
// Warp 0: per K-step the scale copies (tcgen05.cp shared -> tensor memory) and the four MMAs (M = 128 rows); warp 1: the
// weights (one lane, bulk copies, completion in bytes); warps 2-5: the tile's activation rows - codes by 16-byte cp.async
// gathers into four swizzled A tiles, scale words through registers into the lane-major order tcgen05.cp reads; warps 6-9:
// epilogue (thread = TMEM lane = row).  Two stages of 256 columns; every wait is time-bounded with a status word.
// With n_ff <= 512 the down product runs as prefill_down_resident_kernel instead (the tile's rows stay in shared memory).
#include <atomic>
#include <cuda_fp16.h>

#include "common.cuh"
#include "experts.cuh"
#include "nvf4.cuh"
#include "tc5.cuh"

namespace bsx {
namespace {

constexpr int kStagesQ = 2;
constexpr int kThreadsQ = 32 * 10;
constexpr int kATileQ = 128 * 128;                 // one term's A tile of a stage: 128 rows x 128 bytes
constexpr int kSFQ = 4 * 512;                      // four K-steps of 32 x 4 scale words
enum { QMODE_GU = 0, QMODE_DOWN = 1 };

template <int MODE>
struct Geo {
    static constexpr int kN = MODE == QMODE_GU ? 256 : 128;           // weight rows (accumulator columns) of an item
    static constexpr int kBlocks = kN / 128;                           // packed blocks of the B operand
    static constexpr int kAccSets = MODE == QMODE_GU ? 1 : 2;
    // a stage: [A term 0..3 | SFA term 0..3 | B codes (kBlocks x 16 KB) | SFB (kBlocks x 2 KB)]
    static constexpr int kOffSFA = kTermsF * kATileQ;
    static constexpr int kOffB = kOffSFA + kTermsF * kSFQ;
    static constexpr int kOffSFB = kOffB + kBlocks * kATileQ;
    static constexpr int kStage = kOffSFB + kBlocks * kSFQ;            // 110,592 (gate/up) or 92,160 (down): multiples of 1024
    static constexpr size_t kSmem = 1024 + (size_t) kStagesQ * kStage + 256;
    // tensor memory: accumulators first, then per stage the scale columns: SFA 4 terms x 4 steps x 4, SFB 4 steps x 4 kBlocks
    static constexpr uint32_t kTmemSF = kAccSets * kN;
    static constexpr uint32_t kSFACols = kTermsF * 16, kSFBCols = 16 * kBlocks, kSFStage = kSFACols + kSFBCols;
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t) (kN >> 3) << 17) | ((uint32_t) (128 >> 4) << 24);
};

// a 128-row tile of one expert with everything the kernels need about it in one 16-byte load (blob 0: held elsewhere)
struct __align__(16) TileRec {
    unsigned long long blob;
    int row0, rows;
};

__global__ void __launch_bounds__(256) tile_records_kernel(const int32_t* __restrict__ tiles, const int32_t* __restrict__ n_tiles,
                                                           const int32_t* __restrict__ off, const unsigned long long* __restrict__ blob_table,
                                                           TileRec* __restrict__ recs, int64_t cap_tiles) {
    const int64_t t = (int64_t) blockIdx.x * 256 + threadIdx.x;
    if (t >= cap_tiles || t >= *n_tiles) return;
    const int expert = tiles[2 * t], row0 = tiles[2 * t + 1];
    TileRec r;
    r.blob = blob_table[expert];
    r.row0 = row0;
    r.rows = min(128, off[expert + 1] - row0);
    recs[t] = r;
}

struct PrefillFArgs {
    bsx_expert_layout L;
    const TileRec* recs;                     // [n_tiles]
    const int32_t* src;                      // [rows] token of each row
    const int32_t* n_tiles;
    const uint8_t* codes;                    // activation images of this product's A operand
    const uint8_t* sfs;
    const float* inv;
    float* h;                                // [rows + 128][I] fp32 SwiGLU output
    float* dm;                               // [rows][H] fp32
    int32_t* status;
};

__device__ __forceinline__ uint64_t sf_desc_q(uint32_t addr) {   // 32 rows x 16 bytes, 8-row groups 128 bytes apart, no swizzle
    return (uint64_t) ((addr & 0x3FFFFu) >> 4) | ((uint64_t) (128 >> 4) << 16) | ((uint64_t) (128 >> 4) << 32) | ((uint64_t) 1 << 46);
}

// activation rows -> FP4 images.  FROM_H = false: rows of x (fp32 or bf16), image row = token; true: rows of h, image row =
// dispatch row, as many as the dispatch has (off[E], read on the device).
template <bool FROM_H, int TPR>
__global__ void __launch_bounds__(256) prefill_images_kernel(const void* __restrict__ src, int kind, int64_t n_rows, const int32_t* __restrict__ n_rows_dev,
                                                              int64_t K, uint8_t* __restrict__ codes, uint8_t* __restrict__ sfs, float* __restrict__ inv) {
    __shared__ float shf[8];
    const int64_t n = n_rows_dev ? min(n_rows, (int64_t) *n_rows_dev) : n_rows;
    const int64_t i = (int64_t) blockIdx.x * (256 / TPR) + threadIdx.x / TPR;
    if ((int64_t) blockIdx.x * (256 / TPR) >= n) return;       // whole block past the end
    fp4_image_row<TPR>(src, kind, i < n ? i : 0, K, i < n, (int) i, codes, sfs, inv, shf);
}

template <bool FROM_H>
void launch_images(const void* src, int kind, int64_t rows, const int32_t* rows_dev, int64_t K, uint8_t* codes, uint8_t* sfs, float* inv, cudaStream_t st) {
    const int64_t n_sb = K / 16;
    if (n_sb <= 32) prefill_images_kernel<FROM_H, 32><<<(unsigned) ((rows + 7) / 8), 256, 0, st>>>(src, kind, rows, rows_dev, K, codes, sfs, inv);
    else if (n_sb <= 128) prefill_images_kernel<FROM_H, 128><<<(unsigned) ((rows + 1) / 2), 256, 0, st>>>(src, kind, rows, rows_dev, K, codes, sfs, inv);
    else prefill_images_kernel<FROM_H, 256><<<(unsigned) rows, 256, 0, st>>>(src, kind, rows, rows_dev, K, codes, sfs, inv);
}

template <int MODE>
__global__ void __launch_bounds__(kThreadsQ, 1) prefill_nvf4_kernel(PrefillFArgs a) {
    using G = Geo<MODE>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStagesQ * G::kStage);
    uint64_t* empty = full + kStagesQ;
    uint64_t* acc_full = empty + kStagesQ;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t K = MODE == QMODE_GU ? a.L.n_embd : a.L.n_ff;
    const int n_chunk = (int) (K >> 8);
    const int n_out = MODE == QMODE_GU ? (int) a.L.n_ff : (int) a.L.n_embd;       // neurons, or down rows
    const int n_n = n_out / 128;                                                    // items per row tile
    const int n_items = *a.n_tiles * n_n;
    const PackedGeom geo = packed_geom(a.L.n_embd, a.L.n_ff);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesQ; ++s) {
            mbar_init(&full[s], 1 + 128);    // the weight loader's expect_tx arrival + the 128 activation-loader lanes
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
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    // item -> (tile: expert, first row, live rows; first neuron / down row n0); items of experts held elsewhere are skipped by
    // every role alike
    struct Item { const uint8_t* blob; int row0, rows, n0; };
    auto get_item = [&](int item, Item& it) -> bool {
        const int tile = item / n_n;
        const TileRec r = a.recs[tile];
        if (r.blob == 0ull) return false;
        it.blob = reinterpret_cast<const uint8_t*>(r.blob);
        it.row0 = r.row0;
        it.rows = r.rows;
        it.n0 = (item - tile * n_n) * 128;
        return true;
    };

    if (warp == 0) {
        // ---- MMA issuer
        if (lane == 0) {
            uint32_t kc = 0, ti = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                Item it;
                if (!get_item(item, it)) continue;
                const uint32_t acc = ti % G::kAccSets;
                ok = mbar_wait(&acc_empty[acc], ((ti / G::kAccSets) & 1u) ^ 1u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d = tmem + acc * G::kN;
                for (int c = 0; c < n_chunk; ++c, ++kc) {
                    const uint32_t s = kc % kStagesQ;
                    ok = mbar_wait(&full[s], (kc / kStagesQ) & 1u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t st = smem_u32(smem + s * G::kStage);
                    const uint32_t tsfa = tmem + G::kTmemSF + s * G::kSFStage, tsfb = tsfa + G::kSFACols;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
#pragma unroll
                        for (int b = 0; b < G::kBlocks; ++b)
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tsfb + (uint32_t) (4 * G::kBlocks * k + 4 * b)),
                                         "l"(sf_desc_q(st + (uint32_t) G::kOffSFB + b * kSFQ + k * 512))
                                         : "memory");
                        const uint64_t bd = smem_desc_sw128(st + (uint32_t) G::kOffB + k * 32);
#pragma unroll
                        for (int t = 0; t < kTermsF; ++t) {
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tsfa + (uint32_t) (16 * t + 4 * k)),
                                         "l"(sf_desc_q(st + (uint32_t) G::kOffSFA + t * kSFQ + k * 512))
                                         : "memory");
                            const uint32_t accum = (c | k | t) ? 1u : 0u;
                            asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
                                         "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::"r"(d),
                                         "l"(smem_desc_sw128(st + (uint32_t) (t * kATileQ) + k * 32)), "l"(bd), "r"(G::kIdesc), "r"(tsfa + (uint32_t) (16 * t + 4 * k)),
                                         "r"(tsfb + (uint32_t) (4 * G::kBlocks * k)), "r"(accum)
                                         : "memory");
                        }
                    }
                    umma_commit(&empty[s]);
                }
                if (!ok) break;
                umma_commit(&acc_full[acc]);
                ++ti;
            }
            if (!ok) atomicOr(a.status, 1);
        }
    } else if (warp == 1) {
        // ---- weight loader: one lane; per stage each packed block of the item as two bulk copies (codes, scale words)
        if (lane == 0) {
            uint32_t issued = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                Item it;
                if (!get_item(item, it)) continue;
                const int tile = it.n0 >> 7;
                const uint8_t* blk[G::kBlocks];
                if (MODE == QMODE_GU) {
                    blk[0] = it.blob + geo.gate + (size_t) tile * n_chunk * kBlockF;
                    if (G::kBlocks > 1) blk[G::kBlocks - 1] = it.blob + geo.up + (size_t) tile * n_chunk * kBlockF;
                } else {
                    blk[0] = it.blob + geo.down + (size_t) tile * n_chunk * kBlockF;
                }
                for (int c = 0; c < n_chunk; ++c, ++issued) {
                    const uint32_t s = issued % kStagesQ;
                    ok = mbar_wait(&empty[s], ((issued / kStagesQ) & 1u) ^ 1u);
                    if (!ok) break;
                    const uint32_t st = smem_u32(smem + s * G::kStage), bar = smem_u32(&full[s]);
                    asm volatile("{\n.reg .b64 t;\nmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n}\n" ::"r"(bar), "r"((uint32_t) (G::kBlocks * kBlockF))
                                 : "memory");
#pragma unroll
                    for (int b = 0; b < G::kBlocks; ++b) {
                        const uint8_t* g = blk[b] + (size_t) c * kBlockF;
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(st + (uint32_t) G::kOffB + b * kATileQ),
                                     "l"(g), "r"((uint32_t) kATileQ), "r"(bar)
                                     : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(st + (uint32_t) G::kOffSFB + b * kSFQ),
                                     "l"(g + kATileQ), "r"((uint32_t) kSFQ), "r"(bar)
                                     : "memory");
                    }
                }
            }
            if (!ok) atomicOr(a.status, 1);
        }
    } else if (warp <= 5) {
        // ---- activation loaders (128 lanes).  Codes: lane = (16-byte piece c8, row group r16); rows r16 + 16 i, every term.
        // Scales: lane = row m; for each term and K-step one word into slot (m % 32, m / 32) of that step's block.  A lane
        // arrives on a stage when its copies there have landed.
        const int tl = threadIdx.x - 64;
        const int c8 = tl & 7, r16 = tl >> 3;
        uint32_t issued = 0, arrived = 0;
        // Software pipeline over items so that no item starts with a chain of dependent loads: the tile record of the item after
        // next and the row indices of the next item are requested while this item streams.
        auto next_valid = [&](int from, TileRec& r) {     // first item >= from (in this CTA's stride) whose expert is held here
            int it = from;
            for (; it < n_items; it += gridDim.x) {
                r = a.recs[it / n_n];
                if (r.blob != 0ull) break;
            }
            return it;
        };
        auto load_idx = [&](const TileRec& r, int (&idx)[9]) {   // image rows of this lane's 8 code rows and its scale row
#pragma unroll
            for (int i = 0; i < 9; ++i) {
                const int rw = i < 8 ? r16 + 16 * i : tl;
                const int rr = rw < r.rows ? rw : 0;
                idx[i] = MODE == QMODE_GU ? a.src[r.row0 + rr] : r.row0 + rr;
            }
        };
        TileRec rec0, rec1, rec2;
        int idx0[9], idx1[9];
        int item = next_valid(blockIdx.x, rec0);
        int item1 = item < n_items ? next_valid(item + gridDim.x, rec1) : n_items;
        if (item < n_items) load_idx(rec0, idx0);
        if (item1 < n_items) load_idx(rec1, idx1);
        while (item < n_items && ok) {
            const int item2 = item1 < n_items ? next_valid(item1 + gridDim.x, rec2) : n_items;
            Item it;
            it.blob = reinterpret_cast<const uint8_t*>(rec0.blob);
            it.row0 = rec0.row0;
            it.rows = rec0.rows;
            it.n0 = (item - (item / n_n) * n_n) * 128;
            // image rows behind the tile's rows: the row's token (gate/up) or the dispatch row itself (down); rows past the
            // expert's last row read the tile's first row (their results are never stored)
            const uint8_t* crow[8];
            uint32_t cdst[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = r16 + 16 * i;
                crow[i] = a.codes + (size_t) idx0[i] * kTermsF * (size_t) (K >> 1) + c8 * 16;
                cdst[i] = (uint32_t) ((r >> 3) * 1024 + (r & 7) * 128 + ((c8 ^ (r & 7)) << 4));
            }
            const uint8_t* srow = a.sfs + (size_t) idx0[8] * kTermsF * (size_t) (K >> 4);
            const uint32_t sdst = (uint32_t) (G::kOffSFA + (tl & 31) * 16 + (tl >> 5) * 4);
            for (int c = 0; c < n_chunk; ++c) {
                // hand over what is already on its way before blocking on the next slot (it frees only when the tensor core has
                // consumed the stage before this one)
                if (issued > arrived) {
                    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    for (; arrived < issued; ++arrived) mbar_arrive(&full[arrived % kStagesQ]);
                }
                const uint32_t s = issued % kStagesQ;
                ok = mbar_wait(&empty[s], ((issued / kStagesQ) & 1u) ^ 1u);
                if (!ok) break;
                const uint32_t st = smem_u32(smem + s * G::kStage);
#pragma unroll
                for (int t = 0; t < kTermsF; ++t) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(st + (uint32_t) (t * kATileQ) + cdst[i]),
                                     "l"(crow[i] + (size_t) t * (size_t) (K >> 1) + (size_t) c * 128)
                                     : "memory");
                }
                // this row's scale words: 16 bytes a term (the chunk's four K-steps) through registers, then one word into slot
                // (m % 32, m / 32) of each step's block (four rows share a 16-byte slot, so no 16-byte copy can place them)
                uint4 sv[kTermsF];
#pragma unroll
                for (int t = 0; t < kTermsF; ++t) sv[t] = *reinterpret_cast<const uint4*>(srow + (size_t) t * (size_t) (K >> 4) + (size_t) c * 16);
#pragma unroll
                for (int t = 0; t < kTermsF; ++t) {
                    const uint32_t w[4] = {sv[t].x, sv[t].y, sv[t].z, sv[t].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(st + sdst + (uint32_t) (t * kSFQ + k * 512)), "r"(w[k]) : "memory");
                }
                asm volatile("cp.async.commit_group;\n" ::: "memory");
                ++issued;
            }
            // advance the pipeline: the next item's indices were requested one item ago; request those of the item after it
            item = item1;
            item1 = item2;
            rec0 = rec1;
            rec1 = rec2;
#pragma unroll
            for (int i = 0; i < 9; ++i) idx0[i] = idx1[i];
            if (item1 < n_items) load_idx(rec1, idx1);
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (; arrived < issued; ++arrived) mbar_arrive(&full[arrived % kStagesQ]);
        if (!ok) atomicOr(a.status, 1);
    } else {
        // ---- epilogue: thread p reads TMEM lane p (= tile row p).  A warp may only read lanes 32 (warp % 4) .. + 31.
        const int p = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t) ((warp & 3) * 32) << 16;
        uint32_t ti = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            Item it;
            if (!get_item(item, it)) continue;
            const bool row_live = p < it.rows;
            const float* tail = reinterpret_cast<const float*>(it.blob + geo.tail);
            const int64_t ir = !row_live ? 0 : (MODE == QMODE_GU ? (int64_t) a.src[it.row0 + p] : (int64_t) (it.row0 + p));
            const float f = row_live ? a.inv[ir] : 0.f;
            const float sg = tail[0] * f, su = tail[1] * f, sd = tail[2] * f;
            const uint32_t acc = ti % G::kAccSets;
            ok = __all_sync(kFull, mbar_wait(&acc_full[acc], (ti / G::kAccSets) & 1u));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t tbase = tmem + lane_base + acc * G::kN;
            if (MODE == QMODE_GU) {
                float* hrow = a.h + (size_t) (it.row0 + p) * a.L.n_ff + it.n0;
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 16) {
                    uint32_t g[16], u[16];
                    tmem_ld16(tbase + (uint32_t) c0, g);
                    tmem_ld16(tbase + (uint32_t) (128 + c0), u);
                    if (row_live) {
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            reinterpret_cast<float4*>(hrow + c0)[v] =
                                make_float4(swiglu(__uint_as_float(g[4 * v]) * sg, __uint_as_float(u[4 * v]) * su, a.L),
                                            swiglu(__uint_as_float(g[4 * v + 1]) * sg, __uint_as_float(u[4 * v + 1]) * su, a.L),
                                            swiglu(__uint_as_float(g[4 * v + 2]) * sg, __uint_as_float(u[4 * v + 2]) * su, a.L),
                                            swiglu(__uint_as_float(g[4 * v + 3]) * sg, __uint_as_float(u[4 * v + 3]) * su, a.L));
                    }
                }
            } else {
                float* orow = a.dm + (size_t) (it.row0 + p) * a.L.n_embd + it.n0;
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t d[32];
                    tmem_ld32(tbase + (uint32_t) c0, d);
                    if (row_live) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            reinterpret_cast<float4*>(orow + c0)[v] = make_float4(__uint_as_float(d[4 * v]) * sd, __uint_as_float(d[4 * v + 1]) * sd,
                                                                                 __uint_as_float(d[4 * v + 2]) * sd, __uint_as_float(d[4 * v + 3]) * sd);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(&acc_empty[acc]);
            ++ti;
        }
        if (!ok && lane == 0) atomicOr(a.status, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------- down product with the tile's rows resident
// When n_ff <= 512 a tile's SwiGLU rows - 128 rows x n_ff columns as four FP4 terms, 72 KB per 256 columns with their scale
// words - fit in shared memory for the whole tile, so they are fetched once instead of once per block of down rows, and the
// kernel streams only weights: one bulk copy a stage brings a block of 128 down rows over all of K (KC packed blocks, which
// are consecutive in the blob).  Item = a 128-row tile; per tile 16 x (n_embd / 2048) stages, each one accumulator of 128
// columns, two accumulators in flight.  Tensor memory: accumulators [0, 256), the tile's activation scales [256, 256 + 64 KC),
// per stage the weight scales.
template <int KC>
struct GeoR {
    static constexpr int kABytes = KC * kTermsF * kATileQ;          // [chunk][term] code tiles
    static constexpr int kOffSFA = kABytes;                           // [chunk][term][step] scale blocks
    static constexpr int kOffB = kOffSFA + KC * kTermsF * kSFQ;       // two stages of KC packed blocks
    static constexpr int kStageB = KC * kBlockF;
    static constexpr int kBars = kOffB + 2 * kStageB;
    static constexpr size_t kSmem = 1024 + (size_t) kBars + 256;
    static constexpr uint32_t kTmemSFA = 256, kTmemSFB = 256 + 64 * KC, kSFBStage = 16 * KC;
    static constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | ((uint32_t) (128 >> 3) << 17) | ((uint32_t) (128 >> 4) << 24);
};

template <int KC>
__global__ void __launch_bounds__(kThreadsQ, 1) prefill_down_resident_kernel(PrefillFArgs a) {
    using G = GeoR<KC>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    uint64_t* b_full = reinterpret_cast<uint64_t*>(smem + G::kBars);
    uint64_t* b_empty = b_full + 2;
    uint64_t* acc_full = b_empty + 2;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* a_full = acc_empty + 2;
    uint64_t* a_empty = a_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a_empty + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t K = a.L.n_ff;
    const int n_nb = (int) (a.L.n_embd / 128);            // blocks of 128 down rows = stages per tile
    const int n_tiles = *a.n_tiles;
    const PackedGeom geo = packed_geom(a.L.n_embd, a.L.n_ff);

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&b_full[s], 1);
            mbar_init(&b_empty[s], 1);
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 128);
        }
        mbar_init(a_full, 128);
        mbar_init(a_empty, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t sbase = smem_u32(smem);
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t ti = 0, nbc = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                if (a.recs[tile].blob == 0ull) continue;
                ok = mbar_wait(a_full, ti & 1u);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // the tile's activation scales: shared -> tensor memory, once
#pragma unroll
                for (int c = 0; c < KC; ++c)
#pragma unroll
                    for (int t = 0; t < kTermsF; ++t)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tmem + G::kTmemSFA + (uint32_t) (64 * c + 16 * t + 4 * k)),
                                         "l"(sf_desc_q(sbase + (uint32_t) G::kOffSFA + (uint32_t) (((c * kTermsF + t) * 4 + k) * 512)))
                                         : "memory");
                for (int nb = 0; nb < n_nb; ++nb, ++nbc) {
                    const uint32_t s = nbc & 1u, par = (nbc >> 1) & 1u;
                    ok = mbar_wait(&acc_empty[s], par ^ 1u);
                    if (ok) ok = mbar_wait(&b_full[s], par);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t sb = sbase + (uint32_t) G::kOffB + s * G::kStageB;
                    const uint32_t tsfb = tmem + G::kTmemSFB + s * G::kSFBStage;
                    const uint32_t d = tmem + s * 128;
#pragma unroll
                    for (int c = 0; c < KC; ++c)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tsfb + (uint32_t) (16 * c + 4 * k)),
                                         "l"(sf_desc_q(sb + (uint32_t) (c * kBlockF + kATileQ + k * 512)))
                                         : "memory");
                            const uint64_t bd = smem_desc_sw128(sb + (uint32_t) (c * kBlockF) + k * 32);
#pragma unroll
                            for (int t = 0; t < kTermsF; ++t) {
                                const uint32_t accum = (c | k | t) ? 1u : 0u;
                                asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
                                             "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n}\n" ::"r"(d),
                                             "l"(smem_desc_sw128(sbase + (uint32_t) ((c * kTermsF + t) * kATileQ) + k * 32)), "l"(bd), "r"(G::kIdesc),
                                             "r"(tmem + G::kTmemSFA + (uint32_t) (64 * c + 16 * t + 4 * k)), "r"(tsfb + (uint32_t) (16 * c + 4 * k)), "r"(accum)
                                             : "memory");
                            }
                        }
                    umma_commit(&b_empty[s]);
                    umma_commit(&acc_full[s]);
                }
                if (!ok) break;
                umma_commit(a_empty);       // the resident rows may be replaced once every MMA of the tile has read them
                ++ti;
            }
            if (!ok) atomicOr(a.status, 1);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t nbc = 0;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const unsigned long long bp = a.recs[tile].blob;
                if (bp == 0ull) continue;
                const uint8_t* down = reinterpret_cast<const uint8_t*>(bp) + geo.down;
                for (int nb = 0; nb < n_nb; ++nb, ++nbc) {
                    const uint32_t s = nbc & 1u;
                    ok = mbar_wait(&b_empty[s], ((nbc >> 1) & 1u) ^ 1u);
                    if (!ok) break;
                    const uint32_t bar = smem_u32(&b_full[s]);
                    asm volatile("{\n.reg .b64 t;\nmbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1;\n}\n" ::"r"(bar), "r"((uint32_t) G::kStageB) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(sbase + (uint32_t) G::kOffB + s * G::kStageB),
                                 "l"(down + (size_t) nb * G::kStageB), "r"((uint32_t) G::kStageB), "r"(bar)
                                 : "memory");
                }
            }
            if (!ok) atomicOr(a.status, 1);
        }
    } else if (warp <= 5) {
        // ---- the tile's rows (images of dispatch rows row0 ..): codes by 16-byte cp.async, scale words through registers
        const int tl = threadIdx.x - 64;
        const int c8 = tl & 7, r16 = tl >> 3;
        const uint32_t sdst = sbase + (uint32_t) (G::kOffSFA + (tl & 31) * 16 + (tl >> 5) * 4);
        uint32_t ti = 0;
        TileRec rec, nrec;
        int tile = blockIdx.x;
        for (; tile < n_tiles; tile += gridDim.x) {
            rec = a.recs[tile];
            if (rec.blob != 0ull) break;
        }
        while (tile < n_tiles && ok) {
            int ntile = tile + gridDim.x;             // the next tile's record is requested while this one loads
            for (; ntile < n_tiles; ntile += gridDim.x) {
                nrec = a.recs[ntile];
                if (nrec.blob != 0ull) break;
            }
            ok = mbar_wait(a_empty, (ti & 1u) ^ 1u);
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = r16 + 16 * i;
                const int64_t ir = rec.row0 + (r < rec.rows ? r : 0);
                const uint8_t* g = a.codes + (size_t) ir * kTermsF * (size_t) (K >> 1) + c8 * 16;
                const uint32_t dst = sbase + (uint32_t) ((r >> 3) * 1024 + (r & 7) * 128 + ((c8 ^ (r & 7)) << 4));
#pragma unroll
                for (int c = 0; c < KC; ++c)
#pragma unroll
                    for (int t = 0; t < kTermsF; ++t)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + (uint32_t) ((c * kTermsF + t) * kATileQ)),
                                     "l"(g + (size_t) t * (size_t) (K >> 1) + (size_t) c * 128)
                                     : "memory");
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            {
                const int64_t ir = rec.row0 + (tl < rec.rows ? tl : 0);
                const uint8_t* srow = a.sfs + (size_t) ir * kTermsF * (size_t) (K >> 4);
#pragma unroll
                for (int c = 0; c < KC; ++c)
#pragma unroll
                    for (int t = 0; t < kTermsF; ++t) {
                        const uint4 sv = *reinterpret_cast<const uint4*>(srow + (size_t) t * (size_t) (K >> 4) + (size_t) c * 16);
                        const uint32_t w[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            asm volatile("st.shared.u32 [%0], %1;\n" ::"r"(sdst + (uint32_t) (((c * kTermsF + t) * 4 + k) * 512)), "r"(w[k]) : "memory");
                    }
            }
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            mbar_arrive(a_full);
            ++ti;
            tile = ntile;
            rec = nrec;
        }
        if (!ok) atomicOr(a.status, 1);
    } else {
        // ---- epilogue: thread p = tile row p reads TMEM lane p of each finished accumulator (128 down rows at a time)
        const int p = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t) ((warp & 3) * 32) << 16;
        uint32_t nbc = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const TileRec rec = a.recs[tile];
            if (rec.blob == 0ull) continue;
            const bool row_live = p < rec.rows;
            const float* tail = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(rec.blob) + geo.tail);
            const float sd = row_live ? tail[2] * a.inv[rec.row0 + p] : 0.f;
            float* orow = a.dm + (size_t) (rec.row0 + p) * a.L.n_embd;
            for (int nb = 0; nb < n_nb; ++nb, ++nbc) {
                const uint32_t s = nbc & 1u;
                ok = __all_sync(kFull, mbar_wait(&acc_full[s], (nbc >> 1) & 1u));
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t d[32];
                    tmem_ld32(tmem + lane_base + s * 128 + (uint32_t) c0, d);
                    if (row_live) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            reinterpret_cast<float4*>(orow + nb * 128 + c0)[v] = make_float4(__uint_as_float(d[4 * v]) * sd, __uint_as_float(d[4 * v + 1]) * sd,
                                                                                            __uint_as_float(d[4 * v + 2]) * sd, __uint_as_float(d[4 * v + 3]) * sd);
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                mbar_arrive(&acc_empty[s]);
            }
            if (!ok) break;
        }
        if (!ok && lane == 0) atomicOr(a.status, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
    }
}

template <int KC>
int32_t launch_down_resident(const PrefillFArgs& a, cudaStream_t st) {
    static std::atomic<bool> configured[64];   // per device; threads of different devices call concurrently
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_down_resident_kernel<KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) GeoR<KC>::kSmem);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    prefill_down_resident_kernel<KC><<<(unsigned) sm_count(), kThreadsQ, GeoR<KC>::kSmem, st>>>(a);
    return launch_status();
}

size_t al256q(size_t v) { return (v + 255) & ~(size_t) 255; }

template <int MODE>
int32_t launch_q(const PrefillFArgs& a, cudaStream_t st) {
    static std::atomic<bool> configured[64];   // per device; threads of different devices call concurrently
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_nvf4_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) Geo<MODE>::kSmem);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    prefill_nvf4_kernel<MODE><<<(unsigned) sm_count(), kThreadsQ, Geo<MODE>::kSmem, st>>>(a);
    return launch_status();
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_experts_prefill_packed_scratch_bytes(const bsx_expert_layout* L, int64_t n_tokens, int64_t cap_rows) {
    if (!L || n_tokens < 0 || cap_rows < 0 || !bsx_expert_packed_bytes(L)) return 0;
    const size_t H = (size_t) L->n_embd, I = (size_t) L->n_ff, R = (size_t) cap_rows + 128;
    return al256q((size_t) n_tokens * kTermsF * H / 2) + al256q((size_t) n_tokens * kTermsF * H / 16) + al256q((size_t) n_tokens * 4) + al256q(R * I * 4) +
           al256q(R * kTermsF * I / 2) + al256q(R * kTermsF * I / 16) + al256q(R * 4) + al256q(((size_t) cap_rows / 128 + 1025) * sizeof(TileRec)) + 256;
}

extern "C" int32_t bsx_experts_prefill_packed(const bsx_expert_layout* layout, const unsigned long long* blob_table, const int32_t* off,
                                              const int32_t* src, const int32_t* tiles, const int32_t* n_tiles, int64_t cap_tiles, int64_t cap_rows,
                                              const void* x, int32_t x_kind, int64_t n_tokens, int32_t n_expert, void* scratch, float* dm, int32_t* status,
                                              void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout || !blob_table || !off || !src || !tiles || !n_tiles || !aligned(x, 16) || !aligned(scratch, 256) || !aligned(dm, 16) || !status)
        return BSX_E_POINTER;
    if (!bsx_expert_packed_bytes(layout)) return BSX_E_TYPE;
    if (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16) return BSX_E_GEOMETRY;
    if (cap_tiles < 0 || cap_rows < 0 || n_tokens < 0 || n_expert < 1) return BSX_E_GEOMETRY;
    if (cap_tiles == 0 || n_tokens == 0 || cap_rows == 0) return BSX_OK;
    const bsx_expert_layout& L = *layout;
    const cudaStream_t st = (cudaStream_t) stream;
    const size_t H = (size_t) L.n_embd, I = (size_t) L.n_ff, R = (size_t) cap_rows + 128;
    uint8_t* p = static_cast<uint8_t*>(scratch);
    uint8_t* xcodes = p;
    p += al256q((size_t) n_tokens * kTermsF * H / 2);
    uint8_t* xsf = p;
    p += al256q((size_t) n_tokens * kTermsF * H / 16);
    float* xinv = reinterpret_cast<float*>(p);
    p += al256q((size_t) n_tokens * 4);
    float* h = reinterpret_cast<float*>(p);
    p += al256q(R * I * 4);
    uint8_t* hcodes = p;
    p += al256q(R * kTermsF * I / 2);
    uint8_t* hsf = p;
    p += al256q(R * kTermsF * I / 16);
    float* hinv = reinterpret_cast<float*>(p);
    p += al256q(R * 4);
    TileRec* recs = reinterpret_cast<TileRec*>(p);
    if (cap_tiles > cap_rows / 128 + 1025) return BSX_E_LIMIT;      // more tiles than rows / 128 + experts can make
    tile_records_kernel<<<(unsigned) ((cap_tiles + 255) / 256), 256, 0, st>>>(tiles, n_tiles, off, blob_table, recs, cap_tiles);
    PrefillFArgs a;
    a.L = L;
    a.recs = recs;
    a.src = src;
    a.n_tiles = n_tiles;
    a.h = h;
    a.dm = dm;
    a.status = status;
    launch_images<false>(x, x_kind, n_tokens, nullptr, (int64_t) H, xcodes, xsf, xinv, st);
    a.codes = xcodes;
    a.sfs = xsf;
    a.inv = xinv;
    int32_t rc = launch_q<QMODE_GU>(a, st);
    if (rc != BSX_OK) return rc;
    launch_images<true>(h, BSX_X_F32, cap_rows, off + n_expert, (int64_t) I, hcodes, hsf, hinv, st);
    a.codes = hcodes;
    a.sfs = hsf;
    a.inv = hinv;
    // n_ff <= 512: the tile's rows stay in shared memory and only weights stream
    if (I == 256) return launch_down_resident<1>(a, st);
    if (I == 512) return launch_down_resident<2>(a, st);
    return launch_q<QMODE_DOWN>(a, st);
}
