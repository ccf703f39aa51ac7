// experts_prefill.cu - prompt-sized grouped experts for NVFP4 blobs on the 5th-generation tensor cores (tcgen05).
//
// A ragged grouped GEMM over the dispatch's expert-sorted rows: for every 128-row tile of one expert,
//   gate/up:  [128 rows x H] . [H x 2I]  -> SwiGLU ->  h [rows x I]           (fp16, in scratch)
//   down:     [128 rows x I] . [I x H]   ->             dm [rows x H]          (fp32, unweighted, row = dispatch slot)
// which is what Basalt's fp4::run_group computes (include/basalt/prefill/moe_fp4.hpp:43-113, src/prefill/moe_fp4.cu:368-518,
// :654-676) - but that kernel is mma.sync kind::mxf4nvf4 for sm_120a, does not assemble for sm_100, and rounds activations
// to FP4.  Here the NVFP4 weights are decoded EXACTLY to fp16 (E2M1 x UE4M3 has at most 5 significant bits) by the producer
// warps straight into 128-byte-swizzled shared memory, activations are fp16 (bf16 inputs convert exactly after a per-row
// power-of-two scale), and tcgen05.mma kind::f16 accumulates in fp32 in tensor memory.  So the result sits ~2e-4 from the
// dequantised fp32 reference instead of the reference kernel's ~1e-2 .. 0.2, at bf16-class tensor throughput.
//
// Persistent CTAs, one per SM, each looping over work items (128-row tile of one expert, 256 weight rows).  Warp roles:
// warp 0 allocates all 512 TMEM columns (two 256-column accumulators) and its lane 0 issues the MMAs (M = 128, N = 256);
// warps 1-2 load the tile's activation rows (cp.async gather through `src`); warps 3-18 decode NVFP4 weight rows to fp16
// straight into 128-byte-swizzled shared memory (two groups of 256 threads, a thread per weight row, the groups taking
// alternate pairs of 64-column k-blocks); warps 19-22 are the epilogue (thread = TMEM lane = output row), which drains one
// accumulator while the tensor core fills the other.  K-blocks move through a 4-stage ring guarded by mbarriers; every wait
// is bounded and reports through a status word instead of hanging.
//
// Both operands use the SAME permutation of k inside each 16-column group, (0,8,1,9,...,7,15) - the order cvt.e2m1x2 emits
// a sub-block's values in - so no shuffling is needed: the activation image (made by a small kernel here) and the SwiGLU
// output are simply written in that order.
#include <atomic>
#include <cuda_fp16.h>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"
#include "tc5.cuh"

namespace bsx {
namespace {

constexpr int kTileM = 128;        // rows (tokens) per tile = TMEM lanes
constexpr int kTileN = 256;        // weight rows per tile = TMEM columns of one accumulator
constexpr int kBlockK = 64;        // fp16 per k-block: one 128-byte swizzle row
constexpr int kStagesP = 4;
constexpr int kLoaderWarps = 2, kDecoderWarps = 16, kEpilogueWarps = 4;
constexpr int kGroupThreads = 256; // one group of weight decoders: a thread per weight row of the tile
constexpr int kThreadsP = 32 * (1 + kLoaderWarps + kDecoderWarps + kEpilogueWarps);
constexpr float kHScale = 0.25f;   // the SwiGLU output is stored as fp16(h / 4): fp16 then holds |h| up to 2.6e5

enum { PMODE_GU = 0, PMODE_DOWN = 1 };
enum { WT_NVFP4 = 0, WT_Q6K = 1, WT_IQ1M = 2 };      // how the decoder warps read a weight row
constexpr float kWScaleKQ = 16.f;  // K / I-quant weights are stored as fp16(16 w): typical weights (~1e-2) sit well inside fp16's normal range
enum { kStatusTimeout = 1 };

constexpr uint32_t kInstrDesc = instr_desc_f16(kTileM, kTileN);

__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n.reg .b8 b0, b1, b2, b3;\nmov.b32 {b0, b1, b2, b3}, %4;\ncvt.rn.f16x2.e2m1x2 %0, b0;\ncvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\ncvt.rn.f16x2.e2m1x2 %3, b3;\n}\n"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// UE4M3 byte -> fp16 pair {d, d}, d = scale / 2^8 (see experts_mma.cu: the epilogue multiplies by 2^8); 0x7F -> 0
__device__ __forceinline__ uint32_t scale_pair_bits(uint32_t byte) {
    const uint32_t b = byte & 0x7Fu;
    const uint32_t v = b == 0x7Fu ? 0u : b << 7;
    return v | (v << 16);
}

struct PrefillArgs {
    bsx_expert_layout L;
    const unsigned long long* blob_table;   // [E] device addresses
    const int32_t* off;                      // [E + 1] row offsets per expert
    const int32_t* src;                      // [rows] token of each row
    const int32_t* tiles;                    // {expert, first row} per 128-row tile
    const int32_t* n_tiles;
    const __half* xh;                        // [T][H] fp16, permuted, row-scaled
    const float* xinv;                       // [T]
    const uint16_t* grid;                    // the IQ1 codebook on this device
    __half* h;                               // [rows][I] fp16 (permuted, times kHScale)
    float* dm;                               // [rows][H] fp32
    int32_t* status;                         // sticky error word (0 = ok)
};

// x [T][H] (fp32 or bf16) -> fp16 rows scaled by a power of two into fp16's range, k-permuted inside 16-column groups
__global__ void __launch_bounds__(256) prefill_prep_x_kernel(const void* __restrict__ x, int kind, int64_t T, int64_t H, __half* __restrict__ xh,
                                                             float* __restrict__ xinv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = (int64_t) blockIdx.x * 8 + warp;
    if (t >= T) return;
    auto ld = [&](int64_t c) {
        return kind == BSX_X_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(x)[t * H + c]) : static_cast<const float*>(x)[t * H + c];
    };
    float amax = 0.f;
    for (int64_t c = lane; c < H; c += 32) amax = fmaxf(amax, fabsf(ld(c)));
    amax = warp_max_xor(amax);
    int ex = 0;
    float s = 1.f, iv = 1.f;
    if (amax > 0.f && amax <= 3.0e38f) {
        frexpf(amax, &ex);
        ex = max(-100, min(100, 14 - ex));
        s = ldexpf(1.f, ex);
        iv = ldexpf(1.f, -ex);
    }
    if (lane == 0) xinv[t] = iv;
    for (int64_t c = lane; c < H; c += 32) xh[t * H + (c & ~(int64_t) 15) + perm16((int) (c & 15))] = __float2half_rn(ld(c) * s);
}

template <int MODE, bool ALIGNED, int WT>
__global__ void __launch_bounds__(kThreadsP, 1) prefill_gemm_kernel(PrefillArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte aligned operand stages: A then B per stage
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    constexpr int kABytes = kTileM * kBlockK * 2, kBBytes = kTileN * kBlockK * 2, kStage = kABytes + kBBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStagesP * kStage);
    uint64_t* full = bars;                        // [S] loader lanes + one decoder group arrive
    uint64_t* empty = bars + kStagesP;            // [S] tcgen05.commit arrives
    uint64_t* acc_full = bars + 2 * kStagesP;     // [2] tcgen05.commit after a tile's last MMA
    uint64_t* acc_empty = acc_full + 2;           // [2] the 128 epilogue threads arrive
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    uint32_t* lut = tmem_slot + 2;                // [256] fp16 scale pairs
    uint16_t* s_grid = reinterpret_cast<uint16_t*>(lut + 256);   // [2048] the IQ1 codebook (IQ1_M rows only)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t K = MODE == PMODE_GU ? a.L.n_embd : a.L.n_ff;
    const int nkb = (int) (K / kBlockK);
    const int n_out = MODE == PMODE_GU ? (int) a.L.n_ff : (int) a.L.n_embd;      // neurons, or down rows
    constexpr int kOutPerTile = MODE == PMODE_GU ? kTileN / 2 : kTileN;
    const int n_n = (n_out + kOutPerTile - 1) / kOutPerTile;
    const int n_items = *a.n_tiles * n_n;

    for (int i = threadIdx.x; i < 256; i += kThreadsP) lut[i] = scale_pair_bits(i);
    if (WT == WT_IQ1M)
        for (int i = threadIdx.x; i < 2048; i += kThreadsP) s_grid[i] = a.grid[i];
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesP; ++s) {
            mbar_init(&full[s], kGroupThreads + 32 * kLoaderWarps);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 32 * kEpilogueWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();   // lane 0 initialised the barriers above: reconverge before the warp-wide allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    bool ok = true;

    // A work item: tile = item / n_n (expert, first row), weight rows n0 = (item % n_n) * kOutPerTile ...; every role walks the
    // same item sequence and skips the same items (experts another device holds), so their k-block counters stay in step.
    struct Item { const uint8_t* blob; int row0, rows, n0; };
    auto get_item = [&](int item, Item& it) -> bool {
        const int tile = item / n_n;
        const int expert = a.tiles[2 * tile];
        const unsigned long long bp = a.blob_table[expert];
        if (bp == 0ull) return false;
        it.blob = reinterpret_cast<const uint8_t*>(bp);
        it.row0 = a.tiles[2 * tile + 1];
        it.rows = min(kTileM, a.off[expert + 1] - it.row0);
        it.n0 = (item - tile * n_n) * kOutPerTile;
        return true;
    };

    if (warp == 0) {
        // ---- MMA issuer: one lane feeds the tensor core, four k = 16 instructions per 64-column k-block
        if (lane == 0) {
            uint32_t kc = 0, ti = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                Item it;
                if (!get_item(item, it)) continue;
                const uint32_t acc = ti & 1u;
                ok = mbar_wait(&acc_empty[acc], ((ti >> 1) & 1u) ^ 1u);     // the epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                for (int kb = 0; kb < nkb; ++kb, ++kc) {
                    const uint32_t s = kc % kStagesP;
                    ok = mbar_wait(&full[s], (kc / kStagesP) & 1u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t sa = smem_u32(smem + s * kStage), sb = sa + kABytes;
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)
                        umma_f16(tmem + acc * kTileN, smem_desc_sw128(sa + k * 32), smem_desc_sw128(sb + k * 32), kInstrDesc, (kb | k) ? 1u : 0u);
                    umma_commit(&empty[s]);      // the stage may be refilled once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[acc]);     // fires when every MMA of the tile has finished
                ++ti;
            }
            if (!ok) atomicOr(a.status, kStatusTimeout);
        }
    } else if (warp <= kLoaderWarps) {
        // ---- activation loaders.  Lane l of loader warp w copies 16-byte chunk l % 8 of rows 64 w + l / 8 + 4 i: eight lanes
        // cover one row's 128 bytes.  Rows past the expert's last row read some valid row instead (never stored).  A lane
        // runs up to two k-blocks ahead of its own completed copies and arrives on a stage once its copies there landed.
        const int lw = warp - 1, c = lane & 7, r4 = lane >> 3;
        const uint8_t* abase = reinterpret_cast<const uint8_t*>(MODE == PMODE_GU ? a.xh : a.h);
        uint32_t dsto[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r7 = 4 * h + r4;
            dsto[h] = (uint32_t) (lw * 8 * 1024 + r7 * 128 + ((c ^ r7) << 4));
        }
        uint32_t issued = 0, arrived = 0;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            Item it;
            if (!get_item(item, it)) continue;
            uint32_t aoff[16];   // row starts in 16-byte units
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int r = lw * 64 + 4 * i + r4;
                const uint32_t grow = MODE == PMODE_GU ? (uint32_t) a.src[it.row0 + (r < it.rows ? r : 0)] : (uint32_t) (it.row0 + r);
                aoff[i] = grow * (uint32_t) (K >> 3) + (uint32_t) c;
            }
            for (int kb = 0; kb < nkb; ++kb) {
                const uint32_t s = issued % kStagesP;
                ok = mbar_wait(&empty[s], ((issued / kStagesP) & 1u) ^ 1u);
                if (!ok) break;
                const uint32_t dst = smem_u32(smem + s * kStage);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const uint8_t* g = abase + ((size_t) aoff[i] + (size_t) kb * 8) * 16;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + (uint32_t) ((i >> 1) * 1024) + dsto[i & 1]), "l"(g) : "memory");
                }
                asm volatile("cp.async.commit_group;\n" ::: "memory");
                ++issued;
                if (issued - arrived > 2) {
                    asm volatile("cp.async.wait_group 2;\n" ::: "memory");
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    mbar_arrive(&full[arrived % kStagesP]);
                    ++arrived;
                }
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        for (; arrived < issued; ++arrived) mbar_arrive(&full[arrived % kStagesP]);
        if (!ok) atomicOr(a.status, kStatusTimeout);
    } else if (warp <= kLoaderWarps + kDecoderWarps) {
        // ---- weight decoders: thread (group, row r) turns the NVFP4 blocks of weight row r of the tile into fp16 B-tile rows
        const int td = threadIdx.x - 32 * (1 + kLoaderWarps);
        const int grp = td >> 8, r = td & 255;
        const uint32_t swz = (uint32_t) (r & 7);
        const uint32_t row_off = (uint32_t) (kABytes + (r >> 3) * 1024 + (r & 7) * 128);
        auto weight_row = [&](const Item& it) -> const uint8_t* {
            if (MODE == PMODE_GU) {     // B rows 0..127 = gate rows, 128..255 = the matching up rows
                const int n = min(it.n0 + (r & 127), n_out - 1);
                return r < 128 ? it.blob + (size_t) n * a.L.gu_row : it.blob + a.L.up_off + (size_t) n * a.L.up_row;
            }
            return it.blob + a.L.down_off + (size_t) min(it.n0 + r, n_out - 1) * a.L.d_row;
        };
        // one NVFP4 block (9 words: 4 scale bytes, 32 code bytes) -> 64 fp16 of the B tile, already in the permuted k order
        auto store_b = [&](uint32_t s, const uint32_t* cur) {
            uint4* brow = reinterpret_cast<uint4*>(smem + s * kStage + row_off);
#pragma unroll
            for (int sub = 0; sub < 4; ++sub) {
                const uint32_t sc = lut[(cur[0] >> (8 * sub)) & 0xFFu];
                uint32_t q0[4], q1[4];
                cvt_e2m1x8(cur[1 + 2 * sub], q0);
                cvt_e2m1x8(cur[2 + 2 * sub], q1);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    q0[i] = hmul2_bits(q0[i], sc);
                    q1[i] = hmul2_bits(q1[i], sc);
                }
                brow[(2 * sub) ^ swz] = make_uint4(q0[0], q0[1], q0[2], q0[3]);
                brow[(2 * sub + 1) ^ swz] = make_uint4(q1[0], q1[1], q1[2], q1[3]);
            }
        };
        // the pair of blocks q (k-blocks 2q, 2q + 1): 72 bytes at offset 72 q of the row; 16-byte loads when rows are whole
        // 144-byte chunks (then 72 q is a multiple of 16 for even q and of 8 for odd q)
        const int npair = (nkb + 1) >> 1;
        auto load_pair = [&](const uint8_t* wrow, int q, uint32_t (&w)[18]) {
            const uint8_t* src = wrow + (size_t) q * 72;
            if (ALIGNED) {
                if ((q & 1) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 v = reinterpret_cast<const uint4*>(src)[i];
                        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
                    }
                    const uint2 t = reinterpret_cast<const uint2*>(src)[8];
                    w[16] = t.x; w[17] = t.y;
                } else {
                    const uint2 t = reinterpret_cast<const uint2*>(src)[0];
                    w[0] = t.x; w[1] = t.y;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 v = reinterpret_cast<const uint4*>(src + 8)[i];
                        w[2 + 4 * i] = v.x; w[3 + 4 * i] = v.y; w[4 + 4 * i] = v.z; w[5 + 4 * i] = v.w;
                    }
                }
            } else {
                const int nw = 2 * q + 1 < nkb ? 18 : 9;
#pragma unroll
                for (int i = 0; i < 18; ++i) w[i] = i < nw ? reinterpret_cast<const uint32_t*>(src)[i] : 0u;
            }
        };
        if constexpr (WT == WT_NVFP4) {
            // the stream of own pairs runs across items: the first pair of the next item is requested while the last pair of this
            // one is decoded, so a tile switch does not expose a load
            uint32_t wc[18], wn[18];
            uint32_t kc = 0;
            int item = blockIdx.x;
            Item it;
            while (item < n_items && !get_item(item, it)) item += gridDim.x;
            if (item < n_items && grp < npair) load_pair(weight_row(it), grp, wn);
            while (item < n_items && ok) {
                const uint8_t* wrow = weight_row(it);
                int nxt = item + gridDim.x;
                Item itn;
                while (nxt < n_items && !get_item(nxt, itn)) nxt += gridDim.x;
                for (int q = grp; q < npair && ok; q += 2) {
#pragma unroll
                    for (int i = 0; i < 18; ++i) wc[i] = wn[i];
                    if (q + 2 < npair) load_pair(wrow, q + 2, wn);
                    else if (nxt < n_items) load_pair(weight_row(itn), grp, wn);
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int kb = 2 * q + j;
                        if (kb < nkb && ok) {
                            const uint32_t kk = kc + (uint32_t) kb, s = kk % kStagesP;
                            ok = mbar_wait(&empty[s], ((kk / kStagesP) & 1u) ^ 1u);
                            if (ok) {
                                store_b(s, &wc[9 * j]);
                                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> visible to the tensor core
                                mbar_arrive(&full[s]);
                            }
                        }
                    }
                }
                kc += (uint32_t) nkb;
                item = nxt;
                it = itn;
            }
        } else {
            // K- and I-quant rows (Q6_K: 210 bytes per 256 values, IQ1_M: 56): the thread decodes its row's 64 values of a k-block
            // exactly (formats.cuh), stores them as fp16(16 w) - the rounding, 2^-11 relative, is the only one - in the permuted
            // k order, and hands the stage over.  The decode runs before the wait for the stage, so it overlaps the tensor core.
            constexpr int kBB = WT == WT_Q6K ? 210 : 56;
            uint32_t kc = 0;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                Item it;
                if (!get_item(item, it)) continue;
                const uint8_t* wrow = weight_row(it);
                for (int q = grp; q < npair && ok; q += 2) {
#pragma unroll 1
                    for (int j = 0; j < 2; ++j) {
                        const int kb = 2 * q + j;
                        if (kb >= nkb || !ok) continue;
                        float v[64];
                        const uint8_t* blk = wrow + (size_t) (kb >> 2) * kBB;
                        const int u0 = 2 * (kb & 3);
                        if (WT == WT_Q6K) {
                            decode_q6k_32(blk, u0, v);
                            decode_q6k_32(blk, u0 + 1, v + 32);
                        } else {
                            decode_iq1m_32(blk, u0, s_grid, v);
                            decode_iq1m_32(blk, u0 + 1, s_grid, v + 32);
                        }
                        const uint32_t kk = kc + (uint32_t) kb, s = kk % kStagesP;
                        ok = mbar_wait(&empty[s], ((kk / kStagesP) & 1u) ^ 1u);
                        if (!ok) break;
                        uint4* brow = reinterpret_cast<uint4*>(smem + s * kStage + row_off);
#pragma unroll
                        for (int sub = 0; sub < 4; ++sub) {
                            const float* w = v + 16 * sub;
                            uint32_t p0[4], p1[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const __half2 a2 = __floats2half2_rn(w[i] * kWScaleKQ, w[i + 8] * kWScaleKQ);
                                const __half2 b2 = __floats2half2_rn(w[4 + i] * kWScaleKQ, w[12 + i] * kWScaleKQ);
                                p0[i] = *reinterpret_cast<const uint32_t*>(&a2);
                                p1[i] = *reinterpret_cast<const uint32_t*>(&b2);
                            }
                            brow[(2 * sub) ^ swz] = make_uint4(p0[0], p0[1], p0[2], p0[3]);
                            brow[(2 * sub + 1) ^ swz] = make_uint4(p1[0], p1[1], p1[2], p1[3]);
                        }
                        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                        mbar_arrive(&full[s]);
                    }
                }
                kc += (uint32_t) nkb;
            }
        }
        if (!ok) atomicOr(a.status, kStatusTimeout);
    } else {
        // ---- epilogue: thread p reads TMEM lane p (= output row p) of the finished accumulator.  A warp may only read the 32
        // TMEM lanes 32 (warp % 4) .. + 31.  tcgen05.ld is warp-wide: every lane runs the loads; only the stores are predicated.
        const int p = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t) ((warp & 3) * 32) << 16;
        uint32_t ti = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            Item it;
            if (!get_item(item, it)) continue;
            const uint32_t acc = ti & 1u;
            ok = __all_sync(kFull, mbar_wait(&acc_full[acc], (ti >> 1) & 1u));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const bool row_live = p < it.rows;
            // NVFP4 blobs end in {s_gate, s_up, s_down, 0}; the block scales were used as scale / 2^8.  K / I-quant rows have no
            // tail and were stored as 16 w.
            const bool nv_tail = a.L.gu_type == kTypeNVFP4;
            const float* tail = reinterpret_cast<const float*>(it.blob + a.L.bytes - 16);
            constexpr float kUnscale = WT == WT_NVFP4 ? 256.f : 1.f / kWScaleKQ;
            const uint32_t tbase = tmem + lane_base + acc * kTileN;
            if (MODE == PMODE_GU) {
                const float f = row_live ? a.xinv[a.src[it.row0 + p]] * kUnscale : 0.f;
                const float sg = (nv_tail ? tail[0] : 1.f) * f, su = (nv_tail ? tail[1] : 1.f) * f;
                __half* hrow = a.h + (size_t) (it.row0 + p) * a.L.n_ff + it.n0;
#pragma unroll 1
                for (int c0 = 0; c0 < kTileN / 2; c0 += 16) {
                    uint32_t g[16], u[16];
                    tmem_ld16(tbase + (uint32_t) c0, g);
                    tmem_ld16(tbase + (uint32_t) (kTileN / 2 + c0), u);
                    __half out[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float hv = swiglu(__uint_as_float(g[j]) * sg, __uint_as_float(u[j]) * su, a.L) * kHScale;
                        out[perm16(j)] = __float2half_rn(fminf(fmaxf(hv, -65504.f), 65504.f));
                    }
                    if (row_live && it.n0 + c0 < n_out) {
                        reinterpret_cast<uint4*>(hrow + c0)[0] = reinterpret_cast<const uint4*>(out)[0];
                        reinterpret_cast<uint4*>(hrow + c0)[1] = reinterpret_cast<const uint4*>(out)[1];
                    }
                }
            } else {
                const float f = (nv_tail ? tail[2] : 1.f) * (kUnscale / kHScale);
                float* orow = a.dm + (size_t) (it.row0 + p) * a.L.n_embd + it.n0;
#pragma unroll 1
                for (int c0 = 0; c0 < kTileN; c0 += 32) {
                    uint32_t d[32];
                    tmem_ld32(tbase + (uint32_t) c0, d);
                    if (row_live && it.n0 + c0 < n_out) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            reinterpret_cast<float4*>(orow + c0)[v] = make_float4(__uint_as_float(d[4 * v]) * f, __uint_as_float(d[4 * v + 1]) * f,
                                                                                 __uint_as_float(d[4 * v + 2]) * f, __uint_as_float(d[4 * v + 3]) * f);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(&acc_empty[acc]);
            ++ti;
        }
        if (!ok && lane == 0) atomicOr(a.status, kStatusTimeout);
    }
    // everyone is done with tensor memory before warp 0 gives it back
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
    }
}

size_t align256p(size_t v) { return (v + 255) & ~(size_t) 255; }
constexpr size_t kSmemP = 1024 + kStagesP * (kTileM * kBlockK * 2 + kTileN * kBlockK * 2) + 256 + 1024 + 4096 + 64;   // 203,136 bytes: one CTA per SM

int wt_of(int type) { return type == kTypeNVFP4 ? WT_NVFP4 : type == kTypeQ6K ? WT_Q6K : type == kTypeIQ1M ? WT_IQ1M : -1; }

template <int MODE, bool ALIGNED, int WT>
cudaError_t configure_one() { return cudaFuncSetAttribute(prefill_gemm_kernel<MODE, ALIGNED, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) kSmemP); }

template <int MODE>
void launch_mode(int wt, bool aligned16, unsigned grid, const PrefillArgs& a, cudaStream_t st) {
    if (wt == WT_NVFP4) {
        if (aligned16) prefill_gemm_kernel<MODE, true, WT_NVFP4><<<grid, kThreadsP, kSmemP, st>>>(a);
        else prefill_gemm_kernel<MODE, false, WT_NVFP4><<<grid, kThreadsP, kSmemP, st>>>(a);
    } else if (wt == WT_Q6K) {
        prefill_gemm_kernel<MODE, false, WT_Q6K><<<grid, kThreadsP, kSmemP, st>>>(a);
    } else {
        prefill_gemm_kernel<MODE, false, WT_IQ1M><<<grid, kThreadsP, kSmemP, st>>>(a);
    }
}

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_experts_prefill_scratch_bytes(const bsx_expert_layout* L, int64_t n_tokens, int64_t cap_rows) {
    if (!L || n_tokens < 0 || cap_rows < 0) return 0;
    return align256p((size_t) n_tokens * L->n_embd * 2) + align256p((size_t) n_tokens * 4) + align256p((size_t) (cap_rows + kTileM) * L->n_ff * 2) + 256;
}

extern "C" int32_t bsx_experts_prefill(const bsx_expert_layout* layout, const unsigned long long* blob_table, const int32_t* off,
                                       const int32_t* src, const int32_t* tiles, const int32_t* n_tiles, int64_t cap_tiles, int64_t cap_rows,
                                       const void* x, int32_t x_kind, int64_t n_tokens, void* scratch, float* dm, int32_t* status, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (!layout || !blob_table || !off || !src || !tiles || !n_tiles || !aligned(x, 16) || !aligned(scratch, 256) || !aligned(dm, 16) || !status)
        return BSX_E_POINTER;
    const bsx_expert_layout& L = *layout;
    const int wt_gu = wt_of(L.gu_type), wt_d = wt_of(L.d_type);
    if (wt_gu < 0 || wt_d < 0 || L.up_type != L.gu_type) return BSX_E_TYPE;       // NVFP4, Q6_K or IQ1_M; gate and up of one format
    if ((L.gu_type == kTypeNVFP4) != (L.d_type == kTypeNVFP4) && L.gu_type == kTypeNVFP4) return BSX_E_TYPE;   // an NVFP4 tail needs NVFP4 gate / up
    if (L.n_embd % 64 || L.n_ff % 64 || (x_kind != BSX_X_F32 && x_kind != BSX_X_BF16)) return BSX_E_GEOMETRY;
    if ((wt_gu != WT_NVFP4 && L.n_embd % 256) || (wt_d != WT_NVFP4 && L.n_ff % 256)) return BSX_E_GEOMETRY;   // whole 256-value blocks
    if (cap_tiles < 0 || cap_tiles > 65535 || cap_rows < 0 || n_tokens < 0) return BSX_E_GEOMETRY;
    if (cap_tiles == 0 || n_tokens == 0) return BSX_OK;
    const cudaStream_t st = (cudaStream_t) stream;
    uint8_t* p = static_cast<uint8_t*>(scratch);
    PrefillArgs a;
    a.L = L;
    a.blob_table = blob_table;
    a.off = off;
    a.src = src;
    a.tiles = tiles;
    a.n_tiles = n_tiles;
    __half* xh = reinterpret_cast<__half*>(p);
    p += align256p((size_t) n_tokens * L.n_embd * 2);
    float* xinv = reinterpret_cast<float*>(p);
    p += align256p((size_t) n_tokens * 4);
    a.xh = xh;
    a.xinv = xinv;
    a.grid = iq1_device_grid();
    if (!a.grid) return (int32_t) cudaErrorInvalidSymbol;
    a.h = reinterpret_cast<__half*>(p);
    a.dm = dm;
    a.status = status;
    static std::atomic<bool> configured[64];   // per device; threads of different devices call concurrently
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        cudaError_t e = configure_one<PMODE_GU, true, WT_NVFP4>();
        if (e == cudaSuccess) e = configure_one<PMODE_GU, false, WT_NVFP4>();
        if (e == cudaSuccess) e = configure_one<PMODE_DOWN, true, WT_NVFP4>();
        if (e == cudaSuccess) e = configure_one<PMODE_DOWN, false, WT_NVFP4>();
        if (e == cudaSuccess) e = configure_one<PMODE_GU, false, WT_Q6K>();
        if (e == cudaSuccess) e = configure_one<PMODE_DOWN, false, WT_Q6K>();
        if (e == cudaSuccess) e = configure_one<PMODE_GU, false, WT_IQ1M>();
        if (e == cudaSuccess) e = configure_one<PMODE_DOWN, false, WT_IQ1M>();
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    prefill_prep_x_kernel<<<(unsigned) ((n_tokens + 7) / 8), 256, 0, st>>>(x, x_kind, n_tokens, L.n_embd, xh, xinv);
    // persistent CTAs, one per SM; rows that are whole 144-byte chunks (K % 256 == 0) take the variant with 16-byte weight loads
    const unsigned grid = (unsigned) sm_count();
    launch_mode<PMODE_GU>(wt_gu, L.n_embd % 256 == 0, grid, a, st);
    launch_mode<PMODE_DOWN>(wt_d, L.n_ff % 256 == 0, grid, a, st);
    return launch_status();
}
