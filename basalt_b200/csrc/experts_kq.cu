// experts_kq.cu - decode-sized grouped experts for the ggml K- and I-quant formats (Q6_K, IQ1_M) read in place: a bandwidth-bound
// weight stream through shared memory with the dot products on the integer tensor cores.
//
// Why integers.  At 1.75 bits a weight (IQ1_M) the stream is so dense that the decode instructions, not HBM, set the pace: a
// warp-per-row fp32 kernel spends ~8 instructions on every weight.  Here a weight costs about two: the codes stay small
// integers, the activations become int8 too, and mma.sync m16n8k32 (u8 x s8 -> s32) does the multiplying.
//   * Activations: a row x becomes two int8 terms under one scale per row, x s ~ q1 + q2 / 254 (|q| <= 127), so the rounding
//     error is ~1e-4 of the row's norm (one int8 term, what Basalt's q8_1 rows carry, would leave ~1e-2).  A pass multiplies 4
//     entries x 2 terms = the 8 columns of the MMA.
//   * IQ1_M (include/basalt/ggml/ggml_common.h:350-362, decode rule src/kernels/cpu/ggml/ggml_quants.c:1266-1314): a weight is
//     d m (g + delta) with g in {-1, 0, 1} from the 2048-point codebook, m = 2 s + 1 (3-bit s per 16 weights), delta = +-1/8
//     per 8 weights, d an fp16 per 256.  With c = g + 1 in {0, 1, 2}:  8 w / d = 8 m c - m (8 -+ 1).  The first term is the
//     MMA operand (one table word per 8 weights gives their c as nibbles; times m they stay below 31); the second is
//     constant over a group of 8, so it multiplies the group's activation SUM: one more k-step per 256 weights whose operands
//     are the 32 group coefficients m (8 -+ 1) <= 135 (u8) and the 32 negated group sums split as 16 hi + lo (s8 each).
//     Everything up to the factor d / 8 is exact integer arithmetic.
//   * Q6_K (ggml_common.h:279-285, ggml_quants.c:1048-1075): a weight is d sc (q - 32), sc an int8 per 16 weights: one
//     m16n8k16 s8 MMA per scale group, its int32 result scaled by d sc in fp32.
// Each warp owns 16 weight rows (8 gate rows with their 8 up rows, so SwiGLU stays in the thread; or 16 down rows) and
// streams them through its own cp.async ring in chunks of 512 columns; a block's warps share the pass's activation columns.
// Blocks are persistent and draw (pass, row block) units from a counter.
//
// Semantics: Basalt's native_expert_grouped (include/basalt/kernels/iq_kernels.hpp:77-92; its IQ1_M dot src/kernels/cuda/
// iq_kernels.cu:227-257 with the grid table staged in shared memory :1516-1521), minus the single-term q8_1 rounding.
#include <atomic>

#include <cuda_fp16.h>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"
#include "pdl.cuh"

namespace bsx {
namespace {

constexpr int kRowsQ = 16;      // weight rows per warp tile
constexpr int kColsQ = 8;       // MMA n: 4 entries x 2 int8 terms
constexpr int kEntQ = 4;
constexpr float kTerm2 = 1.0f / 254.0f;

enum { QMODE_GU = 0, QMODE_DOWN = 1 };

template <int TYPE> struct QT;
template <> struct QT<kTypeIQ1M> {
    static constexpr int kBlock = 56, kWarps = 16, kStages = 3, kPiece = 16, kPad = 32;
    static constexpr bool kCorr = true;
};
template <> struct QT<kTypeQ6K> {
    static constexpr int kBlock = 210, kWarps = 8, kStages = 3, kPiece = 4, kPad = 16;
    static constexpr bool kCorr = false;
};
constexpr int kChunkBlocks = 2;   // 512 columns a stage

__device__ __forceinline__ void cpa16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cpa4(uint32_t dst, const void* src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// D (16 x 8, s32) += A (16 x 32, u8, row) x B (32 x 8, s8, col)
__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D (16 x 8, s32) = A (16 x 16, s8, row) x B (16 x 8, s8, col)
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// ---------------------------------------------------------------- activation images
// One warp per image row: the row as two int8 terms under one scale, x s ~ q1 + q2 / 254, s = 127 / max|x|; inv[row] = 1 / s.
// Layout: img[row][term][K] int8 in column order.  CORR (IQ1_M): per 256 columns the 32 negated group-of-8 sums of each term as
// 16 hi + lo, corr[row][term][K / 256][hi 32 bytes | lo 32 bytes], a group at the byte its coefficient has in the A fragment:
// group 4 u + t (u = 32-column unit, t = group inside it) -> byte 4 t + p (u < 4) or 16 + 4 t + p with p = 0, 2, 1, 3 for
// u % 4 = 0, 1, 2, 3 (the order in which the product kernel can assemble the coefficients cheaply).
// FROM_H = false: rows of x (row i of x when the caller gave the number of x rows, else the row of entry i); true: row e of
// the SwiGLU output.  The last block lists the passes (up to 4 consecutive entries of a group) and zeroes the work counter.
template <bool FROM_H, bool CORR>
__global__ void __launch_bounds__(256)
kq_image_kernel(ExpertArgs a, int8_t* __restrict__ img, int8_t* __restrict__ corr, float* __restrict__ inv, int2* __restrict__ items,
                int* __restrict__ n_items) {
    pdl_wait();
    pdl_launch_dependents();
    const int ng = min(*a.n_groups, (int) a.cap_groups);
    const int total = min(a.grp_start[ng], (int) a.cap_entries);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x == gridDim.x - 1) {
        __shared__ int sh[8];
        __shared__ int s_base;
        if (threadIdx.x == 0) s_base = 0;
        __syncthreads();
        for (int g0 = 0; g0 < ng; g0 += 256) {
            const int g = g0 + threadIdx.x;
            const int s0 = g < ng ? a.grp_start[g] : 0;
            const int cnt = g < ng ? max(0, min(a.grp_start[g + 1], (int) a.cap_entries) - s0) : 0;
            const int np = (cnt + kEntQ - 1) / kEntQ;
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
            for (int p = 0; p < np; ++p) items[before + x - np + p] = make_int2(g, s0 + p * kEntQ);
            __syncthreads();
            if (threadIdx.x == 255) s_base = before + x;
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            n_items[0] = s_base;
            n_items[1] = 0;
        }
        return;
    }
    const int i = blockIdx.x * 8 + warp;
    const int n_img = FROM_H ? total : (a.n_x_rows > 0 ? a.n_x_rows : total);
    if (i >= n_img) return;
    const int64_t K = FROM_H ? a.L.n_ff : a.L.n_embd;
    const int64_t row = FROM_H ? (int64_t) i : (a.n_x_rows > 0 ? (int64_t) i : (int64_t) a.ent_tok[i]);
    const void* src = FROM_H ? (const void*) a.h : a.x;
    const int kind = FROM_H ? BSX_X_F32 : a.x_kind;
    const int n_sb = (int) (K >> 4);
    float amax = 0.f;
    for (int sb = lane; sb < n_sb; sb += 32) {
        float v[16];
        load16(src, kind, row, K, sb, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = warp_max_xor(amax);
    float s = 1.f, iv = 1.f;
    if (amax > 0.f && amax <= 3.0e38f) {
        s = 127.f / amax;
        iv = amax / 127.f;
    }
    if (lane == 0) inv[i] = iv;
    const int nblk = (int) (K >> 8);
    int8_t* q1 = img + (size_t) i * 2 * K;
    int8_t* q2 = q1 + K;
    for (int sb = lane; sb < n_sb; sb += 32) {
        float v[16];
        load16(src, kind, row, K, sb, v);
        uint32_t w1[4], w2[4];
        int sum1[2] = {0, 0}, sum2[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float xs = v[j] * s;
            int a1 = __float2int_rn(xs);
            a1 = max(-127, min(127, a1));
            int a2 = __float2int_rn((xs - (float) a1) * 254.f);
            a2 = max(-127, min(127, a2));
            if ((j & 3) == 0) { w1[j >> 2] = 0u; w2[j >> 2] = 0u; }
            w1[j >> 2] |= (uint32_t) (a1 & 0xFF) << (8 * (j & 3));
            w2[j >> 2] |= (uint32_t) (a2 & 0xFF) << (8 * (j & 3));
            sum1[j >> 3] += a1;
            sum2[j >> 3] += a2;
        }
        reinterpret_cast<uint4*>(q1)[sb] = make_uint4(w1[0], w1[1], w1[2], w1[3]);
        reinterpret_cast<uint4*>(q2)[sb] = make_uint4(w2[0], w2[1], w2[2], w2[3]);
        if (CORR) {
            const int blk = sb >> 4;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int gi = ((sb & 15) << 1) + h;               // group inside the 256-column block
                const int u = gi >> 2, t = gi & 3;
                const int pos = ((u & 1) << 1) | ((u >> 1) & 1);      // units (0, 1, 2, 3) of a half sit in bytes (0, 2, 1, 3)
                const int slot = (u < 4 ? 0 : 16) + 4 * t + pos;
#pragma unroll
                for (int term = 0; term < 2; ++term) {
                    const int neg = -(term ? sum2[h] : sum1[h]);
                    const int hi = neg >> 4, lo = neg & 15;       // neg = 16 hi + lo, 0 <= lo < 16 (arithmetic shift floors)
                    int8_t* c = corr + (((size_t) i * 2 + term) * nblk + blk) * 64;
                    c[slot] = (int8_t) hi;
                    c[32 + slot] = (int8_t) lo;
                }
            }
        }
    }
}

// ---------------------------------------------------------------- block decoders
// IQ1_M: one 256-weight block of rows g and g + 8 (raw 56-byte blocks ra, rb in shared memory, 8-byte aligned) against the 8
// activation columns; adds d / 8-scaled... the caller scales: tot[i] += I[i] * d[row] where I is the exact integer
// 8 m c q - coefficient sums described at the top.  bcol: this lane's column, at the block's first byte plus 8 t;
// ccol: the column's 64 correction bytes of this block.
__device__ __forceinline__ void iq1m_block(const uint8_t* ra, const uint8_t* rb, const uint2* __restrict__ tab, const uint8_t* bcol,
                                           const uint8_t* ccol, int t, float (&tot)[4]) {
    uint32_t wa[14], wb[14];
#pragma unroll
    for (int i = 0; i < 7; ++i) {
        const uint2 va = reinterpret_cast<const uint2*>(ra)[i], vb = reinterpret_cast<const uint2*>(rb)[i];
        wa[2 * i] = va.x; wa[2 * i + 1] = va.y;
        wb[2 * i] = vb.x; wb[2 * i + 1] = vb.y;
    }
    // words 0-7: qs (unit u = bytes 4u..4u+3), 8-11: qh (unit u = bytes 2u, 2u+1; group t = nibble t), 12-13: four scale words
    int acc[4] = {0, 0, 0, 0};
    const uint32_t sel = 0x4440u | (uint32_t) t;     // byte t of a word, zero-extended
    const int s4 = 4 * t, s3 = 3 * (t >> 1);
    uint32_t msum[4] = {0u, 0u, 0u, 0u};              // the groups' scales m as bytes, in the correction operand's order (below)
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        uint32_t a[4];
        constexpr int kPos[4] = {0, 2, 1, 3};        // unit u of a half sits in byte kPos[u & 3] of that half's correction word
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t* w = r ? wb : wa;
            const uint32_t qsb = __byte_perm(w[u], 0u, sel);
            const uint32_t nib = (w[8 + (u >> 1)] >> (16 * (u & 1) + s4)) & 0xFu;
            const uint2 e = tab[nib * 256u + qsb];                                         // 12-bit index: the delta bit rides along
            const uint32_t sw = w[12 + (u >> 2)] >> s3;                                    // the thread's scale field of unit u now sits at a fixed bit
            const int fb = 16 * ((u >> 1) & 1) + 6 * (u & 1);
            const uint32_t m = fb > 0 ? (((sw >> (fb - 1)) & 14u) | 1u) : (((sw << 1) & 14u) | 1u);   // 2 s + 1
            a[r] = e.x * m;
            a[2 + r] = e.y * m;
            msum[(u < 4 ? 0 : 2) + r] += m << (8 * kPos[u & 3]);
        }
        const uint2 b = *reinterpret_cast<const uint2*>(bcol + 32 * u);
        mma_u8s8_k32(acc, a[0], a[1], a[2], a[3], b.x, b.y);
    }
    // the correction operand: byte = m (8 - 8 delta) = 7 m + 2 m [delta = -1/8], four groups at a time.  The delta bits of units
    // (0, 1) are bits 4t+3 and 4t+19 of qh word 0, of units (2, 3) the same bits of qh word 1: shifted and merged they land in bytes
    // 0, 2 and 1, 3 - the order kPos gives the scales.
    uint32_t ca[4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t* w = r ? wb : wa;
        const uint32_t dlo = ((w[8] >> (s4 + 3)) & 0x00010001u) | (((w[9] >> (s4 + 3)) & 0x00010001u) << 8);
        const uint32_t dhi = ((w[10] >> (s4 + 3)) & 0x00010001u) | (((w[11] >> (s4 + 3)) & 0x00010001u) << 8);
        ca[r] = 7u * msum[r] + 2u * (msum[r] & (dlo * 0xFFu));
        ca[2 + r] = 7u * msum[2 + r] + 2u * (msum[2 + r] & (dhi * 0xFFu));
    }
    int chi[4] = {0, 0, 0, 0}, clo[4] = {0, 0, 0, 0};
    {
        const uint32_t h0 = *reinterpret_cast<const uint32_t*>(ccol + 4 * t), h1 = *reinterpret_cast<const uint32_t*>(ccol + 16 + 4 * t);
        const uint32_t l0 = *reinterpret_cast<const uint32_t*>(ccol + 32 + 4 * t), l1 = *reinterpret_cast<const uint32_t*>(ccol + 48 + 4 * t);
        mma_u8s8_k32(chi, ca[0], ca[1], ca[2], ca[3], h0, h1);
        mma_u8s8_k32(clo, ca[0], ca[1], ca[2], ca[3], l0, l1);
    }
    // the fp16 super-scale: the top nibbles of the four scale words
    float d[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t* w = r ? wb : wa;
        const uint32_t bits = ((w[12] >> 12) & 0x000Fu) | ((w[12] >> 24) & 0x00F0u) | ((w[13] >> 4) & 0x0F00u) | ((w[13] >> 16) & 0xF000u);
        d[r] = __half2float(__ushort_as_half((unsigned short) bits));
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) tot[i] = fmaf((float) (8 * acc[i] + 16 * chi[i] + clo[i]), d[i >> 1], tot[i]);
}

// a byte of shared memory at any alignment, two bytes, four bytes (blocks of 210 bytes are only 2-byte aligned)
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) { return *reinterpret_cast<const uint16_t*>(p); }
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }

// four 6-bit codes (one a byte) -> four s8 values code - 32: the low five bits stay, bits 5-7 become the sign
__device__ __forceinline__ uint32_t q6_to_s8(uint32_t v) { return (v & 0x1F1F1F1Fu) + ((~v & 0x20202020u) * 7u); }

// Q6_K: one 256-weight block of rows g and g + 8 (raw 210-byte blocks in shared memory, 2-byte aligned); bcol: this lane's
// column at the block's first byte plus 4 t.  tot[i] += sum over the 16 scale groups of (int dot) * d * sc.
__device__ __forceinline__ void q6k_block(const uint8_t* ra, const uint8_t* rb, const uint8_t* bcol, int t, float (&tot)[4]) {
    const float da = __half2float(__ushort_as_half((unsigned short) ld_u16(ra + 208))), db = __half2float(__ushort_as_half((unsigned short) ld_u16(rb + 208)));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int lo = 64 * h + 16 * j + 4 * t;
            const uint32_t qa1 = ld_u32_a2(ra + lo), qa2 = ld_u32_a2(ra + lo + 32), qah = ld_u32_a2(ra + 128 + 32 * h + 16 * j + 4 * t);
            const uint32_t qb1 = ld_u32_a2(rb + lo), qb2 = ld_u32_a2(rb + lo + 32), qbh = ld_u32_a2(rb + 128 + 32 * h + 16 * j + 4 * t);
#pragma unroll
            for (int sub = 0; sub < 4; ++sub) {
                const uint32_t la = ((((sub & 1) ? qa2 : qa1) >> (sub >= 2 ? 4 : 0)) & 0x0F0F0F0Fu) | (((qah >> (2 * sub)) & 0x03030303u) << 4);
                const uint32_t lb = ((((sub & 1) ? qb2 : qb1) >> (sub >= 2 ? 4 : 0)) & 0x0F0F0F0Fu) | (((qbh >> (2 * sub)) & 0x03030303u) << 4);
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bcol + 128 * h + 32 * sub + 16 * j);
                int c[4];
                mma_s8_k16(c, q6_to_s8(la), q6_to_s8(lb), b0);
                const int is = 8 * h + 2 * sub + j;
                const float sa = da * (float) (int) (int8_t) ra[192 + is], sb = db * (float) (int) (int8_t) rb[192 + is];
                tot[0] = fmaf((float) c[0], sa, tot[0]);
                tot[1] = fmaf((float) c[1], sa, tot[1]);
                tot[2] = fmaf((float) c[2], sb, tot[2]);
                tot[3] = fmaf((float) c[3], sb, tot[3]);
            }
        }
    }
}

// ---------------------------------------------------------------- the product kernel
// MODE GU: rows = 8 gate rows r0.. with the up rows r0..; columns = the entries' x images; writes h (fp32).
// MODE DOWN: rows = 16 down rows; columns = the entries' h images; writes out rows through ent_dst.
template <int TYPE, int MODE>
__global__ void __launch_bounds__(QT<TYPE>::kWarps * 32, 1)
kq_mma_kernel(ExpertArgs a, const int8_t* __restrict__ img, const int8_t* __restrict__ corr, const float* __restrict__ inv,
              const int2* __restrict__ items, int* __restrict__ n_items, int tiles_per_warp, int n_row_blocks) {
    using Q = QT<TYPE>;
    constexpr int kWarps = Q::kWarps, kThreads = kWarps * 32, kStages = Q::kStages;
    constexpr int kChunkBytes = kChunkBlocks * Q::kBlock;      // bytes of one row in a stage
    constexpr int kStageBytes = kRowsQ * kChunkBytes;
    constexpr int kPiecesRow = kChunkBytes / Q::kPiece, kPieces = kRowsQ * kPiecesRow;
    constexpr int kCopies = (kPieces + 31) / 32;
    extern __shared__ __align__(128) uint8_t smem[];
    const int64_t K = MODE == QMODE_GU ? a.L.n_embd : a.L.n_ff;
    const int nblk = (int) (K >> 8);
    const int cstride = (int) K + Q::kPad;                                   // bytes between activation columns
    const int xstride = nblk * 64 + 16;                                        // ... and between their correction columns
    uint8_t* xs = smem;                                                        // [8][cstride]
    uint8_t* cs = xs + (size_t) kColsQ * cstride;                              // [8][xstride] (IQ1_M)
    uint2* tab = reinterpret_cast<uint2*>(cs + (Q::kCorr ? (size_t) kColsQ * xstride : 0));   // [4096] (IQ1_M)
    uint8_t* wbase = reinterpret_cast<uint8_t*>(tab) + (Q::kCorr ? 32768 : 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t* wring = wbase + (size_t) warp * kStages * kStageBytes;
    const uint32_t wring_s = (uint32_t) __cvta_generic_to_shared(wring);
    const uint32_t xs_s = (uint32_t) __cvta_generic_to_shared(xs), cs_s = (uint32_t) __cvta_generic_to_shared(cs);
    __shared__ int s_ir[kEntQ];
    __shared__ int s_work;

    if (Q::kCorr) {
        // the codebook as 8 bytes per point, coordinate i's code c = g + 1 in byte i: the two words are the two MMA operand
        // registers of an 8-weight group.  Indexed by the block's 12-bit (qh nibble, qs byte) pair, whose top bit (the group's
        // delta sign) does not change the point: 4096 entries, each point twice.
        for (int i = threadIdx.x; i < 4096; i += kThreads) {
            const uint32_t p = a.grid[i & 2047];
            uint32_t lo = 0u, hi = 0u;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                lo |= ((p >> (2 * c)) & 3u) << (8 * c);
                hi |= ((p >> (2 * c + 8)) & 3u) << (8 * c);
            }
            tab[i] = make_uint2(lo, hi);
        }
    }
    pdl_wait();
    pdl_launch_dependents();

    const int64_t n_rows = MODE == QMODE_GU ? a.L.n_ff : a.L.n_embd;
    constexpr int kTileRows = MODE == QMODE_GU ? 8 : 16;
    constexpr int tile_stride = kWarps * kTileRows;
    const int n_chunks = nblk / kChunkBlocks;
    const size_t row_bytes = MODE == QMODE_GU ? (size_t) a.L.gu_row : (size_t) a.L.d_row;

    // this lane's copy duty inside a stage: pieces lane, lane + 32, ...; piece p -> row p / kPiecesRow
    const int n_work = n_items[0] * n_row_blocks;
    for (;;) {
        __syncthreads();   // the previous unit is done with xs, cs, s_ir and s_work
        if (threadIdx.x == 0) s_work = atomicAdd(&n_items[1], 1);
        __syncthreads();
        const int work = s_work;
        if (work >= n_work) break;
        const int item = work / n_row_blocks, rb = work - item * n_row_blocks;
        const int64_t r0 = (int64_t) rb * tiles_per_warp * tile_stride + warp * kTileRows;
        int live_tiles = 0;
        while (live_tiles < tiles_per_warp && r0 + (int64_t) live_tiles * tile_stride < n_rows) ++live_tiles;
        const int n_units = live_tiles * n_chunks;
        const int2 it = items[item];
        const int grp = it.x, eb = it.y;
        const uint8_t* blob = reinterpret_cast<const uint8_t*>(a.grp_ptr[grp]);
        const int e1 = min(a.grp_start[grp + 1], (int) a.cap_entries);
        const int ntok = min(kEntQ, e1 - eb);
        const int ncol = 2 * ntok;
        if (threadIdx.x < ntok) s_ir[threadIdx.x] = (MODE == QMODE_GU && a.n_x_rows > 0) ? a.ent_tok[eb + threadIdx.x] : eb + (int) threadIdx.x;
        __syncthreads();
        // the pass's activation columns (and their correction bytes): column c = 2 entry + term.  Columns beyond ncol keep
        // whatever they held: an MMA column depends on its own B column only, and those results are never stored.
        {
            const int per_col = (int) (K >> 4);
            for (int i = threadIdx.x; i < ncol * per_col; i += kThreads) {
                const int c = i / per_col, q = i - c * per_col;
                cpa16(xs_s + (uint32_t) (c * cstride + q * 16), img + ((size_t) s_ir[c >> 1] * 2 + (c & 1)) * K + (size_t) q * 16);
            }
            if (Q::kCorr) {
                const int per_cc = nblk * 4;
                for (int i = threadIdx.x; i < ncol * per_cc; i += kThreads) {
                    const int c = i / per_cc, q = i - c * per_cc;
                    cpa16(cs_s + (uint32_t) (c * xstride + q * 16), corr + ((size_t) s_ir[c >> 1] * 2 + (c & 1)) * nblk * 64 + (size_t) q * 16);
                }
            }
            cpa_commit();
        }
        // the weight stream: (tile, chunk) stages of this warp's 16 rows
        const uint8_t* rowp[kCopies];
        uint32_t dsto[kCopies];
#pragma unroll
        for (int j = 0; j < kCopies; ++j) {
            const int p = lane + 32 * j;
            const int row = p < kPieces ? p / kPiecesRow : 0, off = p < kPieces ? (p - row * kPiecesRow) * Q::kPiece : 0;
            const uint8_t* rp;
            if (MODE == QMODE_GU)
                rp = row < 8 ? blob + (size_t) (r0 + row) * a.L.gu_row : blob + a.L.up_off + (size_t) (r0 + row - 8) * a.L.up_row;
            else
                rp = blob + a.L.down_off + (size_t) (r0 + row) * a.L.d_row;
            rowp[j] = rp + off;
            dsto[j] = (uint32_t) (row * kChunkBytes + off);
        }
        const size_t tile_bytes = (size_t) tile_stride * row_bytes;
        int iss_unit = 0, iss_chunk = 0;
        size_t iss_off = 0;
        auto issue = [&]() {
            if (iss_unit < n_units) {
                const uint32_t dst = wring_s + (uint32_t) (iss_unit % kStages) * kStageBytes;
#pragma unroll
                for (int j = 0; j < kCopies; ++j)
                    if (lane + 32 * j < kPieces) {
                        if (Q::kPiece == 16) cpa16(dst + dsto[j], rowp[j] + iss_off);
                        else cpa4(dst + dsto[j], rowp[j] + iss_off);
                    }
                ++iss_unit;
                if (++iss_chunk == n_chunks) {
                    iss_chunk = 0;
                    iss_off += tile_bytes - (size_t) (n_chunks - 1) * kChunkBytes;
                } else {
                    iss_off += kChunkBytes;
                }
            }
            cpa_commit();
        };
#pragma unroll
        for (int c = 0; c < kStages - 1; ++c) issue();
        cpa_wait<kStages - 1>();   // the activation group (the oldest) has landed
        __syncthreads();

        // epilogue constants of this thread's entry (columns 2 t, 2 t + 1)
        float f = 0.f;
        int64_t orow = 0;
        if (t < ntok) {
            f = inv[s_ir[t]] * (Q::kCorr ? 0.125f : 1.f);
            orow = MODE == QMODE_GU ? (int64_t) (eb + t) * a.L.n_ff : (int64_t) a.ent_dst[eb + t] * a.L.n_embd;
        }
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        const uint8_t* bcol = xs + (size_t) g * cstride + (Q::kCorr ? 8 * t : 4 * t);
        const uint8_t* ccol = cs + (size_t) g * xstride;
        int tile = 0, chunk = 0;
        for (int unit = 0; unit < n_units; ++unit) {
            issue();
            cpa_wait<kStages - 1>();
            __syncwarp();
            const uint8_t* st = wring + (size_t) (unit % kStages) * kStageBytes;
#pragma unroll
            for (int b = 0; b < kChunkBlocks; ++b) {
                const int blk = chunk * kChunkBlocks + b;
                const uint8_t* ra = st + g * kChunkBytes + b * Q::kBlock;
                const uint8_t* rbp = st + (g + 8) * kChunkBytes + b * Q::kBlock;
                if constexpr (Q::kCorr) iq1m_block(ra, rbp, tab, bcol + 256 * blk, ccol + 64 * blk, t, tot);
                else q6k_block(ra, rbp, bcol + 256 * blk, t, tot);
            }
            __syncwarp();   // every lane is done with this stage before a later issue overwrites it
            if (++chunk != n_chunks) continue;
            const int64_t rt = r0 + (int64_t) tile * tile_stride;
            chunk = 0;
            ++tile;
            const float v0 = (tot[0] + tot[1] * kTerm2) * f, v1 = (tot[2] + tot[3] * kTerm2) * f;
            tot[0] = tot[1] = tot[2] = tot[3] = 0.f;
            if (t < ntok) {
                if (MODE == QMODE_GU) {
                    a.h[orow + rt + g] = swiglu(v0, v1, a.L);
                } else {
                    store_out(a.out, a.out_kind, orow + rt + g, v0);
                    store_out(a.out, a.out_kind, orow + rt + g + 8, v1);
                }
            }
        }
        cpa_wait<0>();
    }
    cpa_wait<0>();
}

size_t al256q(size_t v) { return (v + 255) & ~(size_t) 255; }

template <int TYPE>
size_t kq_smem(int64_t K) {
    using Q = QT<TYPE>;
    return (size_t) kColsQ * (K + Q::kPad) + (Q::kCorr ? (size_t) kColsQ * ((K >> 8) * 64 + 16) + 32768 : 0) +
           (size_t) Q::kWarps * Q::kStages * kRowsQ * kChunkBlocks * Q::kBlock + 128;
}

template <int TYPE, int MODE>
int32_t kq_launch(const ExpertArgs& a, const int8_t* img, const int8_t* corr, const float* inv, const int2* items, int* n_items, cudaStream_t st) {
    using Q = QT<TYPE>;
    const int64_t K = MODE == QMODE_GU ? a.L.n_embd : a.L.n_ff;
    const size_t smem = kq_smem<TYPE>(K);
    static std::atomic<bool> configured[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(kq_mma_kernel<TYPE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    const int64_t rows = MODE == QMODE_GU ? a.L.n_ff : a.L.n_embd;
    const int64_t row_bytes = K / 256 * Q::kBlock;
    const int64_t tile_bytes = (int64_t) Q::kWarps * kRowsQ * row_bytes;                 // one row tile of every warp
    const int64_t tile_rows = (MODE == QMODE_GU ? 8 : 16) * Q::kWarps;
    const int64_t n_tiles = (rows + tile_rows - 1) / tile_rows;
    int64_t tpw0 = (384 * 1024 + tile_bytes - 1) / tile_bytes;                           // a unit streams ~400 KB
    tpw0 = tpw0 < 1 ? 1 : tpw0 > 8 ? 8 : tpw0;
    const int64_t n_blocks = (n_tiles + tpw0 - 1) / tpw0;
    const int tpw = (int) ((n_tiles + n_blocks - 1) / n_blocks);
    const int n_row_blocks = (int) ((n_tiles + tpw - 1) / tpw);
    launch_k(kq_mma_kernel<TYPE, MODE>, dim3((unsigned) sm_count()), dim3(Q::kWarps * 32), smem, st, a, img, corr, inv, items, n_items, tpw, n_row_blocks);
    return launch_status();
}

bool kq_type(int t) { return t == kTypeIQ1M || t == kTypeQ6K; }

// the layout's K dimension works for the stream: whole 512-column chunks, 16-byte aligned rows where the copies are 16 bytes
bool kq_dim_ok(int type, int64_t K, int64_t rows) {
    if (K % 512 || rows % 8) return false;
    const int64_t rb = K / 256 * (type == kTypeIQ1M ? 56 : 210);
    return rb % (type == kTypeIQ1M ? 16 : 4) == 0;
}

}  // namespace

// scratch beyond the SwiGLU buffer: x images, h images (2 int8 terms each), their correction bytes, inverse scales, pass list
size_t experts_kq_scratch_bytes(int64_t cap, int64_t H, int64_t I) {
    return al256q((size_t) cap * 2 * H) + al256q((size_t) cap * 2 * I) + al256q((size_t) cap * 2 * (H / 256) * 64) + al256q((size_t) cap * 2 * (I / 256 + 1) * 64) +
           2 * al256q((size_t) cap * 4) + al256q((size_t) (cap + 1) * 8 + 16);
}

int32_t experts_grouped_kq(const ExpertArgs& a, cudaStream_t st) {
    const bsx_expert_layout& L = a.L;
    if (!kq_type(L.gu_type) || L.up_type != L.gu_type || !kq_type(L.d_type)) return BSX_E_TYPE;
    if (!kq_dim_ok(L.gu_type, L.n_embd, L.n_ff) || !kq_dim_ok(L.d_type, L.n_ff, L.n_embd) || L.n_embd % 16) return BSX_E_TYPE;
    if ((L.gu_type == kTypeIQ1M ? kq_smem<kTypeIQ1M>(L.n_embd) : kq_smem<kTypeQ6K>(L.n_embd)) > 225 * 1024) return BSX_E_TYPE;
    if ((L.d_type == kTypeIQ1M ? kq_smem<kTypeIQ1M>(L.n_ff) : kq_smem<kTypeQ6K>(L.n_ff)) > 225 * 1024) return BSX_E_TYPE;
    const int64_t cap = a.cap_entries, H = L.n_embd, I = L.n_ff;
    uint8_t* p = reinterpret_cast<uint8_t*>(a.h) + al256q((size_t) cap * I * 4);
    int8_t* ximg = reinterpret_cast<int8_t*>(p);
    p += al256q((size_t) cap * 2 * H);
    int8_t* himg = reinterpret_cast<int8_t*>(p);
    p += al256q((size_t) cap * 2 * I);
    int8_t* xcorr = reinterpret_cast<int8_t*>(p);
    p += al256q((size_t) cap * 2 * (H / 256) * 64);
    int8_t* hcorr = reinterpret_cast<int8_t*>(p);
    p += al256q((size_t) cap * 2 * (I / 256 + 1) * 64);
    float* xinv = reinterpret_cast<float*>(p);
    p += al256q((size_t) cap * 4);
    float* hinv = reinterpret_cast<float*>(p);
    p += al256q((size_t) cap * 4);
    int* n_items = reinterpret_cast<int*>(p);
    int2* items = reinterpret_cast<int2*>(n_items + 4);
    const int phase = experts_phase(a.L);
    const int64_t x_rows = a.n_x_rows > 0 ? a.n_x_rows : cap;
    const unsigned nbx = (unsigned) ((x_rows + 7) / 8 + 1), nbh = (unsigned) ((cap + 7) / 8 + 1);
    int32_t rc = BSX_OK;
    if (phase != 2) {
        if (L.gu_type == kTypeIQ1M) {
            launch_k(kq_image_kernel<false, true>, dim3(nbx), dim3(256), 0, st, a, ximg, xcorr, xinv, items, n_items);
            rc = kq_launch<kTypeIQ1M, QMODE_GU>(a, ximg, xcorr, xinv, items, n_items, st);
        } else {
            launch_k(kq_image_kernel<false, false>, dim3(nbx), dim3(256), 0, st, a, ximg, xcorr, xinv, items, n_items);
            rc = kq_launch<kTypeQ6K, QMODE_GU>(a, ximg, xcorr, xinv, items, n_items, st);
        }
    }
    if (rc != BSX_OK || phase == 1) return rc;
    if (L.d_type == kTypeIQ1M) {
        launch_k(kq_image_kernel<true, true>, dim3(nbh), dim3(256), 0, st, a, himg, hcorr, hinv, items, n_items);
        return kq_launch<kTypeIQ1M, QMODE_DOWN>(a, himg, hcorr, hinv, items, n_items, st);
    }
    launch_k(kq_image_kernel<true, false>, dim3(nbh), dim3(256), 0, st, a, himg, hcorr, hinv, items, n_items);
    return kq_launch<kTypeQ6K, QMODE_DOWN>(a, himg, hcorr, hinv, items, n_items, st);
}

}  // namespace bsx
