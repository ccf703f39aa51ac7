// experts_mma.cu - decode-sized grouped experts for NVFP4 blobs: a bandwidth-bound weight stream through shared memory with
// the dot products on the tensor cores.
//
// Shape of the work (HBM-bound): every touched expert's gate, up and down rows are read exactly once per pass of up to 8
// activation columns.  Each warp owns 16 weight rows (8 gate rows paired with the 8 matching up rows, or 16 down rows) and
// streams them in 256-column chunks (144 bytes a row) through its own 4-stage cp.async ring, so no block-wide barrier sits
// in the stream and ~110 KB a SM is in flight.  A row's E2M1 codes go to fp16 pairs with cvt.rn.f16x2.e2m1x2 (one ALU-pipe
// instruction per byte, the scarce resource here: the ALU pipe issues at half rate), are multiplied by the block's UE4M3
// scale as fp16 (the product has at most 5 significant bits: exact; the scale comes from a 256-entry shared-memory table)
// and feed mma.sync.m16n8k16 with fp32 accumulation.  Each of a row group's four threads owns one 16-value sub-block, so it
// decodes one scale per row and block.  The activation columns (8 bf16 tokens, or 4 fp32 tokens split into hi + lo fp16
// terms, each row pre-scaled by a power of two so it fits fp16) are prepared once per call by a small kernel into
// B-fragment order and copied into shared memory by cp.async.  Gate and up rows of one neuron land in the same thread's
// accumulators, so SwiGLU is fused; a second small kernel turns the SwiGLU output into the down product's fp16 image.
//
// Semantics: Basalt's native_expert_grouped (include/basalt/kernels/iq_kernels.hpp:77-92; kernels src/kernels/cuda/iq_kernels.cu:
// 1605-1658 gate/up, :2512-2524 SwiGLU, :2140-2164 down), NVFP4 decoding per src/kernels/cpu/ggml/ggml_quants.c:1397-1422,
// tail scales per iq_kernels.cu:683-701 - but without the int8 rounding of x and h the reference applies.
#include <atomic>
#include <cuda_fp16.h>

#include "common.cuh"
#include "experts.cuh"
#include "formats.cuh"

namespace bsx {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 4;
constexpr int kRowBytes = 144;                 // 4 NVFP4 blocks = 256 columns of one row
constexpr int kRows = 16;                      // weight rows per warp
constexpr int kStageBytes = kRows * kRowBytes; // 2304
constexpr int kPieces = kStageBytes / 16;      // 144 16-byte pieces a stage
constexpr int kCols = 8;                       // MMA n: activation columns per pass

enum { MODE_GU = 0, MODE_DOWN = 1 };

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// four E2M1 pairs (one byte each) of a 32-bit word -> four fp16 pairs; low nibble in the low half
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "mov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
}

__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// UE4M3 scale byte -> fp16 pair {d, d} with d = scale / 2^8: (byte & 0x7F) << 7 puts E4M3's exponent and mantissa where
// fp16 keeps them (value 2^(e-15) (1 + m/8), subnormals included) while the scale itself is 2^(e-7) (1 + m/8) (ggml halves
// it only because its E2M1 table is doubled; the cvt above yields undoubled values), so the epilogue multiplies the sums
// by 2^8.  0x7F decodes to 0 and bit 7 is ignored (src/kernels/cpu/ggml/ggml_quants.c:1397-1406).
__device__ __forceinline__ uint32_t scale_pair_bits(uint32_t byte) {
    const uint32_t b = byte & 0x7Fu;
    const uint32_t v = b == 0x7Fu ? 0u : b << 7;
    return v | (v << 16);
}

// Where column c of an activation row sits in its fp16 image, which is laid out so that a thread's B fragments are two
// 16-byte pieces per 64 columns: piece (gran, h, t) holds, for sub-block t of granule gran, the values the thread with
// id-in-group t needs for MMA steps 2h and 2h + 1.  Step s takes code bytes 2s and 2s + 1 of the sub-block's 8 bytes; byte b
// holds values b (low nibble -> k slot 2t) and b + 8 (high nibble -> k slot 2t + 1), bytes 2s + 1 go to slots 2t + 8, 2t + 9.
__device__ __forceinline__ int image_index(int c) {
    const int gran = c >> 6, t = (c >> 4) & 3, jj = c & 15, b = jj & 7, half = jj >> 3;
    const int step = b >> 1, reg = b & 1;
    return (((gran * 2 + (step >> 1)) * 4 + t) << 3) + 4 * (step & 1) + 2 * reg + half;
}

__device__ __forceinline__ float load_x(const void* x, int kind, int64_t row, int64_t K, int c) {
    if (kind == BSX_X_F32) return static_cast<const float*>(x)[row * K + c];
    if (kind == BSX_X_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(x)[row * K + c]);
    const uint8_t* b = static_cast<const uint8_t*>(x) + (row * (K / 32) + (c >> 5)) * 36;
    return __half2float(*reinterpret_cast<const __half*>(b)) * (float) (int8_t) b[4 + (c & 31)];
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    return (uint32_t) __half_as_ushort(__float2half_rn(lo)) | ((uint32_t) __half_as_ushort(__float2half_rn(hi)) << 16);
}

// One warp per activation row: the row -> fp16 image(s) in fragment order plus the inverse of the power of two it was
// scaled by (so that its largest magnitude lands in [2^13, 2^14), inside fp16 whatever the row's range).  A lane takes one
// 16-value sub-block at a time, which is exactly two 16-byte pieces of the image (see image_index).
// FROM_H = false: rows of x (kind x_kind, width n_embd) - row i of x when the caller gave the number of x rows, else the
// row of entry i; true: row e of the SwiGLU output h (fp32, width n_ff).
// The last block lists the passes of the product that follows: a pass is up to 8 / TERMS consecutive entries of one group,
// items[i] = {group, first entry}, so that kernel's blocks take one pass each however the entries are spread.
template <bool FROM_H, int TERMS>
__global__ void __launch_bounds__(256)
prep_image_kernel(ExpertArgs a, __half* __restrict__ img, float* __restrict__ inv, int2* __restrict__ items, int* __restrict__ n_items) {
    const int ng = min(*a.n_groups, (int) a.cap_groups);
    const int total = min(a.grp_start[ng], (int) a.cap_entries);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.x == gridDim.x - 1) {
        constexpr int NTOK = kCols / TERMS;
        __shared__ int sh[8];
        __shared__ int s_base;
        if (threadIdx.x == 0) s_base = 0;
        __syncthreads();
        for (int g0 = 0; g0 < ng; g0 += 256) {
            const int g = g0 + threadIdx.x;
            const int s0 = g < ng ? a.grp_start[g] : 0;
            const int cnt = g < ng ? max(0, min(a.grp_start[g + 1], (int) a.cap_entries) - s0) : 0;
            const int np = (cnt + NTOK - 1) / NTOK;
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
            for (int p = 0; p < np; ++p) items[before + x - np + p] = make_int2(g, s0 + p * NTOK);
            __syncthreads();
            if (threadIdx.x == 255) s_base = before + x;
            __syncthreads();
        }
        if (threadIdx.x == 0) {
            n_items[0] = s_base;
            n_items[1] = 0;      // the work counter of the product kernel that follows
        }
        return;
    }
    const int i = blockIdx.x * 8 + warp;   // image row
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
    int ex = 0;
    float s = 1.f, iv = 1.f;
    if (amax > 0.f && amax <= 3.0e38f) {
        frexpf(amax, &ex);                          // amax = f 2^ex, f in [0.5, 1)
        ex = max(-100, min(100, 14 - ex));
        s = ldexpf(1.f, ex);
        iv = ldexpf(1.f, -ex);
    }
    if (lane == 0) inv[i] = iv;
    uint4* out = reinterpret_cast<uint4*>(img + (size_t) i * K * TERMS);
    for (int sb = lane; sb < n_sb; sb += 32) {
        float v[16];
        load16(src, kind, row, K, sb, v);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= s;
        // pieces (gran, 0, t) and (gran, 1, t): values {0,8,1,9,2,10,3,11} and {4,12,5,13,6,14,7,15}
        const int piece = ((sb >> 2) * 2) * 4 + (sb & 3);
        out[piece] = make_uint4(pack_half2(v[0], v[8]), pack_half2(v[1], v[9]), pack_half2(v[2], v[10]), pack_half2(v[3], v[11]));
        out[piece + 4] = make_uint4(pack_half2(v[4], v[12]), pack_half2(v[5], v[13]), pack_half2(v[6], v[14]), pack_half2(v[7], v[15]));
        if (TERMS == 2) {
            float r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = v[j] - __half2float(__float2half_rn(v[j]));
            uint4* lo = out + (K >> 3);
            lo[piece] = make_uint4(pack_half2(r[0], r[8]), pack_half2(r[1], r[9]), pack_half2(r[2], r[10]), pack_half2(r[3], r[11]));
            lo[piece + 4] = make_uint4(pack_half2(r[4], r[12]), pack_half2(r[5], r[13]), pack_half2(r[6], r[14]), pack_half2(r[7], r[15]));
        }
    }
}

// MODE_GU:  rows = 8 gate rows r0.. paired with up rows r0..; columns = the entries' x images; writes h (fp32).
// MODE_DOWN: rows = 16 down rows; columns = the entries' h images; writes out rows through ent_dst.
// TERMS = 1: 8 entries a pass; TERMS = 2: 4 entries a pass, each as hi + lo fp16 columns.
template <int MODE, int TERMS>
__global__ void __launch_bounds__(kThreads, 2)
nvfp4_mma_kernel(ExpertArgs a, const __half* __restrict__ img, const float* __restrict__ inv, const int2* __restrict__ items,
                 int* __restrict__ n_items, int tiles_per_warp, int n_row_blocks) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int64_t K = MODE == MODE_GU ? a.L.n_embd : a.L.n_ff;
    const int n_gran = (int) (K >> 6);                       // 64-column granules
    __half* xs = reinterpret_cast<__half*>(smem);            // [n_gran][2][8 cols][4][8]
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem + (size_t) K * kCols * 2);   // [256] scale pairs
    uint4* zero = reinterpret_cast<uint4*>(smem + (size_t) K * kCols * 2 + 1024);   // 64 zero bytes: the B fragments of unused columns
    uint8_t* wbase = smem + (size_t) K * kCols * 2 + 1152;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    uint8_t* wring = wbase + (size_t) warp * kStages * kStageBytes;
    const uint32_t wring_s = (uint32_t) __cvta_generic_to_shared(wring);
    const uint32_t xs_s = (uint32_t) __cvta_generic_to_shared(xs);
    constexpr int NTOK = kCols / TERMS;

    __shared__ int s_ir[kCols];                        // image row of each entry of the pass
    lut[threadIdx.x] = scale_pair_bits(threadIdx.x);   // 256 threads, 256 entries; the first barrier below publishes it
    if (threadIdx.x < 4) zero[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);

    const int64_t n_rows = MODE == MODE_GU ? a.L.n_ff : a.L.n_embd;      // neurons (pairs) or down rows
    // A work unit is (pass, row block): a row block covers tiles_per_warp row tiles per warp; tile j of warp w starts at row (or
    // neuron) r0 + j * tile_stride.  The blocks are persistent and draw work units from a counter in global memory (zeroed by
    // the image kernel that runs before this one), so no block idles while another still has several units queued.
    constexpr int kTileRows = MODE == MODE_GU ? 8 : 16;
    constexpr int tile_stride = kWarps * kTileRows;
    __shared__ int s_work;
    const int n_chunks = n_gran >> 2;
    const int pieces_per_col = (int) (K >> 3);               // 16-byte pieces of one image

    // this lane's copy duty inside a stage: pieces lane, lane + 32, ... (< 144); row = piece / 9
    int cp_row[5], cp_off[5];
    uint32_t cp_dst[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        const int p = lane + 32 * j;
        cp_row[j] = p / 9;
        cp_off[j] = (p % 9) * 16;
        cp_dst[j] = (uint32_t) (cp_row[j] * kRowBytes + cp_off[j]);
    }

    const int n_work = n_items[0] * n_row_blocks;
    for (;;) {
        __syncthreads();   // the previous unit is done with xs and s_work
        if (threadIdx.x == 0) s_work = atomicAdd(&n_items[1], 1);
        __syncthreads();
        const int work = s_work;
        if (work >= n_work) break;
        const int item = work / n_row_blocks, rb = work - item * n_row_blocks;
        const int64_t r0 = (int64_t) rb * tiles_per_warp * tile_stride + warp * kTileRows;
        int live_tiles = 0;
        while (live_tiles < tiles_per_warp && r0 + (int64_t) live_tiles * tile_stride < n_rows) ++live_tiles;
        const int n_units = live_tiles * n_chunks;               // (tile, chunk) stages this warp streams for this unit
        const int2 it = items[item];
        const int grp = it.x;
        const uint8_t* blob = reinterpret_cast<const uint8_t*>(a.grp_ptr[grp]);
        const float* tail = reinterpret_cast<const float*>(blob + a.L.bytes - 16);
        const int e1 = min(a.grp_start[grp + 1], (int) a.cap_entries);
        // global address of this lane's pieces at chunk 0
        const uint8_t* src[5];
#pragma unroll
        for (int j = 0; j < 5; ++j) {
            const int row = cp_row[j];
            const uint8_t* rp;
            if (MODE == MODE_GU)
                rp = row < 8 ? blob + (size_t) (r0 + row) * a.L.gu_row : blob + a.L.up_off + (size_t) (r0 + row - 8) * a.L.up_row;
            else
                rp = blob + a.L.down_off + (size_t) (r0 + row) * a.L.d_row;
            src[j] = rp + cp_off[j];
        }
        const size_t tile_bytes = (size_t) tile_stride * (MODE == MODE_GU ? a.L.gu_row : a.L.d_row);
        // the next (tile, chunk) unit to request and its global byte offset from the tile-0, chunk-0 addresses
        int iss_unit = 0, iss_chunk = 0;
        size_t iss_off = 0;
        auto issue = [&]() {
            if (iss_unit < n_units) {
                const uint32_t dst = wring_s + (uint32_t) (iss_unit & (kStages - 1)) * kStageBytes;
#pragma unroll
                for (int j = 0; j < 5; ++j)
                    if (lane + 32 * j < kPieces) cp_async16(dst + cp_dst[j], src[j] + iss_off);
                ++iss_unit;
                if (++iss_chunk == n_chunks) {
                    iss_chunk = 0;
                    iss_off += tile_bytes - (size_t) (n_chunks - 1) * kRowBytes;
                } else {
                    iss_off += kRowBytes;
                }
            }
            cp_async_commit();
        };
        {
            const int eb = it.y;
            const int ntok = min(NTOK, e1 - eb);
            const int ncol = ntok * TERMS;
            if (threadIdx.x < ntok)
                s_ir[threadIdx.x] = (MODE == MODE_GU && a.n_x_rows > 0) ? a.ent_tok[eb + threadIdx.x] : eb + (int) threadIdx.x;
            __syncthreads();
            // the activation columns: image piece q of column c goes to piece ((q >> 2) * 8 + c) * 4 + (q & 3) of xs
            for (int i = threadIdx.x; i < ncol * pieces_per_col; i += kThreads) {
                const int c = i / pieces_per_col, q = i - c * pieces_per_col;
                const int ir = s_ir[c / TERMS], term = c % TERMS;
                const __half* sp = img + ((size_t) ir * TERMS + term) * K + (size_t) q * 8;
                cp_async16(xs_s + (uint32_t) ((((q >> 2) * kCols + c) * 4 + (q & 3)) * 16), sp);
            }
            cp_async_commit();
            // the weight stream
            iss_unit = 0;
            iss_chunk = 0;
            iss_off = 0;
#pragma unroll
            for (int c = 0; c < kStages - 1; ++c) issue();
            cp_async_wait<kStages - 1>();   // the activation group (the oldest) has landed
            __syncthreads();

            // per-pass epilogue constants, fetched before the stream starts so that no tile's epilogue waits on global memory:
            // the columns' inverse row scales times the tail scale(s) and the 2^8 of the fp16 block scales, and the output rows
            float f0 = 0.f, f1 = 0.f;
            int64_t o0 = 0, o1 = 0;
            {
                const int j0 = TERMS == 1 ? 2 * t : t, j1 = 2 * t + 1;
                if (j0 < ntok) f0 = inv[s_ir[j0]] * 256.f;
                if (TERMS == 1 && j1 < ntok) f1 = inv[s_ir[j1]] * 256.f;
                if (MODE == MODE_GU) {
                    o0 = (int64_t) (eb + j0) * a.L.n_ff;
                    o1 = (int64_t) (eb + j1) * a.L.n_ff;
                } else {
                    if (j0 < ntok) o0 = (int64_t) a.ent_dst[eb + j0] * a.L.n_embd;
                    if (TERMS == 1 && j1 < ntok) o1 = (int64_t) a.ent_dst[eb + j1] * a.L.n_embd;
                }
            }
            const float sg = tail[0], su = tail[1], sd = tail[2];
            // two accumulator sets, so that consecutive MMAs do not wait on each other
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, acd[4] = {0.f, 0.f, 0.f, 0.f};
            // this lane's B fragments: its column's pieces, or (column unused in this pass) the zero area with stride 0
            const bool col_live = g < ncol;
            const uint4* bcol = col_live ? reinterpret_cast<const uint4*>(xs) + g * 4 + t : zero;
            const int bstep = col_live ? 2 * kCols * 4 : 0;      // uint4 per 64-column granule
            const int bhalf = col_live ? kCols * 4 : 0;          // the second half-granule
            int tile = 0, chunk = 0;
            for (int unit = 0; unit < n_units; ++unit) {
                issue();
                cp_async_wait<kStages - 1>();
                __syncwarp();
                const uint8_t* st = wring + (size_t) (unit & (kStages - 1)) * kStageBytes;
                const uint32_t* ra = reinterpret_cast<const uint32_t*>(st + g * kRowBytes);          // row g
                const uint32_t* rb = reinterpret_cast<const uint32_t*>(st + (g + 8) * kRowBytes);    // row g + 8
                const uint4* bp = bcol + (size_t) chunk * 4 * bstep;
#pragma unroll
                for (int blk = 0; blk < 4; ++blk) {
                    const uint4 b0 = bp[blk * bstep], b1 = bp[blk * bstep + bhalf];
                    const uint32_t sa = lut[reinterpret_cast<const uint8_t*>(ra)[36 * blk + t]];
                    const uint32_t sb = lut[reinterpret_cast<const uint8_t*>(rb)[36 * blk + t]];
                    uint32_t qa0[4], qa1[4], qb0[4], qb1[4];
                    cvt_e2m1x8(ra[9 * blk + 1 + 2 * t], qa0);
                    cvt_e2m1x8(ra[9 * blk + 2 + 2 * t], qa1);
                    cvt_e2m1x8(rb[9 * blk + 1 + 2 * t], qb0);
                    cvt_e2m1x8(rb[9 * blk + 2 + 2 * t], qb1);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        qa0[i] = hmul2_bits(qa0[i], sa);
                        qa1[i] = hmul2_bits(qa1[i], sa);
                        qb0[i] = hmul2_bits(qb0[i], sb);
                        qb1[i] = hmul2_bits(qb1[i], sb);
                    }
                    mma_f16(acc, qa0[0], qb0[0], qa0[1], qb0[1], b0.x, b0.y);
                    mma_f16(acd, qa0[2], qb0[2], qa0[3], qb0[3], b0.z, b0.w);
                    mma_f16(acc, qa1[0], qb1[0], qa1[1], qb1[1], b1.x, b1.y);
                    mma_f16(acd, qa1[2], qb1[2], qa1[3], qb1[3], b1.z, b1.w);
                }
                __syncwarp();   // every lane is done with this stage before a later issue overwrites it
                if (++chunk != n_chunks) continue;
                // the tile is complete: undo the row scale and the 2^-8 of the fp16 block scales, apply the tail scales
                const int64_t rt = r0 + (int64_t) tile * tile_stride;
                chunk = 0;
                ++tile;
                const float c0 = acc[0] + acd[0], c1 = acc[1] + acd[1], c2 = acc[2] + acd[2], c3 = acc[3] + acd[3];
                acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                acd[0] = acd[1] = acd[2] = acd[3] = 0.f;
                if (MODE == MODE_GU) {
                    if (TERMS == 1) {
                        if (2 * t < ntok) a.h[o0 + rt + g] = swiglu(c0 * f0 * sg, c2 * f0 * su, a.L);
                        if (2 * t + 1 < ntok) a.h[o1 + rt + g] = swiglu(c1 * f1 * sg, c3 * f1 * su, a.L);
                    } else if (t < ntok) {
                        a.h[o0 + rt + g] = swiglu((c0 + c1) * f0 * sg, (c2 + c3) * f0 * su, a.L);
                    }
                } else {
                    if (TERMS == 1) {
                        if (2 * t < ntok) {
                            store_out(a.out, a.out_kind, o0 + rt + g, c0 * f0 * sd);
                            store_out(a.out, a.out_kind, o0 + rt + g + 8, c2 * f0 * sd);
                        }
                        if (2 * t + 1 < ntok) {
                            store_out(a.out, a.out_kind, o1 + rt + g, c1 * f1 * sd);
                            store_out(a.out, a.out_kind, o1 + rt + g + 8, c3 * f1 * sd);
                        }
                    } else if (t < ntok) {
                        store_out(a.out, a.out_kind, o0 + rt + g, (c0 + c1) * f0 * sd);
                        store_out(a.out, a.out_kind, o0 + rt + g + 8, (c2 + c3) * f0 * sd);
                    }
                }
            }
            cp_async_wait<0>();
        }
    }
    cp_async_wait<0>();
}

size_t smem_bytes(int64_t K) { return (size_t) K * kCols * 2 + 1152 + (size_t) kWarps * kStages * kStageBytes; }
size_t align256(size_t v) { return (v + 255) & ~(size_t) 255; }

template <int MODE, int TERMS>
int32_t launch(const ExpertArgs& a, const __half* img, const float* inv, const int2* items, int* n_items, cudaStream_t st) {
    const int64_t K = MODE == MODE_GU ? a.L.n_embd : a.L.n_ff;
    const size_t smem = smem_bytes(K);
    static std::atomic<bool> configured[64];   // per device; threads of different devices call concurrently
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int32_t) cudaErrorInvalidDevice;
    if (!configured[dev].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(nvfp4_mma_kernel<MODE, TERMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int32_t) e;
        configured[dev].store(true, std::memory_order_release);
    }
    const int64_t rows = MODE == MODE_GU ? a.L.n_ff : a.L.n_embd;
    // a work unit streams ~150 KB of weights (enough to hide its start-up: activation copy, first loads); the row tiles of an
    // expert are dealt evenly over the units
    const int64_t tile_bytes = (int64_t) kWarps * 16 * (K / 64 * 36);
    const int64_t tile_rows = MODE == MODE_GU ? kWarps * 8 : kWarps * 16;
    const int64_t n_tiles = (rows + tile_rows - 1) / tile_rows;
    int64_t tpw0 = (150 * 1024 + tile_bytes - 1) / tile_bytes;
    tpw0 = tpw0 < 1 ? 1 : tpw0 > 8 ? 8 : tpw0;
    const int64_t n_blocks = (n_tiles + tpw0 - 1) / tpw0;
    const int tpw = (int) ((n_tiles + n_blocks - 1) / n_blocks);
    const int n_row_blocks = (int) ((n_tiles + tpw - 1) / tpw);
    nvfp4_mma_kernel<MODE, TERMS><<<(unsigned) (2 * sm_count()), kThreads, smem, st>>>(a, img, inv, items, n_items, tpw, n_row_blocks);
    return launch_status();
}

}  // namespace

// scratch beyond the SwiGLU buffer: the x images (up to two fp16 terms), the h images (two terms), the inverse row scales
size_t experts_mma_scratch_bytes(int64_t cap_entries, int64_t n_embd, int64_t n_ff) {
    // the pass list: at most one pass per entry, 8 bytes each, plus its count
    return align256((size_t) cap_entries * n_embd * 4) + align256((size_t) cap_entries * n_ff * 4) + 2 * align256((size_t) cap_entries * 4) +
           align256((size_t) (cap_entries + 1) * 8 + 16);
}

int32_t experts_grouped_mma(const ExpertArgs& a, cudaStream_t st) {
    const bsx_expert_layout& L = a.L;
    if (L.gu_type != kTypeNVFP4 || L.up_type != kTypeNVFP4 || L.d_type != kTypeNVFP4) return BSX_E_TYPE;
    // 16-byte row chunks: both K dimensions must be whole 256-column chunks; the activation image must fit shared memory
    if (L.n_embd % 256 || L.n_ff % 256 || L.n_ff % 8 || L.n_embd % 16) return BSX_E_TYPE;
    if (smem_bytes(L.n_embd) > 200 * 1024 || smem_bytes(L.n_ff) > 200 * 1024) return BSX_E_TYPE;
    // scratch: [h fp32][x images][h images][x inverse scales][h inverse scales]
    uint8_t* p = reinterpret_cast<uint8_t*>(a.h) + align256((size_t) a.cap_entries * L.n_ff * 4);
    __half* ximg = reinterpret_cast<__half*>(p);
    p += align256((size_t) a.cap_entries * L.n_embd * 4);
    __half* himg = reinterpret_cast<__half*>(p);
    p += align256((size_t) a.cap_entries * L.n_ff * 4);
    float* xinv = reinterpret_cast<float*>(p);
    float* hinv = xinv + align256((size_t) a.cap_entries * 4) / 4;
    int* n_items = reinterpret_cast<int*>(hinv + align256((size_t) a.cap_entries * 4) / 4);
    int2* items = reinterpret_cast<int2*>(n_items + 4);
    const int phase = experts_phase(a.L);
    // a warp per image row, 8 a block, plus the block that lists the passes
    const int64_t x_rows = a.n_x_rows > 0 ? a.n_x_rows : a.cap_entries;
    const unsigned nbx = (unsigned) ((x_rows + 7) / 8 + 1), nbh = (unsigned) ((a.cap_entries + 7) / 8 + 1);
    int32_t rc = BSX_OK;
    if (phase != 2) {
        if (a.x_kind == BSX_X_BF16) {
            prep_image_kernel<false, 1><<<nbx, 256, 0, st>>>(a, ximg, xinv, items, n_items);
            rc = launch<MODE_GU, 1>(a, ximg, xinv, items, n_items, st);
        } else {
            prep_image_kernel<false, 2><<<nbx, 256, 0, st>>>(a, ximg, xinv, items, n_items);
            rc = launch<MODE_GU, 2>(a, ximg, xinv, items, n_items, st);
        }
    }
    if (rc != BSX_OK || phase == 1) return rc;
    prep_image_kernel<true, 2><<<nbh, 256, 0, st>>>(a, himg, hinv, items, n_items);
    return launch<MODE_DOWN, 2>(a, himg, hinv, items, n_items, st);
}

}  // namespace bsx
