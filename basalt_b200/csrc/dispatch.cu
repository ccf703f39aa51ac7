// dispatch.cu - token-to-expert dispatch on sm_100a: expert histogram, prefix-sum offsets, stable permutation, tile list,
// and the decode-window plan.
//
// Replaces the Basalt engine's host counting sort (src/models/qwen4exp/prefill/routing.cpp:67-108, which costs a device-to-host
// copy, a stream synchronise and a host-to-device copy per layer), its GPU grouping (src/models/qwen4exp/prefill/moe_fused.cu:
// 99-168, whose atomicAdd cursors leave the row order inside an expert undefined) and the decode plan
// (src/models/inkling2/kernels/ops.cu:275-340).  Here the permutation is the host path's stable counting sort, computed on
// the device without position atomics: every warp owns a contiguous chunk of pairs, counts it, a scan turns the
// [expert][chunk] counts into chunk bases, and each warp places its pairs in order with __match_any_sync ranks.
#include <atomic>

#include "common.cuh"
#include "pdl.cuh"
#include "plan.cuh"

namespace bsx {
namespace {

constexpr int kChunk = 256;          // pairs per warp chunk
constexpr int kWarpsPerBlock = 8;
constexpr int kMaxExpert = 1024;

__host__ __device__ inline int64_t n_chunks_of(int64_t n) { return (n + kChunk - 1) / kChunk; }

// per-warp histogram of one chunk -> tbl[e * n_chunks + c]
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dispatch_count_kernel(const int32_t* __restrict__ ids, int64_t n, int E, int n_chunks, int32_t* __restrict__ tbl) {
    extern __shared__ int32_t hist[];   // [warps][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * kWarpsPerBlock + warp;
    int32_t* h = hist + (size_t) warp * E;
    for (int e = lane; e < E; e += 32) h[e] = 0;
    __syncwarp();
    if (c < n_chunks) {
        const int64_t i0 = (int64_t) c * kChunk;
        for (int j = 0; j < kChunk; j += 32) {
            const int64_t i = i0 + j + lane;
            const int e = i < n ? ids[i] : -1;
            const bool ok = (unsigned) e < (unsigned) E;
            const unsigned peers = __match_any_sync(kFull, ok ? e : -1 - lane);
            if (ok && (__ffs(peers) - 1) == lane) h[e] += __popc(peers);
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32) tbl[(size_t) e * n_chunks + c] = h[e];
    }
}

// Prompt-sized dispatches (hundreds of chunks): step (1) of dispatch_scan_kernel as its own launch, one warp per expert over
// as many blocks as that takes; the totals go to cnt[].
__global__ void __launch_bounds__(256)
dispatch_rowscan_kernel(int E, int n_chunks, int32_t* __restrict__ tbl, int32_t* __restrict__ cnt) {
    const int lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (e >= E) return;
    int32_t* row = tbl + (size_t) e * n_chunks;
    int carry = 0;
    for (int c0 = 0; c0 < n_chunks; c0 += 32) {
        const int c = c0 + lane;
        const int v = c < n_chunks ? row[c] : 0;
        int x = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(kFull, x, o);
            if (lane >= o) x += y;
        }
        if (c < n_chunks) row[c] = carry + x - v;
        carry += __shfl_sync(kFull, x, 31);
    }
    if (lane == 0) cnt[e] = carry;
}

// one block of 1024 threads: (1) a warp per expert scans its chunk counts into exclusive chunk bases and the expert's
// total (skipped when dispatch_rowscan_kernel has done it: rows_done); (2) a block scan over the experts gives off[], and
// the tile list.
__global__ void __launch_bounds__(1024)
dispatch_scan_kernel(int E, int n_chunks, int32_t* __restrict__ tbl, int32_t* __restrict__ cnt, int32_t* __restrict__ off,
                     int tile_rows, int32_t* __restrict__ tiles, int32_t* __restrict__ n_tiles, int rows_done) {
    __shared__ int s_cnt[kMaxExpert];
    __shared__ int sh[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (rows_done) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = cnt[e];
    }
    for (int e = warp; e < E && !rows_done; e += nw) {
        int32_t* row = tbl + (size_t) e * n_chunks;
        int carry = 0;
        for (int c0 = 0; c0 < n_chunks; c0 += 32) {
            const int c = c0 + lane;
            const int v = c < n_chunks ? row[c] : 0;
            int x = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int y = __shfl_up_sync(kFull, x, o);
                if (lane >= o) x += y;
            }
            if (c < n_chunks) row[c] = carry + x - v;
            carry += __shfl_sync(kFull, x, 31);
        }
        if (lane == 0) s_cnt[e] = carry;
    }
    __syncthreads();
    const int e = threadIdx.x;
    const int c = e < E ? s_cnt[e] : 0;
    const int nt = tile_rows > 0 ? (c + tile_rows - 1) / tile_rows : 0;
    int rows = 0, ntl = 0;
    const int o = block_excl_sum(c, &rows, sh);
    const int to = block_excl_sum(nt, &ntl, sh);
    if (e < E) {
        cnt[e] = c;
        off[e] = o;
        if (tiles)
            for (int i = 0; i < nt; ++i) {
                tiles[2 * (to + i)] = e;
                tiles[2 * (to + i) + 1] = o + i * tile_rows;
            }
    }
    if (e == 0) {
        off[E] = rows;
        if (n_tiles) *n_tiles = ntl;
    }
}

// each warp replays its chunk in order: a pair's row = off[e] + (pairs of e in earlier chunks) + (earlier pairs of e in
// this chunk), the last term from a per-warp running count plus the pair's rank among the lanes holding the same expert.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dispatch_place_kernel(const int32_t* __restrict__ ids, int64_t n, int k, int E, int n_chunks, const int32_t* __restrict__ tbl,
                      const int32_t* __restrict__ off, int32_t* __restrict__ slot, int32_t* __restrict__ src) {
    extern __shared__ int32_t run[];   // [warps][E]: absolute next row of expert e for this chunk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = blockIdx.x * kWarpsPerBlock + warp;
    if (c >= n_chunks) return;
    int32_t* r = run + (size_t) warp * E;
    for (int e = lane; e < E; e += 32) r[e] = off[e] + tbl[(size_t) e * n_chunks + c];
    __syncwarp();
    const int64_t i0 = (int64_t) c * kChunk;
    const unsigned lt = (1u << lane) - 1u;
    for (int j = 0; j < kChunk; j += 32) {
        const int64_t i = i0 + j + lane;
        const int e = i < n ? ids[i] : -1;
        const bool ok = (unsigned) e < (unsigned) E;
        const unsigned peers = __match_any_sync(kFull, ok ? e : -1 - lane);
        int p = -1;
        if (ok) p = r[e] + __popc(peers & lt);
        __syncwarp();
        if (ok && (__ffs(peers) - 1) == lane) r[e] += __popc(peers);
        __syncwarp();
        if (i < n) {
            slot[i] = p;
            if (ok) src[p] = (int32_t) (i / k);
        }
    }
}

// ---------------------------------------------------------------------------------------------- decode-window plan
// One block of 1024 threads, everything in shared memory (plan.cuh).
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int32_t* __restrict__ ids, int n, int k, int E, const unsigned long long* __restrict__ blobs,
                unsigned long long shared_blob, int n_tok, unsigned long long* __restrict__ ptr, int32_t* __restrict__ start,
                int32_t* __restrict__ n_groups, int32_t* __restrict__ dst, int32_t* __restrict__ tok, PassRec* __restrict__ items,
                int* __restrict__ n_items) {
    extern __shared__ unsigned long long smb[];
    const PlanSmem ps = plan_smem(smb, E);
    plan_load_blobs(ps, blobs, E);       // constant addresses: before the wait for the kernel that wrote the ids
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) plan_note_pair(ps, i, ids[i], E);
    __syncthreads();
    plan_finish(ps, n, k, E, shared_blob, n_tok, ptr, start, n_groups, dst, tok, items, n_items);
}

// ---------------------------------------------------------------------------------------------- expert-parallel plan, one launch
// Every rank holds every token's routing (all-gathered); this block turns the pairs that name experts held HERE (a non-zero
// blob address) into groups and entries - ent_dst = the pair's index (its row in the rows buffer), ent_tok = its token's
// index among all gathered tokens - plus one group for the shared expert over this rank's own tokens.  Replaces a full
// dispatch of all pairs (three launches) and the group extraction after it.  ids may come in blocks of `blk` pairs, one per
// source rank, `blk_stride` values apart (the layout an all-gather of [ids | weights] buffers leaves); blk = 0: dense.
// replicated (optional, [E] bytes): experts every rank holds a copy of (hot experts); a pair naming one is computed by the
// rank that owns the pair's TOKEN (pairs own_lo .. own_lo + own_n - 1), so each pair still has exactly one rank.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t* __restrict__ ids, int n, int k, int blk, int blk_stride, int E, const unsigned long long* __restrict__ blobs,
               unsigned long long shared_blob, int tok_lo, int tok_n, unsigned long long* __restrict__ ptr, int32_t* __restrict__ start,
               int32_t* __restrict__ n_groups, int32_t* __restrict__ dst, int32_t* __restrict__ tok, const uint8_t* __restrict__ replicated,
               int own_lo, int own_n) {
    extern __shared__ unsigned long long smb[];
    const PlanSmem ps = plan_smem(smb, E);
    plan_load_blobs(ps, blobs, E);
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int at = blk > 0 ? (i / blk) * blk_stride + (i % blk) : i;
        int e = ids[at];
        if (replicated && (unsigned) e < (unsigned) E && replicated[e] && (i < own_lo || i >= own_lo + own_n)) e = -1;   // its token's owner runs it
        plan_note_pair(ps, i, e, E);
    }
    __syncthreads();
    plan_finish<false>(ps, n, k, E, shared_blob, tok_n, ptr, start, n_groups, dst, tok, nullptr, nullptr, tok_lo);
}

// Groups for the experts this device holds, from a dispatch: the experts with rows and a non-zero blob address become
// groups in ascending order; their dispatch rows, in order, become the entries (ent_dst = the dispatch row, so outputs land
// where the combine's slot[] points; ent_tok = the row's token).  Rows of experts held elsewhere get no entry.
// One block: a scan over the experts, then every thread places rows by binary search in the offsets.
__global__ void __launch_bounds__(1024)
plan_groups_kernel(const int32_t* __restrict__ cnt, const int32_t* __restrict__ off, const int32_t* __restrict__ src, int E,
                   const unsigned long long* __restrict__ blobs, unsigned long long shared_blob, int tok_lo, int tok_n,
                   unsigned long long* __restrict__ ptr, int32_t* __restrict__ start,
                   int32_t* __restrict__ n_groups, int32_t* __restrict__ ent_dst, int32_t* __restrict__ ent_tok) {
    __shared__ int sh[32];
    __shared__ int s_off[kMaxExpert + 1];
    __shared__ int s_first[kMaxExpert];     // first compact entry of expert e, or -1 when it has no group here
    const int e = threadIdx.x;
    const int c = e < E ? cnt[e] : 0;
    const bool used = c > 0 && blobs[e] != 0ull;
    int groups = 0, entries = 0;
    const int g = block_excl_sum(used ? 1 : 0, &groups, sh);
    const int first = block_excl_sum(used ? c : 0, &entries, sh);
    if (e < E) {
        s_off[e] = off[e];
        s_first[e] = used ? first : -1;
    }
    if (used) {
        ptr[g] = blobs[e];
        start[g] = first;
    }
    // a shared expert: one more group, tokens tok_lo .. tok_lo + tok_n - 1, its rows after the dispatch's own
    const int extra = shared_blob != 0ull ? tok_n : 0;
    if (e == 0) {
        s_off[E] = off[E];
        start[groups] = entries;
        if (extra > 0) {
            ptr[groups] = shared_blob;
            start[groups + 1] = entries + extra;
            start[groups + 2] = entries + extra;
            *n_groups = groups + 1;
        } else {
            start[groups + 1] = entries;
            *n_groups = groups;
        }
    }
    __syncthreads();
    const int n_rows = s_off[E];
    for (int t = threadIdx.x; t < extra; t += blockDim.x) {
        ent_dst[entries + t] = n_rows + t;
        ent_tok[entries + t] = tok_lo + t;
    }
    for (int r = threadIdx.x; r < n_rows; r += blockDim.x) {
        int lo = 0, hi = E;                 // the expert with off[x] <= r < off[x + 1]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s_off[mid] <= r) lo = mid; else hi = mid;
        }
        const int f = s_first[lo];
        if (f >= 0) {
            const int i = f + (r - s_off[lo]);
            ent_dst[i] = r;
            ent_tok[i] = src[r];
        }
    }
}

// Scratch of bsx_dispatch_static: the [expert][chunk] count table for up to kStaticMaxPairs pairs over up to kMaxExpert
// experts (1 MiB), resident on every device that loads this library.  Host code may only take its address
// (cudaGetSymbolAddress); the name itself is not a device pointer on the host side.
constexpr int64_t kStaticMaxPairs = 65536;
static __device__ __align__(256) int32_t g_static_dispatch_tbl[kMaxExpert * (kStaticMaxPairs / kChunk)];

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" size_t bsx_dispatch_scratch_bytes(int64_t n_pairs, int32_t E) {
    if (n_pairs < 0 || E < 1) return 0;
    const int64_t nc = n_chunks_of(n_pairs > 0 ? n_pairs : 1);
    return (size_t) E * (size_t) nc * sizeof(int32_t) + 256;
}

// Device address of the static table on the current device; looked up once per device, with that device current.
static int32_t* static_dispatch_table(int32_t* status) {
    static std::atomic<int32_t*> cached[64];   // per device; two host threads racing on a first call store the same address
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *status = (int32_t) e; return nullptr; }
    if (dev < 0 || dev >= 64) { *status = (int32_t) cudaErrorInvalidDevice; return nullptr; }
    int32_t* tbl = cached[dev].load(std::memory_order_acquire);
    if (!tbl) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_dispatch_tbl);
        if (e != cudaSuccess) { *status = (int32_t) e; return nullptr; }
        tbl = static_cast<int32_t*>(p);
        cached[dev].store(tbl, std::memory_order_release);
    }
    *status = BSX_OK;
    return tbl;
}

extern "C" int32_t bsx_dispatch_static(const int32_t* ids, int64_t n_pairs, int32_t k, int32_t E, int32_t* cnt, int32_t* off,
                                       int32_t* slot, int32_t* src, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (E < 1 || k < 1 || n_pairs < 0) return BSX_E_GEOMETRY;
    if (n_pairs > kStaticMaxPairs || E > kMaxExpert) return BSX_E_LIMIT;   // beyond the resident table: use bsx_dispatch with caller scratch
    int32_t status = BSX_OK;
    int32_t* tbl = static_dispatch_table(&status);
    if (!tbl) return status;
    return bsx_dispatch(ids, n_pairs, k, E, cnt, off, slot, src, 0, nullptr, nullptr, tbl, stream);
}

extern "C" int32_t bsx_dispatch(const int32_t* ids, int64_t n_pairs, int32_t k, int32_t E, int32_t* cnt, int32_t* off,
                                int32_t* slot, int32_t* src, int32_t tile_rows, int32_t* tiles, int32_t* n_tiles, void* scratch,
                                void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (E < 1 || E > kMaxExpert || k < 1 || n_pairs < 0 || n_pairs > (int64_t) 1 << 30 || tile_rows < 0) return BSX_E_GEOMETRY;
    if (!cnt || !off || !scratch || (n_pairs > 0 && (!ids || !slot || !src))) return BSX_E_POINTER;
    if (tile_rows > 0 && (!tiles || !n_tiles)) return BSX_E_POINTER;
    const cudaStream_t st = (cudaStream_t) stream;
    const int nc = (int) n_chunks_of(n_pairs > 0 ? n_pairs : 1);
    int32_t* tbl = (int32_t*) scratch;
    const unsigned blocks = (unsigned) ((nc + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const size_t smem = (size_t) kWarpsPerBlock * E * sizeof(int32_t);
    dispatch_count_kernel<<<blocks, kWarpsPerBlock * 32, smem, st>>>(ids, n_pairs, E, nc, tbl);
    const int split = nc > 64 ? 1 : 0;     // many chunks: the per-expert scans get their own, wider launch
    if (split) dispatch_rowscan_kernel<<<(unsigned) ((E + 7) / 8), 256, 0, st>>>(E, nc, tbl, cnt);
    dispatch_scan_kernel<<<1, 1024, 0, st>>>(E, nc, tbl, cnt, off, tile_rows, tile_rows > 0 ? tiles : nullptr,
                                              tile_rows > 0 ? n_tiles : nullptr, split);
    if (n_pairs > 0)
        dispatch_place_kernel<<<blocks, kWarpsPerBlock * 32, smem, st>>>(ids, n_pairs, k, E, nc, tbl, off, slot, src);
    return launch_status();
}

static int32_t plan_launch(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table,
                           unsigned long long shared_blob, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst,
                           int32_t* tok, void* stream, PassRec* items = nullptr, int* n_items = nullptr) {
    if (!stream) return BSX_E_STREAM;
    const int64_t n = (int64_t) T * k;
    if (n <= 0) return BSX_OK;   // the reference returns without touching its outputs (ops.cu:491)
    if (n > BSX_PLAN_MAX_PAIRS) return BSX_E_LIMIT;
    if (E < 1 || E > BSX_PLAN_MAX_EXPERTS) return BSX_E_GEOMETRY;   // E * 16 + n * 4 bytes of shared memory must stay below 48 KB
    if (!ids || !blob_table || !ptr || !start || !n_groups || !dst || !tok) return BSX_E_POINTER;
    const size_t smem = (size_t) E * (sizeof(unsigned long long) + 2 * sizeof(int32_t)) + (size_t) n * sizeof(int32_t);
    launch_k(moe_plan_kernel, dim3(1), dim3(1024), smem, (cudaStream_t) stream, ids, (int) n, k, E, blob_table, shared_blob, (int) T, ptr, start, n_groups, dst, tok, items, n_items);
    return launch_status();
}

namespace bsx {
// the decode-window plan that also writes the packed expert kernels' pass list (plan.cuh)
int32_t moe_plan_with_passes(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table, unsigned long long shared_blob,
                             unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok, PassRec* items, int* n_items,
                             cudaStream_t st) {
    return plan_launch(ids, T, k, E, blob_table, shared_blob, ptr, start, n_groups, dst, tok, (void*) st, items, n_items);
}
}  // namespace bsx

// the tile list of a dispatch from its row bounds alone: one block, a scan over the experts' tile counts
__global__ void __launch_bounds__(1024)
tiles_from_bounds_kernel(const int32_t* __restrict__ off, int E, int tile_rows, int32_t* __restrict__ tiles, int32_t* __restrict__ n_tiles) {
    __shared__ int sh[32];
    const int e = threadIdx.x;
    const int o = e < E ? off[e] : 0;
    const int c = e < E ? off[e + 1] - o : 0;
    const int nt = c > 0 ? (c + tile_rows - 1) / tile_rows : 0;
    int total = 0;
    const int to = block_excl_sum(nt, &total, sh);
    for (int i = 0; i < nt; ++i) {
        tiles[2 * (to + i)] = e;
        tiles[2 * (to + i) + 1] = o + i * tile_rows;
    }
    if (e == 0) *n_tiles = total;
}

extern "C" int32_t bsx_tiles_from_bounds(const int32_t* off, int32_t E, int32_t tile_rows, int32_t* tiles, int32_t* n_tiles, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (E < 1 || E > kMaxExpert || tile_rows < 1) return BSX_E_GEOMETRY;
    if (!off || !tiles || !n_tiles) return BSX_E_POINTER;
    tiles_from_bounds_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(off, E, tile_rows, tiles, n_tiles);
    return launch_status();
}

extern "C" int32_t bsx_ep_plan(const int32_t* ids, int64_t n_pairs, int32_t k, int32_t pairs_per_block, int32_t block_stride, int32_t E,
                               const unsigned long long* blob_table, unsigned long long shared_blob, int32_t tok_lo, int32_t tok_n,
                               const uint8_t* replicated, unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* ent_dst,
                               int32_t* ent_tok, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (E < 1 || E > BSX_PLAN_MAX_EXPERTS || k < 1 || n_pairs < 0 || tok_lo < 0 || tok_n < 0 || pairs_per_block < 0) return BSX_E_GEOMETRY;
    const size_t smem = plan_smem_bytes(E, (int) n_pairs);
    if (n_pairs > BSX_EP_PLAN_MAX_PAIRS || smem > 48 * 1024) return BSX_E_LIMIT;
    if (!ids || !blob_table || !ptr || !start || !n_groups || !ent_dst || !ent_tok) return BSX_E_POINTER;
    launch_k(ep_plan_kernel, dim3(1), dim3(1024), smem, (cudaStream_t) stream, ids, (int) n_pairs, (int) k, (int) pairs_per_block, (int) block_stride, (int) E,
             blob_table, shared_blob, (int) tok_lo, (int) tok_n, ptr, start, n_groups, ent_dst, ent_tok, replicated, (int) (tok_lo * k), (int) (tok_n * k));
    return launch_status();
}

extern "C" int32_t bsx_plan_groups(const int32_t* cnt, const int32_t* off, const int32_t* src, int32_t E,
                                   const unsigned long long* blob_table, unsigned long long* ptr, int32_t* start, int32_t* n_groups,
                                   int32_t* ent_dst, int32_t* ent_tok, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (E < 1 || E > kMaxExpert) return BSX_E_GEOMETRY;
    if (!cnt || !off || !src || !blob_table || !ptr || !start || !n_groups || !ent_dst || !ent_tok) return BSX_E_POINTER;
    plan_groups_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(cnt, off, src, E, blob_table, 0ull, 0, 0, ptr, start, n_groups, ent_dst, ent_tok);
    return launch_status();
}

extern "C" int32_t bsx_plan_groups_shared(const int32_t* cnt, const int32_t* off, const int32_t* src, int32_t E, const unsigned long long* blob_table,
                                          unsigned long long shared_blob, int32_t tok_lo, int32_t tok_n, unsigned long long* ptr, int32_t* start,
                                          int32_t* n_groups, int32_t* ent_dst, int32_t* ent_tok, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (E < 1 || E > kMaxExpert || tok_lo < 0 || tok_n < 0) return BSX_E_GEOMETRY;
    if (!cnt || !off || !src || !blob_table || !ptr || !start || !n_groups || !ent_dst || !ent_tok) return BSX_E_POINTER;
    plan_groups_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(cnt, off, src, E, blob_table, shared_blob, tok_lo, tok_n, ptr, start, n_groups, ent_dst,
                                                              ent_tok);
    return launch_status();
}

extern "C" int32_t bsx_moe_plan(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table,
                                unsigned long long* ptr, int32_t* start, int32_t* n_groups, int32_t* dst, int32_t* tok,
                                void* stream) {
    return plan_launch(ids, T, k, E, blob_table, 0ull, ptr, start, n_groups, dst, tok, stream);
}

extern "C" int32_t bsx_moe_plan_shared(const int32_t* ids, int32_t T, int32_t k, int32_t E, const unsigned long long* blob_table,
                                       unsigned long long shared_blob, unsigned long long* ptr, int32_t* start, int32_t* n_groups,
                                       int32_t* dst, int32_t* tok, void* stream) {
    return plan_launch(ids, T, k, E, blob_table, shared_blob, ptr, start, n_groups, dst, tok, stream);
}
