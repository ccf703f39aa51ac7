// plan.cuh - the decode-window plan as block-wide device routines, shared by the plan kernel (dispatch.cu) and the fused
// selection + plan kernel (router.cu).
//
// The plan (Basalt: moe_plan, src/models/inkling2/kernels/ops.cu:275-340): the experts that have pairs and a non-zero blob address
// become groups in ascending expert order; an expert's entries keep the order of the pairs (a pair's place = the number of
// earlier pairs naming the same expert, the reference's rule, ops.cu:331-339), so no position comes from an atomic.
// Everything lives in shared memory: the pairs are counted per expert with shared-memory atomics, a block scan over the
// experts gives each used expert its group and first entry.
#pragma once
#include "common.cuh"

namespace bsx {

// a pass of the packed expert kernels: up to kPassEntries consecutive entries [eb, eb + ntok) of one group, with the group's blob
constexpr int kPassEntries = 8;
struct __align__(16) PassRec {
    unsigned long long blob;
    int eb, ntok;
};

// block-wide exclusive sum (blockDim a multiple of 32, at most 1024); *total = the block's sum
__device__ inline int block_excl_sum(int v, int* total, int* sh) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) sh[w] = x;
    __syncthreads();
    if (w == 0) {
        int s = lane < nw ? sh[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(kFull, s, o);
            if (lane >= o) s += y;
        }
        sh[lane] = s;
    }
    __syncthreads();
    const int r = x - v + (w > 0 ? sh[w - 1] : 0);
    *total = sh[nw - 1];
    __syncthreads();
    return r;
}

struct PlanSmem {
    unsigned long long* blob;   // [E]
    int32_t* count;             // [E]
    int32_t* first;             // [E]: the expert's first entry
    int32_t* sid;               // [n]: the pairs' ids (-1: no entry)
};
__host__ __device__ inline size_t plan_smem_bytes(int E, int n) { return (size_t) E * 16 + (size_t) n * 4; }
__device__ inline PlanSmem plan_smem(void* base, int E) {
    PlanSmem s;
    s.blob = static_cast<unsigned long long*>(base);
    s.count = reinterpret_cast<int32_t*>(s.blob + E);
    s.first = s.count + E;
    s.sid = s.first + E;
    return s;
}
// every thread of the block; a block barrier must follow before plan_note_pair
__device__ inline void plan_load_blobs(const PlanSmem& s, const unsigned long long* __restrict__ blobs, int E) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        s.blob[e] = blobs[e];
        s.count[e] = 0;
    }
}
// pair i names expert e (any thread, once per pair); a block barrier must follow before plan_finish
__device__ inline void plan_note_pair(const PlanSmem& s, int i, int e, int E) {
    if ((unsigned) e >= (unsigned) E || !s.blob[e]) e = -1;
    s.sid[i] = e;
    if (e >= 0) atomicAdd(&s.count[e], 1);
}
// every thread of the block.  items / n_items (optional): the pass list of the packed expert kernels, made here so that no
// kernel of its own has to.  tok_base: the first token of the shared expert's group (its entries read tokens tok_base ..
// tok_base + n_tok - 1).  STABLE = false: an expert's entries take their places from a shared-memory cursor instead of by counting
// earlier pairs - for callers to whom the order of the entries inside a group does not matter (every entry writes its own row),
// where the counting loop, quadratic in the pairs, would dominate (thousands of pairs).
template <bool STABLE = true>
__device__ inline void plan_finish(const PlanSmem& s, int n, int k, int E, unsigned long long shared_blob, int n_tok,
                                   unsigned long long* __restrict__ ptr, int32_t* __restrict__ start, int32_t* __restrict__ n_groups,
                                   int32_t* __restrict__ dst, int32_t* __restrict__ tok, PassRec* __restrict__ items, int* __restrict__ n_items,
                                   int tok_base = 0) {
    __shared__ int sh[32];
    int at = 0, g = 0, np_total = 0;   // running totals over the expert chunks of blockDim.x
    for (int e0 = 0; e0 < E; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        const int c = e < E ? s.count[e] : 0;
        int rows = 0, used = 0;
        const int o = block_excl_sum(c, &rows, sh);
        const int u = block_excl_sum(c > 0 ? 1 : 0, &used, sh);
        if (e < E) s.first[e] = at + o;
        if (c > 0) {
            ptr[g + u] = s.blob[e];
            start[g + u] = at + o;
        }
        if (items) {
            const int np = (c + kPassEntries - 1) / kPassEntries;
            int passes = 0;
            const int po = block_excl_sum(np, &passes, sh);
            for (int p = 0; p < np; ++p) {
                PassRec r;
                r.blob = s.blob[e];
                r.eb = at + o + p * kPassEntries;
                r.ntok = min(kPassEntries, c - p * kPassEntries);
                items[np_total + po + p] = r;
            }
            np_total += passes;
        }
        at += rows;
        g += used;
    }
    if (shared_blob != 0ull && n_tok > 0) {
        // the shared expert: one more group holding every token, its rows after the routed pairs' rows
        if (threadIdx.x == 0) {
            ptr[g] = shared_blob;
            start[g] = at;
        }
        for (int t = threadIdx.x; t < n_tok; t += blockDim.x) {
            dst[at + t] = n + t;
            tok[at + t] = tok_base + t;
        }
        if (items) {
            const int np = (n_tok + kPassEntries - 1) / kPassEntries;
            for (int p = threadIdx.x; p < np; p += blockDim.x) {
                PassRec r;
                r.blob = shared_blob;
                r.eb = at + p * kPassEntries;
                r.ntok = min(kPassEntries, n_tok - p * kPassEntries);
                items[np_total + p] = r;
            }
            np_total += np;
        }
        at += n_tok;
        ++g;
    }
    if (threadIdx.x == 0) {
        start[g] = at;
        start[g + 1] = at;
        *n_groups = g;
        if (n_items) n_items[0] = np_total;
    }
    __syncthreads();   // first[] is complete
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = s.sid[i];
        if (e < 0) continue;
        int p;
        if (STABLE) {
            int before = 0;
            int j = 0;
            for (; j + 4 <= i; j += 4) before += (s.sid[j] == e) + (s.sid[j + 1] == e) + (s.sid[j + 2] == e) + (s.sid[j + 3] == e);
            for (; j < i; ++j) before += s.sid[j] == e;
            p = s.first[e] + before;
        } else {
            p = atomicAdd(&s.first[e], 1);
        }
        dst[p] = i;
        tok[p] = i / k;
    }
}

// The same plan for a window of a few tokens, from the pairs alone: every thread owns one pair and counts, over the n pairs in
// shared memory, what the scans over the E experts would have told it - how many entries precede its group, its place inside the
// group (pairs keep their order), whether it is its expert's first pair (the group's leader) and, for leaders, how many groups
// and passes come before theirs.  No table of E entries is read or cleared and the block meets at four barriers; the work is
// n^2 shared-memory reads, which for n <= 512 is less than one scan over the experts.  Groups, entries and passes come out in
// exactly the order of plan_finish (ascending expert, pairs in order).  sid[i]: pair i's expert, or -1 (out of range / not held
// here); blob[i]: that expert's blob address; lead: n ints of scratch.  Every thread of the block calls; blockDim.x >= n.
__device__ inline void plan_small(const int32_t* sid, const unsigned long long* blob, int32_t* lead, int n, int k, unsigned long long shared_blob,
                                  int n_tok, unsigned long long* __restrict__ ptr, int32_t* __restrict__ start, int32_t* __restrict__ n_groups,
                                  int32_t* __restrict__ dst, int32_t* __restrict__ tok, PassRec* __restrict__ items, int* __restrict__ n_items,
                                  int tok_base = 0) {
    __shared__ int s_passes;
    const int i = threadIdx.x;
    const int e = i < n ? sid[i] : -1;
    int less = 0, before = 0, cnt = 0;
    if (e >= 0) {
        for (int j = 0; j < n; ++j) {
            const int sj = sid[j];
            less += (sj >= 0) & (sj < e);
            before += (sj == e) & (j < i);
            cnt += sj == e;
        }
        dst[less + before] = i;
        tok[less + before] = i / k;
    }
    const bool leader = e >= 0 && before == 0;
    if (i < n) lead[i] = leader ? cnt : 0;
    if (i == 0) s_passes = 0;
    const int n_valid = __syncthreads_count(e >= 0);       // also publishes lead[] and s_passes
    const int n_lead = __syncthreads_count(leader);
    if (leader) {
        int g = 0, po = 0;
        for (int j = 0; j < n; ++j) {
            const int c = lead[j];
            if (c > 0 && sid[j] < e) {
                ++g;
                po += (c + kPassEntries - 1) / kPassEntries;
            }
        }
        ptr[g] = blob[i];
        start[g] = less;
        const int np = (cnt + kPassEntries - 1) / kPassEntries;
        if (items) {
            for (int p = 0; p < np; ++p) {
                PassRec r;
                r.blob = blob[i];
                r.eb = less + p * kPassEntries;
                r.ntok = min(kPassEntries, cnt - p * kPassEntries);
                items[po + p] = r;
            }
        }
        atomicAdd(&s_passes, np);
    }
    __syncthreads();
    int at = n_valid, g = n_lead, np_total = s_passes;
    if (shared_blob != 0ull && n_tok > 0) {
        // the shared expert: one more group holding every token, its rows after the routed pairs' rows
        if (i == 0) {
            ptr[g] = shared_blob;
            start[g] = at;
        }
        for (int t = i; t < n_tok; t += blockDim.x) {
            dst[at + t] = n + t;
            tok[at + t] = tok_base + t;
        }
        const int np = (n_tok + kPassEntries - 1) / kPassEntries;
        if (items) {
            for (int p = i; p < np; p += blockDim.x) {
                PassRec r;
                r.blob = shared_blob;
                r.eb = at + p * kPassEntries;
                r.ntok = min(kPassEntries, n_tok - p * kPassEntries);
                items[np_total + p] = r;
            }
        }
        np_total += np;
        at += n_tok;
        ++g;
    }
    if (i == 0) {
        start[g] = at;
        start[g + 1] = at;
        *n_groups = g;
        if (n_items) n_items[0] = np_total;
    }
}

}  // namespace bsx
