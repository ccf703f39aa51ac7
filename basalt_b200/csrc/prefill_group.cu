// prefill_group.cu - the prompt path's experts as the Basalt engine drives them: a group of up to 16 consecutive experts of one
// layer at a time, each given by its blob's address, over rows the caller has already grouped by expert.
//
// Basalt's prompt path walks a layer's experts in groups (fp4::Group / fp4::run_group, include/basalt/prefill/moe_fp4.hpp:82-113;
// call site src/models/qwen4exp/prefill/expert_fp4.cpp:10-30): the host knows each expert's blob address and the row bounds
// live on the device.  bsx_experts_prefill wants a device table of blob addresses and a tile list instead; this entry makes
// both on the device (the addresses ride in as kernel arguments, so there is no host-to-device copy and the call stays
// capturable) and runs the same kernels.  Also here: the small planning kernels of that interface (tile and block offsets of
// row bounds, bounds relative to their first).
#include "common.cuh"

namespace bsx {
namespace {

constexpr int kGroupMax = 16;      // fp4::kMaxExperts

struct BlobList {
    unsigned long long p[kGroupMax];
};

__global__ void group_table_kernel(BlobList b, int n, unsigned long long* __restrict__ table) {
    if ((int) threadIdx.x < n) table[threadIdx.x] = b.p[threadIdx.x];
}

// out[0] = 0, out[j + 1] = sum over i <= j of ceil((bounds[i + 1] - bounds[i]) / unit): the first unit of each segment and
// the total (Basalt: plan_kernel / plan_blocks_kernel, src/prefill/moe_fp4.cu:75-109).  One block of 1024 threads.
__global__ void __launch_bounds__(1024) unit_offsets_kernel(const int32_t* __restrict__ bounds, int n, int unit, int32_t* __restrict__ out) {
    __shared__ int sh[32];
    const int j = threadIdx.x, lane = j & 31, w = j >> 5;
    const int cnt = j < n ? bounds[j + 1] - bounds[j] : 0;
    const int v = cnt > 0 ? (cnt + unit - 1) / unit : 0;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(kFull, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) sh[w] = x;
    __syncthreads();
    if (w == 0) {
        int s = sh[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(kFull, s, o);
            if (lane >= o) s += y;
        }
        sh[lane] = s;
    }
    __syncthreads();
    const int incl = x + (w > 0 ? sh[w - 1] : 0);
    if (j < n) out[j + 1] = incl;
    if (j == 0) out[0] = 0;
}

__global__ void rebase_kernel(const int32_t* __restrict__ bounds, int n, int32_t* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= n) out[i] = bounds[i] - bounds[0];
}

size_t al256g(size_t v) { return (v + 255) & ~(size_t) 255; }

}  // namespace
}  // namespace bsx

using namespace bsx;

extern "C" int32_t bsx_unit_offsets(const int32_t* bounds, int32_t n, int32_t unit_rows, int32_t* out, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (n < 1 || n > 1024 || unit_rows < 1) return BSX_E_GEOMETRY;
    if (!bounds || !out) return BSX_E_POINTER;
    unit_offsets_kernel<<<1, 1024, 0, (cudaStream_t) stream>>>(bounds, n, unit_rows, out);
    return launch_status();
}

extern "C" int32_t bsx_rebase_bounds(const int32_t* bounds, int32_t n, int32_t* out, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (n < 0) return BSX_E_GEOMETRY;
    if (!bounds || !out) return BSX_E_POINTER;
    rebase_kernel<<<(unsigned) (n / 256 + 1), 256, 0, (cudaStream_t) stream>>>(bounds, n, out);
    return launch_status();
}

extern "C" size_t bsx_experts_prefill_group_scratch_bytes(const bsx_expert_layout* L, int64_t n_tokens, int64_t cap_rows) {
    const size_t inner = bsx_experts_prefill_scratch_bytes(L, n_tokens, cap_rows);
    if (!inner) return 0;
    return al256g(kGroupMax * 8) + al256g((size_t) (cap_rows / 128 + kGroupMax) * 8) + 256 + inner;
}

extern "C" int32_t bsx_experts_prefill_group(const bsx_expert_layout* layout, const void* const* blobs, int32_t n, const int32_t* bounds,
                                             const int32_t* row_token, int64_t cap_rows, const void* x, int32_t x_kind, int64_t n_tokens,
                                             void* scratch, float* dm, int32_t* status, void* stream) {
    if (!stream) return BSX_E_STREAM;
    if (n < 1 || n > kGroupMax || cap_rows < 0 || n_tokens < 0) return BSX_E_GEOMETRY;
    if (!layout || !blobs || !bounds || !row_token || !aligned(scratch, 256) || !dm || !status) return BSX_E_POINTER;
    BlobList bl;
    for (int i = 0; i < kGroupMax; ++i) bl.p[i] = i < n ? (unsigned long long) (uintptr_t) blobs[i] : 0ull;
    uint8_t* p = static_cast<uint8_t*>(scratch);
    unsigned long long* table = reinterpret_cast<unsigned long long*>(p);
    p += al256g(kGroupMax * 8);
    int32_t* tiles = reinterpret_cast<int32_t*>(p);
    const int64_t cap_tiles = cap_rows / 128 + kGroupMax;
    p += al256g((size_t) cap_tiles * 8);
    int32_t* n_tiles = reinterpret_cast<int32_t*>(p);
    p += 256;
    const cudaStream_t st = (cudaStream_t) stream;
    group_table_kernel<<<1, 32, 0, st>>>(bl, n, table);
    int32_t rc = launch_status();
    if (rc != BSX_OK) return rc;
    rc = bsx_tiles_from_bounds(bounds, n, 128, tiles, n_tiles, stream);
    if (rc != BSX_OK) return rc;
    // rows are absolute: bounds[j] is expert j's first row in dm and in row_token, exactly what the tile list carries
    return bsx_experts_prefill(layout, table, bounds, row_token, tiles, n_tiles, cap_tiles, cap_rows, x, x_kind, n_tokens, p, dm, status, stream);
}
